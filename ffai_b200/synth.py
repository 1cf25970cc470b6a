"""Seeded synthetic MoE layers in the MLX affine-quantized layout.

The benchmark configurations name shapes and value distributions, not data, so
weights and activations are drawn here from one counter-based generator
(Philox, seed given by the caller).  The same host arrays feed both the CUDA
library and the CPU oracle, so no tensors are shipped.

Layouts follow FFAI's stacked expert tensors
(``Sources/FFAI/Models/MoELayer.swift:347-391``): ``weight[E, out, in*bits/32]``
uint32, ``scales/biases[E, out, in/group]`` bf16.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field, replace
from typing import Dict, Optional

import numpy as np

from . import capi


# ───────────────────────── bf16 and bit packing (numpy) ─────────────────────────

def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even on the bit pattern (FFAI ``Tensor.swift:145-150``)."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def pack_bits(q: np.ndarray, bits: int) -> np.ndarray:
    """Pack ``q[..., n]`` (values < 2**bits) into the LSB-first bit stream of
    ``n*bits/32`` little-endian uint32 words per row."""
    n = q.shape[-1]
    assert (n * bits) % 32 == 0 and n % 32 == 0
    lead = q.shape[:-1]
    v = q.reshape(-1, n // 32, 32).astype(np.uint64) & np.uint64((1 << bits) - 1)
    out = np.zeros((v.shape[0], n // 32, bits + 1), dtype=np.uint64)
    for j in range(32):
        bit = j * bits
        wi, sh = bit >> 5, bit & 31
        shifted = v[:, :, j] << np.uint64(sh)
        out[:, :, wi] |= shifted & np.uint64(0xFFFFFFFF)
        if sh + bits > 32:
            out[:, :, wi + 1] |= shifted >> np.uint64(32)
    return out[:, :, :bits].astype(np.uint32).reshape(*lead, n * bits // 32)


def unpack_bits(words: np.ndarray, bits: int, n: int) -> np.ndarray:
    """Inverse of :func:`pack_bits`."""
    lead = words.shape[:-1]
    w = words.reshape(-1, n // 32, bits).astype(np.uint64)
    w = np.concatenate([w, np.zeros_like(w[:, :, :1])], axis=2)
    out = np.empty((w.shape[0], n // 32, 32), dtype=np.uint32)
    mask = np.uint64((1 << bits) - 1)
    for j in range(32):
        bit = j * bits
        wi, sh = bit >> 5, bit & 31
        v = w[:, :, wi] >> np.uint64(sh)
        if sh + bits > 32:
            v = v | (w[:, :, wi + 1] << np.uint64(32 - sh))
        out[:, :, j] = (v & mask).astype(np.uint32)
    return out.reshape(*lead, n)


def dequantize(words: np.ndarray, scales: np.ndarray, biases: np.ndarray, bits: int, gs: int,
               n: int) -> np.ndarray:
    q = unpack_bits(words, bits, n).astype(np.float32)
    s = np.repeat(bf16_to_f32(scales), gs, axis=-1)
    b = np.repeat(bf16_to_f32(biases), gs, axis=-1)
    return s * q + b


def quantize_minmax(w: np.ndarray, bits: int, gs: int):
    """Group min/max affine quantisation: ``scale=(max-min)/(2^b-1)``, ``bias=min``,
    ``q=round((w-bias)/scale)`` clamped — the rule of the reference's CPU transcode
    (``Sources/FFAI/Models/Text/GPTOSSText.swift:1176-1219``).  Scale and bias are
    rounded to bf16 before ``q`` is computed."""
    lead, n = w.shape[:-1], w.shape[-1]
    g = w.reshape(*lead, n // gs, gs).astype(np.float32)
    lo, hi = g.min(axis=-1), g.max(axis=-1)
    levels = float((1 << bits) - 1)
    scale = bf16_to_f32(f32_to_bf16(np.maximum((hi - lo) / levels, 1e-8)))
    bias = bf16_to_f32(f32_to_bf16(lo))
    q = np.rint((g - bias[..., None]) / scale[..., None])
    q = np.clip(q, 0, levels).astype(np.uint32).reshape(*lead, n)
    return pack_bits(q, bits), f32_to_bf16(scale), f32_to_bf16(bias)


# ───────────────────────── layer description ─────────────────────────

@dataclass(frozen=True)
class LayerSpec:
    name: str
    hidden: int
    intermediate: int
    n_experts: int
    top_k: int
    gating_mode: int = capi.GATING_SOFTMAX_THEN_TOPK
    norm_topk_prob: int = 1
    router_expert_bias: int = 0
    activation: int = capi.ACT_SWIGLU
    swiglu_limit: float = 7.0
    swiglu_alpha: float = 1.702
    router_kind: int = capi.LINEAR_BF16
    router_bits: int = 0
    router_group_size: int = 0
    router_has_bias: int = 0
    router_logits_bf16: int = 1
    expert_bits: int = 4
    expert_group_size: int = 64
    expert_row_bias: int = 0
    shared_intermediate: int = 0
    shared_bits: int = 0
    shared_group_size: int = 0
    shared_gate_kind: int = capi.LINEAR_NONE
    shared_gate_bits: int = 0
    shared_gate_group_size: int = 0
    router_logit_scale: float = 0.0     # logits are multiplied by this before routing (0: no scaling)
    router_per_expert_scale: int = 0    # 1: a per-expert factor on the combine weights (Gemma 4)
    routed_scaling_factor: float = 0.0  # sigmoid routing: factor on the combine weights (0: none)
    prefill_weight_cache: int = 0  # 0 automatic, 1 never, 2 always (bf16 copy of the experts for the tensor-core path)
    zipf_s: float = 0.0          # > 0: additive per-expert router bias with a Zipf profile
    zipf_strength: float = 1.0

    def with_(self, **kw) -> "LayerSpec":
        return replace(self, **kw)

    def to_config(self, max_tokens: int, ep_rank: int = 0, ep_world: int = 1) -> capi.MoEConfig:
        cfg = capi.MoEConfig()
        for f in ("hidden", "intermediate", "n_experts", "top_k", "gating_mode", "norm_topk_prob",
                  "router_expert_bias", "activation", "swiglu_limit", "swiglu_alpha", "router_kind",
                  "router_bits", "router_group_size", "router_has_bias", "router_logits_bf16",
                  "expert_bits", "expert_group_size", "expert_row_bias", "shared_intermediate",
                  "shared_bits", "shared_group_size", "shared_gate_kind", "shared_gate_bits",
                  "shared_gate_group_size", "prefill_weight_cache", "router_logit_scale", "routed_scaling_factor"):
            setattr(cfg, f, getattr(self, f))
        cfg.max_tokens = max_tokens
        cfg.ep_rank = ep_rank
        cfg.ep_world = ep_world
        return cfg

    # algorithmic work, as defined for the roofline figures
    def bytes_per_weight(self, bits=None, gs=None) -> float:
        bits = bits or self.expert_bits
        gs = gs or self.expert_group_size
        return bits / 8.0 + 4.0 / gs

    def bytes_per_expert(self) -> float:
        return 3.0 * self.hidden * self.intermediate * self.bytes_per_weight()

    def router_bytes(self) -> float:
        per = {capi.LINEAR_F32: 4.0, capi.LINEAR_BF16: 2.0}.get(self.router_kind)
        if per is None:
            per = self.bytes_per_weight(self.router_bits, self.router_group_size)
        return self.n_experts * self.hidden * per

    def decode_bytes(self, n_tokens: int, distinct_experts: int) -> float:
        return (distinct_experts * self.bytes_per_expert() + self.router_bytes()
                + 2.0 * n_tokens * self.hidden * 2.0)

    def prefill_flops(self, n_tokens: int) -> Dict[str, float]:
        routed = 2.0 * n_tokens * self.top_k * 3.0 * self.hidden * self.intermediate
        shared = 2.0 * n_tokens * 3.0 * self.hidden * self.shared_intermediate
        router = 2.0 * n_tokens * self.hidden * self.n_experts
        return {"routed": routed, "shared": shared, "router": router}


def cfg1_tiny() -> LayerSpec:
    """Tiny layer: T=16, H=512, E=8, k=2, I=1024, fp32 router, softmax→top-2 renormalised."""
    return LayerSpec("cfg1_tiny", 512, 1024, 8, 2, router_kind=capi.LINEAR_F32, router_logits_bf16=0)


def cfg2_gptoss() -> LayerSpec:
    """GPT-OSS-20B-shaped decode layer: H=I=2880, E=32, k=4, biased bf16 router,
    top-4 then softmax, clamped SwiGLU."""
    return LayerSpec("cfg2_gptoss20b", 2880, 2880, 32, 4, gating_mode=capi.GATING_TOPK_THEN_SOFTMAX,
                     activation=capi.ACT_CLAMPED_SWIGLU, router_has_bias=1)


def cfg3_qwen() -> LayerSpec:
    """Qwen3-30B-A3B-shaped prefill layer: H=2048, E=128, k=8, I=768."""
    return LayerSpec("cfg3_qwen3_30b_a3b", 2048, 768, 128, 8)


def cfg4_shared() -> LayerSpec:
    """256-expert layer with a sigmoid-gated shared expert; router/shared/gate 8-bit."""
    return LayerSpec("cfg4_256e_shared", 2048, 512, 256, 8, router_kind=capi.LINEAR_AFFINE,
                     router_bits=8, router_group_size=64, shared_intermediate=512, shared_bits=8,
                     shared_group_size=64, shared_gate_kind=capi.LINEAR_AFFINE, shared_gate_bits=8,
                     shared_gate_group_size=64)


def cfg5_skewed(bits: int) -> LayerSpec:
    """cfg3 shape with a Zipf(1.1) additive router bias and experts at `bits` bits."""
    return cfg3_qwen().with_(name=f"cfg5_skewed_{bits}bit", expert_bits=bits, router_has_bias=1,
                             zipf_s=1.1)


def nemotronh_style() -> LayerSpec:
    """NemotronH-style block: sigmoid routing with a selection bias and a routed scaling factor, experts
    without a gate projection (relu(up)^2), an always-on shared expert of the same form
    (NemotronHText.swift:696-912)."""
    return LayerSpec("nemotronh_style", 512, 256, 16, 4, gating_mode=capi.GATING_SIGMOID_TOPK, router_expert_bias=1,
                     activation=capi.ACT_RELU2, routed_scaling_factor=2.5, shared_intermediate=384,
                     shared_bits=4, shared_group_size=64)


def gemma4_style() -> LayerSpec:
    """Gemma-4-style block: top-k then softmax, logits scaled by hidden^-0.5, per-expert combine scale,
    GELU-GLU experts (Gemma4Text.swift:928-980); the router reads its own normalised input."""
    return LayerSpec("gemma4_style", 1024, 512, 32, 4, gating_mode=capi.GATING_TOPK_THEN_SOFTMAX,
                     activation=capi.ACT_GELU_GLU, router_logit_scale=1024 ** -0.5, router_per_expert_scale=1)


CONFIGS = {"cfg1": cfg1_tiny, "cfg2": cfg2_gptoss, "cfg3": cfg3_qwen, "cfg4": cfg4_shared}


# ───────────────────────── weight generation ─────────────────────────

@dataclass
class HostLayer:
    """Host arrays of one layer plus the ctypes structs that point at them."""
    spec: LayerSpec
    arrays: Dict[str, np.ndarray] = field(default_factory=dict)

    def weights_struct(self, ep_rank: int = 0, ep_world: int = 1) -> capi.MoEWeights:
        """Host-pointer ``ffai_moe_weights``.  Under expert parallelism the expert
        stacks are sliced to this rank's contiguous block of ``E/ep_world`` experts."""
        a, s = self.arrays, self.spec
        w = capi.MoEWeights()
        w.location = capi.MEM_HOST
        keep = []

        def ptr(arr: Optional[np.ndarray]):
            if arr is None:
                return None
            arr = np.ascontiguousarray(arr)
            keep.append(arr)
            return arr.ctypes.data

        def lin(prefix: str) -> capi.Linear:
            return capi.Linear(ptr(a.get(prefix + ".weight")), ptr(a.get(prefix + ".scales")),
                               ptr(a.get(prefix + ".biases")), ptr(a.get(prefix + ".bias")))

        def qproj(prefix: str, shard: bool) -> capi.QProj:
            def sl(arr):
                if arr is None or not shard or ep_world <= 1:
                    return arr
                per = s.n_experts // ep_world
                return arr[ep_rank * per:(ep_rank + 1) * per]
            return capi.QProj(ptr(sl(a.get(prefix + ".weight"))), ptr(sl(a.get(prefix + ".scales"))),
                              ptr(sl(a.get(prefix + ".biases"))), ptr(sl(a.get(prefix + ".row_bias"))))

        w.router = lin("gate")
        w.router_expert_bias = ptr(a.get("gate.expert_bias"))
        w.router_per_expert_scale = ptr(a.get("gate.per_expert_scale"))
        w.gate_proj = qproj("experts.gate_proj", True)
        w.up_proj = qproj("experts.up_proj", True)
        w.down_proj = qproj("experts.down_proj", True)
        if s.shared_intermediate:
            w.shared_gate_proj = qproj("shared_expert.gate_proj", False)
            w.shared_up_proj = qproj("shared_expert.up_proj", False)
            w.shared_down_proj = qproj("shared_expert.down_proj", False)
            w.shared_gate = lin("shared_expert_gate")
        w._keep = keep  # keep the arrays alive as long as the struct
        return w

    def weight_bytes(self) -> int:
        return int(sum(v.nbytes for v in self.arrays.values()))


def _rand_qproj(rng, n: int, out_dim: int, in_dim: int, bits: int, gs: int, row_bias: bool,
                prefix: str, arrays: Dict[str, np.ndarray]) -> None:
    """q ~ U{0..2^b-1}; scale ~ U(0.005,0.02)*15/(2^b-1) so dequantised magnitudes match
    the 4-bit case at every width; bias ~ U(-0.1,0.1); both bf16."""
    words = in_dim * bits // 32
    if bits in (4, 8):
        # uniform random words are uniform random nibbles / bytes
        packed = rng.integers(0, 1 << 32, size=(n, out_dim, words), dtype=np.uint64).astype(np.uint32)
    else:
        q = rng.integers(0, 1 << bits, size=(n, out_dim, in_dim), dtype=np.uint32)
        packed = pack_bits(q, bits)
    g = in_dim // gs
    scale = (0.005 + 0.015 * rng.random((n, out_dim, g), dtype=np.float32)) * np.float32(15.0 / ((1 << bits) - 1))
    bias = -0.1 + 0.2 * rng.random((n, out_dim, g), dtype=np.float32)
    arrays[prefix + ".weight"] = packed
    arrays[prefix + ".scales"] = f32_to_bf16(scale)
    arrays[prefix + ".biases"] = f32_to_bf16(bias)
    if row_bias:
        arrays[prefix + ".row_bias"] = f32_to_bf16(0.1 * rng.standard_normal((n, out_dim), dtype=np.float32))


def _rand_linear(rng, out_dim: int, in_dim: int, kind: int, bits: int, gs: int, prefix: str,
                 arrays: Dict[str, np.ndarray], std: float = 0.02) -> None:
    w = (std * rng.standard_normal((out_dim, in_dim), dtype=np.float32)).astype(np.float32)
    if kind == capi.LINEAR_F32:
        arrays[prefix + ".weight"] = w
    elif kind == capi.LINEAR_BF16:
        arrays[prefix + ".weight"] = f32_to_bf16(w)
    elif kind == capi.LINEAR_AFFINE:
        p, s, b = quantize_minmax(w, bits, gs)
        arrays[prefix + ".weight"], arrays[prefix + ".scales"], arrays[prefix + ".biases"] = p, s, b


def zipf_router_bias(n_experts: int, s: float, strength: float) -> np.ndarray:
    """Additive logit bias ``strength * log(p_e / mean p)`` with ``p_e ∝ (e+1)^-s``."""
    p = 1.0 / np.power(np.arange(1, n_experts + 1, dtype=np.float64), s)
    p /= p.sum()
    return (strength * np.log(p * n_experts)).astype(np.float32)


def make_layer(spec: LayerSpec, seed: int = 0) -> HostLayer:
    rng = np.random.Generator(np.random.Philox(seed))
    a: Dict[str, np.ndarray] = {}
    H, I, E = spec.hidden, spec.intermediate, spec.n_experts
    _rand_linear(rng, E, H, spec.router_kind, spec.router_bits, spec.router_group_size, "gate", a)
    if spec.router_has_bias:
        if spec.zipf_s > 0:
            bias = zipf_router_bias(E, spec.zipf_s, spec.zipf_strength)
        else:
            bias = 0.05 * rng.standard_normal(E, dtype=np.float32)
        a["gate.bias"] = f32_to_bf16(bias)
    if spec.router_expert_bias:
        a["gate.expert_bias"] = (0.02 * rng.standard_normal(E, dtype=np.float32)).astype(np.float32)
    no_gate = spec.activation == capi.ACT_RELU2     # experts without a gate projection: the array is not made at all
    if not no_gate:
        _rand_qproj(rng, E, I, H, spec.expert_bits, spec.expert_group_size, bool(spec.expert_row_bias),
                    "experts.gate_proj", a)
    _rand_qproj(rng, E, I, H, spec.expert_bits, spec.expert_group_size, bool(spec.expert_row_bias),
                "experts.up_proj", a)
    _rand_qproj(rng, E, H, I, spec.expert_bits, spec.expert_group_size, bool(spec.expert_row_bias),
                "experts.down_proj", a)
    if spec.shared_intermediate:
        Is = spec.shared_intermediate
        if not no_gate:
            _rand_qproj(rng, 1, Is, H, spec.shared_bits, spec.shared_group_size, False, "shared_expert.gate_proj", a)
        _rand_qproj(rng, 1, Is, H, spec.shared_bits, spec.shared_group_size, False, "shared_expert.up_proj", a)
        _rand_qproj(rng, 1, H, Is, spec.shared_bits, spec.shared_group_size, False, "shared_expert.down_proj", a)
        if spec.shared_gate_kind != capi.LINEAR_NONE:
            _rand_linear(rng, 1, H, spec.shared_gate_kind, spec.shared_gate_bits,
                         spec.shared_gate_group_size, "shared_expert_gate", a)
    if spec.router_per_expert_scale:   # drawn last so that every other array of a seed stays as it was
        a["gate.per_expert_scale"] = (0.5 + rng.random(E, dtype=np.float32)).astype(np.float32)
    return HostLayer(spec, a)


def requantize_experts(layer: HostLayer, bits: int) -> HostLayer:
    """Re-quantise the expert stacks of `layer` at `bits` bits from their dequantised fp32
    values (the bit-width sweep of the skewed-routing configuration)."""
    s = layer.spec
    a = dict(layer.arrays)
    for proj, in_dim in (("gate_proj", s.hidden), ("up_proj", s.hidden), ("down_proj", s.intermediate)):
        p = "experts." + proj
        ws, ss, bs = [], [], []
        for e in range(s.n_experts):
            w = dequantize(a[p + ".weight"][e], a[p + ".scales"][e], a[p + ".biases"][e],
                           s.expert_bits, s.expert_group_size, in_dim)
            pw, sc, bi = quantize_minmax(w, bits, s.expert_group_size)
            ws.append(pw); ss.append(sc); bs.append(bi)
        a[p + ".weight"], a[p + ".scales"], a[p + ".biases"] = np.stack(ws), np.stack(ss), np.stack(bs)
    return HostLayer(s.with_(expert_bits=bits, name=f"{s.name}_rq{bits}"), a)


def make_tokens(n_tokens: int, hidden: int, seed: int = 0) -> np.ndarray:
    """bf16 activations ~ N(0,1), as uint16 bit patterns [T, H]."""
    rng = np.random.Generator(np.random.Philox(seed + 1_000_003))
    return f32_to_bf16(rng.standard_normal((n_tokens, hidden), dtype=np.float32))
