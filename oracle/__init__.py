"""ctypes wrapper of the CPU oracle (``oracle/moe_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Imported by ``tests/``, by the smoke check and by the CPU-baseline leg of the
benchmark — never by the package ``ffai_b200`` and never on a product path.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

from ffai_b200 import capi

ORACLE_DIR = Path(__file__).resolve().parent
LIB = ORACLE_DIR / "_build" / "libmoe_oracle.so"

_lib = None


def build(force: bool = False) -> Path:
    src = ORACLE_DIR / "moe_oracle.c"
    hdr = ORACLE_DIR.parent / "include" / "ffai_cuda.h"
    if force or not LIB.exists() or LIB.stat().st_mtime < max(src.stat().st_mtime, hdr.stat().st_mtime):
        subprocess.run(["make", "-C", str(ORACLE_DIR), "-B"], check=True, capture_output=True)
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB.exists():
            build()
        L = C.CDLL(str(LIB))
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_expf.restype = C.c_float
        L.orc_expf.argtypes = [C.c_float]
        L.orc_unpack.restype = C.c_uint32
        L.orc_unpack.argtypes = [C.c_void_p, C.c_int, C.c_int64]
        L.orc_glu.restype = C.c_float
        L.orc_glu.argtypes = [C.c_float, C.c_float, C.c_int, C.c_float, C.c_float]
        L.orc_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def route(logits, k, gating_mode, norm_topk_prob, expert_bias=None, routed_scaling=1.0):
    """MoERouter.route on one logits vector → (indices int32[k], weights float32[k])."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    idx = np.zeros(k, dtype=np.int32)
    w = np.zeros(k, dtype=np.float32)
    eb = None if expert_bias is None else np.ascontiguousarray(expert_bias, dtype=np.float32)
    lib().orc_route_scaled(_p(logits), C.c_int(len(logits)), C.c_int(k), C.c_int(gating_mode),
                           C.c_int(norm_topk_prob), _p(eb), C.c_float(routed_scaling), _p(idx), _p(w))
    return idx, w


def pack(q, bits):
    q = np.ascontiguousarray(q, dtype=np.uint32)
    out = np.zeros(q.size * bits // 32, dtype=np.uint32)
    lib().orc_pack(_p(q), C.c_int64(q.size), C.c_int(bits), _p(out))
    return out


def unpack(words, bits, n):
    words = np.ascontiguousarray(words, dtype=np.uint32)
    L = lib()
    return np.array([L.orc_unpack(words.ctypes.data, bits, i) for i in range(n)], dtype=np.uint32)


def dequant_gemv(x, weight, scales, biases, out_dim, in_dim, bits, gs):
    x = np.ascontiguousarray(x, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    biases = np.ascontiguousarray(biases, dtype=np.uint16)
    out = np.zeros(out_dim, dtype=np.float32)
    lib().orc_dequant_gemv(_p(x), _p(weight), _p(scales), _p(biases), _p(out), C.c_int(out_dim),
                           C.c_int(in_dim), C.c_int(bits), C.c_int(gs))
    return out


def gather_dequant_gemm(x, weight, scales, biases, indices, m_total, n_out, k_in, n_experts, bits, gs):
    x = np.ascontiguousarray(x, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    biases = np.ascontiguousarray(biases, dtype=np.uint16)
    indices = np.ascontiguousarray(indices, dtype=np.uint32)
    out = np.zeros((m_total, n_out), dtype=np.float32)
    lib().orc_gather_dequant_gemm(_p(x), _p(weight), _p(scales), _p(biases), _p(indices), _p(out),
                                  C.c_int(m_total), C.c_int(n_out), C.c_int(k_in),
                                  C.c_int(n_experts), C.c_int(bits), C.c_int(gs))
    return out


def plan(indices, n_tokens, k, n_experts):
    indices = np.ascontiguousarray(indices, dtype=np.uint32).reshape(-1)
    counts = np.zeros(n_experts, dtype=np.uint32)
    offsets = np.zeros(n_experts + 1, dtype=np.uint32)
    perm = np.zeros(n_tokens * k, dtype=np.uint32)
    inv = np.zeros(n_tokens * k, dtype=np.uint32)
    lib().orc_plan(_p(indices), C.c_int(n_tokens), C.c_int(k), C.c_int(n_experts), _p(counts),
                   _p(offsets), _p(perm), _p(inv))
    return counts, offsets, perm, inv


def unpermute(expert_out, inv_perm, weights, n_tokens, hidden, k):
    expert_out = np.ascontiguousarray(expert_out, dtype=np.float32)
    inv_perm = np.ascontiguousarray(inv_perm, dtype=np.uint32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    out = np.zeros((n_tokens, hidden), dtype=np.float32)
    lib().orc_unpermute(_p(expert_out), _p(inv_perm), _p(weights), _p(out), C.c_int(n_tokens),
                        C.c_int(hidden), C.c_int(k))
    return out


def mxfp4_to_affine4(packed_bytes, e8m0):
    """MXFP4 codes [n_groups, 16] u8 + scale bytes [n_groups] -> (packed u8 [n_groups,16], scales, biases bf16)."""
    packed_bytes = np.ascontiguousarray(packed_bytes, dtype=np.uint8)
    e8m0 = np.ascontiguousarray(e8m0, dtype=np.uint8)
    n = int(e8m0.size)
    out = np.zeros((n, 16), dtype=np.uint8)
    sc = np.zeros(n, dtype=np.uint16)
    bi = np.zeros(n, dtype=np.uint16)
    lib().orc_mxfp4_to_affine4(_p(packed_bytes), _p(e8m0), C.c_int64(n), _p(out), _p(sc), _p(bi))
    return out, sc, bi


def affine_quantize(w_bf16, bits, gs):
    """[rows, K] bf16 bit patterns -> (packed u32 [rows, K*bits/32], scales, biases bf16 [rows, K/gs])."""
    w_bf16 = np.ascontiguousarray(w_bf16, dtype=np.uint16)
    rows, K = w_bf16.shape
    out = np.zeros((rows, K * bits // 32), dtype=np.uint32)
    sc = np.zeros((rows, K // gs), dtype=np.uint16)
    bi = np.zeros((rows, K // gs), dtype=np.uint16)
    lib().orc_affine_quantize(_p(w_bf16), C.c_int64(rows), C.c_int(K), C.c_int(bits), C.c_int(gs), _p(out), _p(sc), _p(bi))
    return out, sc, bi


def add_rmsnorm(a, b, weight, eps):
    """bf16 bit patterns [rows, n], [rows, n] or None (plain RMSNorm), [n] -> (residual bf16, normed bf16, normed f32)."""
    a = np.ascontiguousarray(a, dtype=np.uint16)
    b = None if b is None else np.ascontiguousarray(b, dtype=np.uint16)
    weight = np.ascontiguousarray(weight, dtype=np.uint16)
    rows, n = a.shape
    res = np.zeros((rows, n), dtype=np.uint16)
    nrm = np.zeros((rows, n), dtype=np.uint16)
    nf = np.zeros((rows, n), dtype=np.float32)
    lib().orc_add_rmsnorm(_p(a), _p(b) if b is not None else None, _p(weight), C.c_float(eps), C.c_int(rows), C.c_int(n), _p(res), _p(nrm), _p(nf))
    return res, nrm, nf


def router_logits(host_layer, x):
    """Router logits [T, E] in the oracle's fixed accumulation order."""
    spec = host_layer.spec
    cfg = spec.to_config(max_tokens=x.shape[0])
    w = host_layer.weights_struct()
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.zeros((x.shape[0], spec.n_experts), dtype=np.float32)
    lib().orc_router_logits(C.byref(cfg), C.byref(w.router), _p(x), C.c_int(x.shape[0]), _p(out))
    return out


class Result:
    __slots__ = ("out_f32", "out_bf16", "indices", "weights", "logits", "counts", "offsets", "perm",
                 "inv_perm")


def moe_forward(host_layer, x, residual=None, token_mask=None, round_stages=False, n_threads=0,
                compute_output=True, x_router=None) -> Result:
    """The whole block on the CPU.  `x`: uint16 bf16 bit patterns [T, H]."""
    spec = host_layer.spec
    T = int(x.shape[0])
    H, E, K = spec.hidden, spec.n_experts, spec.top_k
    cfg = spec.to_config(max_tokens=T)
    w = host_layer.weights_struct()
    x = np.ascontiguousarray(x, dtype=np.uint16)
    r = Result()
    r.out_f32 = np.zeros((T, H), dtype=np.float32) if compute_output else None
    r.out_bf16 = np.zeros((T, H), dtype=np.uint16) if compute_output else None
    r.indices = np.zeros((T, K), dtype=np.uint32)
    r.weights = np.zeros((T, K), dtype=np.float32)
    r.logits = np.zeros((T, E), dtype=np.float32)
    r.counts = np.zeros(E, dtype=np.uint32)
    r.offsets = np.zeros(E + 1, dtype=np.uint32)
    r.perm = np.zeros(T * K, dtype=np.uint32)
    r.inv_perm = np.zeros(T * K, dtype=np.uint32)
    dbg = capi.MoEDebug(r.indices.ctypes.data, r.weights.ctypes.data, r.logits.ctypes.data,
                        r.counts.ctypes.data, r.offsets.ctypes.data, r.perm.ctypes.data,
                        r.inv_perm.ctypes.data)
    res = None if residual is None else np.ascontiguousarray(residual, dtype=np.uint16)
    mask = None if token_mask is None else np.ascontiguousarray(token_mask, dtype=np.uint8)
    xr = None if x_router is None else np.ascontiguousarray(x_router, dtype=np.uint16)
    rc = lib().orc_moe_forward_split(C.byref(cfg), C.byref(w), _p(x), _p(xr), C.c_int(T), _p(r.out_f32),
                               _p(r.out_bf16), _p(res), C.byref(dbg), _p(mask),
                               C.c_int(1 if round_stages else 0), C.c_int(n_threads))
    if rc != 0:
        raise RuntimeError(f"orc_moe_forward failed: {rc}")
    return r
