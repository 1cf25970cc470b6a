"""Writes tests/golden/moe_golden.npz: oracle outputs for a few small seeded cases.

The reference (Swift + Metal) cannot run where this repository is built, so the stored vectors come
from the C oracle (which is itself pinned to the reference's known-answer tests by
tests/test_oracle_golden.py).  They freeze the oracle: a later change to the oracle, to the synthetic
weight generator or to the bit-exact routing arithmetic shows up as a difference against this file.

    python tests/golden/make_golden.py          # rewrites the file
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from ffai_b200 import synth  # noqa: E402


def cases():
    """name -> (spec, tokens, seed, with_residual)"""
    return {
        "cfg1_tiny_t16": (synth.cfg1_tiny(), 16, 0, False),
        "gptoss_small_t5": (synth.cfg2_gptoss().with_(hidden=256, intermediate=256, n_experts=8, name="gptoss_small",
                                                      expert_row_bias=1), 5, 1, True),
        "qwen_small_shared_t9": (synth.cfg4_shared().with_(hidden=256, intermediate=128, n_experts=16, top_k=4,
                                                           shared_intermediate=128, name="qwen_small"), 9, 2, False),
        "gemma_small_t7": (synth.gemma4_style().with_(hidden=256, intermediate=128, n_experts=8, top_k=2, name="gemma_small"), 7, 3, False),
        "six_bit_t6": (synth.LayerSpec("six_bit", 256, 128, 8, 2, expert_bits=6), 6, 4, False),
    }


def mxfp4_case():
    rng = np.random.default_rng(77)
    packed = rng.integers(0, 256, size=(64, 16), dtype=np.uint8)
    packed[:8] &= 0x33
    packed[8:12] = 0x80
    e8m0 = rng.integers(110, 135, size=64, dtype=np.uint8)
    return packed, e8m0


def quant_case():
    rng = np.random.default_rng(78)
    return synth.f32_to_bf16((rng.standard_normal((8, 128)) * rng.uniform(0.05, 3.0, size=(8, 1))).astype(np.float32))


def build():
    out = {}
    for name, (spec, T, seed, with_res) in cases().items():
        host = synth.make_layer(spec, seed)
        x = synth.make_tokens(T, spec.hidden, seed)
        res = synth.make_tokens(T, spec.hidden, seed + 17) if with_res else None
        xr = synth.make_tokens(T, spec.hidden, seed + 40) if spec.name.startswith("gemma") else None
        r = oracle.moe_forward(host, x, residual=res, x_router=xr)
        out[f"{name}/indices"] = r.indices
        out[f"{name}/weights"] = r.weights
        out[f"{name}/logits"] = r.logits
        out[f"{name}/perm"] = r.perm
        out[f"{name}/offsets"] = r.offsets
        out[f"{name}/out_bf16"] = r.out_bf16
        out[f"{name}/out_f32"] = r.out_f32
    packed, e8m0 = mxfp4_case()
    w, s, b = oracle.mxfp4_to_affine4(packed, e8m0)
    out["mxfp4/codes"], out["mxfp4/scales"], out["mxfp4/biases"] = w, s, b
    wq = quant_case()
    for bits in (3, 4, 8):
        p, s, b = oracle.affine_quantize(wq, bits, 64)
        out[f"quant{bits}/codes"], out[f"quant{bits}/scales"], out[f"quant{bits}/biases"] = p, s, b
    return out


if __name__ == "__main__":
    np.savez_compressed(os.path.join(HERE, "moe_golden.npz"), **build())
    print("wrote", os.path.join(HERE, "moe_golden.npz"))
