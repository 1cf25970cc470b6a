"""Parity metrics and small device-memory helpers shared by the tests."""
from __future__ import annotations

import numpy as np

from ffai_b200 import synth

# Output tolerances of the block (bf16 result against the fp32-accumulated oracle):
#   relative RMS error <= 5e-3, and max-abs error <= 2e-2 measured per element in units of
#   max(|oracle value|, RMS of the oracle output).  The raw max-abs figure cannot be gated
#   at 2e-2: at the benchmark's value distributions outputs are O(100..1000), where one
#   bf16 ulp is 1..8, so merely rounding the exact answer to bf16 exceeds it.  Raw,
#   RMS-normalised and per-element figures are all reported.
REL_RMS_TOL = 5e-3
MAX_ABS_NORM_TOL = 2e-2


def parity(got_bf16_bits: np.ndarray, ref_f32: np.ndarray):
    got = synth.bf16_to_f32(got_bf16_bits).astype(np.float64).reshape(ref_f32.shape)
    ref = ref_f32.astype(np.float64)
    rms = float(np.sqrt(np.mean(ref ** 2))) or 1.0
    err = got - ref
    return {
        "rel_rms": float(np.sqrt(np.mean(err ** 2))) / rms,
        "max_abs": float(np.max(np.abs(err))),
        "max_abs_over_rms": float(np.max(np.abs(err))) / rms,
        "max_abs_norm": float(np.max(np.abs(err) / np.maximum(np.abs(ref), rms))),
        "ref_rms": rms,
    }


def assert_parity(got_bf16_bits, ref_f32, rel_rms_tol=REL_RMS_TOL, max_abs_norm_tol=MAX_ABS_NORM_TOL, what=""):
    p = parity(got_bf16_bits, ref_f32)
    assert p["rel_rms"] <= rel_rms_tol, f"{what}: relative RMS {p['rel_rms']:.3e} > {rel_rms_tol} ({p})"
    assert p["max_abs_norm"] <= max_abs_norm_tol, f"{what}: max-abs/max(|ref|,RMS) {p['max_abs_norm']:.3e} > {max_abs_norm_tol} ({p})"
    return p


def to_dev(arr: np.ndarray):
    """numpy (uint16/uint32/float32) -> CUDA tensor holding the same bytes."""
    import torch
    a = np.ascontiguousarray(arr)
    view = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32}.get(a.dtype)
    t = torch.from_numpy(a.view(view) if view else a)
    return t.cuda()


def from_dev(t, dtype):
    return t.cpu().numpy().view(dtype)
