"""CPU checks of the weight-preparation oracles: the MXFP4 -> affine-int4 transcode against an
independent numpy restatement of the reference's host loop (GPTOSSText.swift:1150-1226), and the
affine quantizer against the properties the reference's own tests assert (QuantizedOpsAffineTests.swift)."""
import numpy as np
import pytest

from ffai_b200 import synth

LUT = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def transcode_numpy(packed_bytes, e8m0):
    """float32 numpy, same operations in the same order, written without reading the C oracle."""
    n = e8m0.size
    codes = np.empty((n, 32), dtype=np.uint8)
    codes[:, 0::2] = packed_bytes & 0x0F           # scan order: byte ascending, low nibble first
    codes[:, 1::2] = packed_bytes >> 4
    vals = LUT[codes]
    micro = np.exp2(e8m0.astype(np.float64) - 127.0).astype(np.float32)
    lo = vals.min(axis=1)
    hi = vals.max(axis=1)
    # strict comparisons: the first zero met decides the sign of a zero extreme
    zero = vals == 0
    first_zero = np.where(zero.any(axis=1), zero.argmax(axis=1), 0)
    zsign = np.signbit(vals[np.arange(n), first_zero])
    lo = np.where(lo == 0, np.where(zsign, np.float32(-0.0), np.float32(0.0)), lo).astype(np.float32)
    hi = np.where(hi == 0, np.where(zsign, np.float32(-0.0), np.float32(0.0)), hi).astype(np.float32)
    bias = (lo * micro).astype(np.float32)
    span = ((hi - lo).astype(np.float32) * micro).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        scale = np.where(span > 0, (span / np.float32(15.0)).astype(np.float32), np.float32(0)).astype(np.float32)
        inv = np.where(scale > 0, (np.float32(1.0) / scale).astype(np.float32), np.float32(0)).astype(np.float32)
    code_scale = (micro * inv).astype(np.float32)
    t = ((vals - lo[:, None]).astype(np.float32) * code_scale[:, None]).astype(np.float32)
    q = np.clip(np.where(t >= 0, np.floor(t + np.float32(0.5)), np.ceil(t - np.float32(0.5))), 0, 15).astype(np.uint8)
    out = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    return out, synth.f32_to_bf16(scale), synth.f32_to_bf16(bias)


def random_mxfp4(n, seed, e_lo=100, e_hi=140):
    rng = np.random.default_rng(seed)
    packed = rng.integers(0, 256, size=(n, 16), dtype=np.uint8)
    e8m0 = rng.integers(e_lo, e_hi, size=n, dtype=np.uint8)
    # groups that use a sub-range only (what trained weights look like), flat groups, all-zero groups
    packed[: n // 8] &= 0x33
    packed[n // 8: n // 6] = 0x55
    packed[n // 6: n // 5] = 0x00
    packed[n // 5: n // 4] = 0x80            # +0 and -0 only
    return packed, e8m0


def test_transcode_oracle_matches_independent_restatement(oracle_mod):
    packed, e8m0 = random_mxfp4(4096, 1)
    got = oracle_mod.mxfp4_to_affine4(packed, e8m0)
    ref = transcode_numpy(packed, e8m0)
    for a, b, name in zip(got, ref, ("codes", "scales", "biases")):
        assert np.array_equal(a, b), name


def test_transcode_known_group(oracle_mod):
    # codes 0..7 (values 0, .5, 1, 1.5, 2, 3, 4, 6) four times, micro-scale 2^0: grid step 0.4
    packed = np.tile(np.array([0x10, 0x32, 0x54, 0x76], dtype=np.uint8), 4)[None, :]
    out, sc, bi = oracle_mod.mxfp4_to_affine4(packed, np.array([127], dtype=np.uint8))
    q = np.empty(32, dtype=np.uint8)
    q[0::2] = out[0] & 0x0F
    q[1::2] = out[0] >> 4
    assert q[:8].tolist() == [0, 1, 3, 4, 5, 8, 10, 15]        # 2.5 and 7.5 round away from zero
    assert synth.bf16_to_f32(sc)[0] == pytest.approx(0.4, rel=4e-3) and bi[0] == 0


def test_transcode_keeps_values_within_half_a_step(oracle_mod):
    packed, e8m0 = random_mxfp4(2048, 2)
    out, sc, bi = oracle_mod.mxfp4_to_affine4(packed, e8m0)
    codes = np.empty((2048, 32), dtype=np.uint8); codes[:, 0::2] = packed & 15; codes[:, 1::2] = packed >> 4
    q = np.empty((2048, 32), dtype=np.uint8); q[:, 0::2] = out & 15; q[:, 1::2] = out >> 4
    micro = np.exp2(e8m0.astype(np.float64) - 127.0)
    true = LUT[codes].astype(np.float64) * micro[:, None]
    s = synth.bf16_to_f32(sc).astype(np.float64)[:, None]
    b = synth.bf16_to_f32(bi).astype(np.float64)[:, None]
    err = np.abs(q * s + b - true)
    # half a grid step, plus the bf16 rounding of scale and bias
    assert np.all(err <= 0.5 * s + 2.0 ** -8 * (np.abs(b) + 15 * s) + 1e-30)


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_quantizer_round_trip_and_packing(oracle_mod, bits, gs):
    rng = np.random.default_rng(bits * 10 + gs)
    w = synth.f32_to_bf16(rng.standard_normal((24, 256)).astype(np.float32))
    packed, sc, bi = oracle_mod.affine_quantize(w, bits, gs)
    q = np.stack([synth.unpack_bits(packed[r], bits, 256) for r in range(24)]).astype(np.float64)
    assert q.max() <= 2 ** bits - 1
    s = np.repeat(synth.bf16_to_f32(sc).astype(np.float64), gs, axis=1)
    b = np.repeat(synth.bf16_to_f32(bi).astype(np.float64), gs, axis=1)
    wf = synth.bf16_to_f32(w).astype(np.float64)
    step = np.abs(s)
    # Within about one quantization step, the bound the reference's tests use (QuantizedOpsAffineTests.swift:66,
    # 115, 379: 0.1 for a 0.13 step, 0.01 for 0.005, 0.4 for 0.33).  Half a step is not guaranteed: the grid is
    # re-anchored so that the edge of larger magnitude is exact, which can push the far end past its last level.
    err = np.abs(q * s + b - wf)
    assert np.all(err <= 1.05 * step + 2.0 ** -8 * (np.abs(b) + (2 ** bits - 1) * step) + 1e-6)
    assert np.mean(err <= 0.5 * step + 2.0 ** -8 * (np.abs(b) + (2 ** bits - 1) * step) + 1e-6) > 0.9
    # the edge of larger magnitude is reproduced up to the bf16 rounding of scale and bias
    wg = wf.reshape(24, 256 // gs, gs)
    edge = np.where(np.abs(wg.min(axis=2)) > np.abs(wg.max(axis=2)), wg.min(axis=2), wg.max(axis=2))
    deq = (q * s + b).reshape(24, 256 // gs, gs)
    closest = np.abs(deq - edge[:, :, None]).min(axis=2)
    assert np.all(closest <= 2.0 ** -7 * np.abs(edge) + 1e-6)
    assert q.min() == 0 and q.max() == 2 ** bits - 1


def test_quantizer_flat_and_zero_groups(oracle_mod):
    w = np.zeros((2, 64), dtype=np.float32)
    w[1, :] = 3.0
    packed, sc, bi = oracle_mod.affine_quantize(synth.f32_to_bf16(w), 4, 64)
    q = np.stack([synth.unpack_bits(packed[r], 4, 64) for r in range(2)]).astype(np.float64)
    deq = q * synth.bf16_to_f32(sc).astype(np.float64) + synth.bf16_to_f32(bi).astype(np.float64)
    assert np.all(np.isfinite(deq)) and np.allclose(deq, w, atol=1e-6)


def test_add_rmsnorm_oracle_on_the_reference_pattern(oracle_mod):
    """The inputs of the reference's own check (OpsTests.swift:1017-1019: index patterns, not data), in bf16."""
    rows, n, eps = 2, 128, 1e-6
    i = np.arange(rows * n)
    a = ((i % 19) - 9).astype(np.float32) * np.float32(0.31)
    b = ((i % 13) - 6).astype(np.float32) * np.float32(0.17)
    w = (1.0 + (np.arange(n) % 7) * 0.05).astype(np.float32)
    ab, bb, wb = (synth.f32_to_bf16(v) for v in (a.reshape(rows, n), b.reshape(rows, n), w))
    res, nrm, nf = oracle_mod.add_rmsnorm(ab, bb, wb, eps)
    s = synth.bf16_to_f32(ab).astype(np.float64) + synth.bf16_to_f32(bb).astype(np.float64)
    ref = s / np.sqrt((s * s).mean(axis=1, keepdims=True) + eps) * synth.bf16_to_f32(wb).astype(np.float64)
    assert np.abs(synth.bf16_to_f32(res) - s).max() < 1e-3 * 32      # the reference's 1e-3, widened for bf16 storage
    assert np.abs(nf - ref).max() < 1e-5
    assert np.abs(synth.bf16_to_f32(nrm) - ref).max() < 1e-2


def test_plain_rmsnorm_oracle_on_the_reference_check(oracle_mod):
    """Without a second addend the op is the reference's RMSNorm; its own check (LayersTests.swift:101-128):
    x = 1..128, weight = 1, eps = 1e-6, y = x / sqrt(mean(x^2)) within 1e-2 (bf16 storage here: within 0.5 %)."""
    n = 128
    xs = np.arange(1, n + 1, dtype=np.float32)
    xb = synth.f32_to_bf16(xs.reshape(1, n))
    wb = synth.f32_to_bf16(np.ones(n, dtype=np.float32))
    res, nrm, nf = oracle_mod.add_rmsnorm(xb, None, wb, 1e-6)
    expected = xs / np.sqrt((xs.astype(np.float64) ** 2).mean())
    assert np.array_equal(res, xb)                       # the "sum" is the input itself
    assert np.abs(nf[0] - expected).max() < 1e-2
    assert np.abs(synth.bf16_to_f32(nrm)[0] - expected).max() < 5e-3 * expected.max()
