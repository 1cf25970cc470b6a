"""Weight preparation on the GPU against the CPU oracle, through the C ABI: bit-exact."""
import numpy as np
import pytest

from ffai_b200 import capi, synth
from helpers import from_dev, to_dev
from test_weight_prep_oracle import random_mxfp4

pytestmark = pytest.mark.gpu


def gpu_transcode(lib, packed, e8m0):
    import torch
    n = e8m0.size
    dp, de = to_dev(packed.reshape(-1)), to_dev(e8m0)
    ow = torch.zeros(n * 16, dtype=torch.uint8, device="cuda")
    osc = torch.zeros(n, dtype=torch.int16, device="cuda")
    obi = torch.zeros(n, dtype=torch.int16, device="cuda")
    capi.check(lib.ffai_op_mxfp4_to_affine_int4(dp.data_ptr(), de.data_ptr(), n, ow.data_ptr(), osc.data_ptr(), obi.data_ptr(), None),
               "ffai_op_mxfp4_to_affine_int4")
    torch.cuda.synchronize()
    return from_dev(ow, np.uint8).reshape(n, 16), from_dev(osc, np.uint16), from_dev(obi, np.uint16)


# scale bytes whose power of two leaves the fp32 range make the reference trap (Int of a non-finite value); not tested
@pytest.mark.parametrize("n,seed,e_lo,e_hi", [(1, 0, 120, 130), (777, 1, 100, 140), (1 << 16, 2, 8, 250)])
def test_mxfp4_transcode_bit_exact(ffai_lib, oracle_mod, n, seed, e_lo, e_hi):
    packed, e8m0 = random_mxfp4(n, seed, e_lo, e_hi)
    got = gpu_transcode(ffai_lib, packed, e8m0)
    ref = oracle_mod.mxfp4_to_affine4(packed, e8m0)
    for a, b, name in zip(got, ref, ("codes", "scales", "biases")):
        assert np.array_equal(a, b), name


def test_transcoded_experts_run_through_the_gemv(ffai_lib, oracle_mod):
    """MXFP4 rows -> affine int4 (group 32) on the GPU -> the library's own dequant GEMV == the values MXFP4 encodes,
    up to the transcode's grid (half a step per weight)."""
    import torch
    out_dim, in_dim = 64, 256
    packed, e8m0 = random_mxfp4(out_dim * in_dim // 32, 5, 118, 124)
    w, sc, bi = gpu_transcode(ffai_lib, packed, e8m0)
    x = synth.make_tokens(1, in_dim, 9)
    dx = to_dev(x.reshape(-1))
    dw, dsc, dbi = to_dev(w.reshape(-1).view(np.uint32)), to_dev(sc), to_dev(bi)
    out = torch.zeros(out_dim, dtype=torch.int16, device="cuda")
    capi.check(ffai_lib.ffai_op_dequant_gemv(dx.data_ptr(), dw.data_ptr(), dsc.data_ptr(), dbi.data_ptr(), out.data_ptr(),
                                             out_dim, in_dim, 4, 32, None), "ffai_op_dequant_gemv")
    torch.cuda.synchronize()
    got = synth.bf16_to_f32(from_dev(out, np.uint16)).astype(np.float64)
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6])
    codes = np.empty((e8m0.size, 32), dtype=np.uint8); codes[:, 0::2] = packed & 15; codes[:, 1::2] = packed >> 4
    true_w = (lut[codes] * np.exp2(e8m0.astype(np.float64) - 127)[:, None]).reshape(out_dim, in_dim)
    ref = true_w @ synth.bf16_to_f32(x).astype(np.float64).reshape(-1)
    step = synth.bf16_to_f32(sc).astype(np.float64).reshape(out_dim, -1).max()
    xs = np.abs(synth.bf16_to_f32(x)).sum()
    assert np.all(np.abs(got - ref) <= 0.5 * step * xs + 2.0 ** -7 * np.abs(ref) + 1e-6)


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_affine_quantizer_bit_exact(ffai_lib, oracle_mod, bits, gs):
    import torch
    rng = np.random.default_rng(100 * bits + gs)
    rows, K = 96, 512
    w = rng.standard_normal((rows, K)).astype(np.float32) * rng.uniform(0.01, 4.0, size=(rows, 1)).astype(np.float32)
    w[3] = 0.0                       # a flat row
    w[4, :gs] = 2.5                  # a flat group
    w[5] = np.abs(w[5])              # one-sided groups
    wb = synth.f32_to_bf16(w)
    dwt = to_dev(wb.reshape(-1))
    ow = torch.zeros(rows * K * bits // 32, dtype=torch.int32, device="cuda")
    osc = torch.zeros(rows * K // gs, dtype=torch.int16, device="cuda")
    obi = torch.zeros(rows * K // gs, dtype=torch.int16, device="cuda")
    capi.check(ffai_lib.ffai_op_affine_quantize(dwt.data_ptr(), rows, K, bits, gs, ow.data_ptr(), osc.data_ptr(), obi.data_ptr(), None),
               "ffai_op_affine_quantize")
    torch.cuda.synchronize()
    rp, rs, rb = oracle_mod.affine_quantize(wb, bits, gs)
    assert np.array_equal(from_dev(osc, np.uint16).reshape(rs.shape), rs), "scales"
    assert np.array_equal(from_dev(obi, np.uint16).reshape(rb.shape), rb), "biases"
    assert np.array_equal(from_dev(ow, np.uint32).reshape(rp.shape), rp), "codes"


def test_weight_prep_rejects_bad_arguments(ffai_lib):
    assert ffai_lib.ffai_op_mxfp4_to_affine_int4(None, None, 4, None, None, None, None) == capi.FFAI_ERR_INVALID_ARG
    assert ffai_lib.ffai_op_affine_quantize(None, 1, 64, 4, 64, None, None, None, None) == capi.FFAI_ERR_INVALID_ARG


@pytest.mark.parametrize("rows,n", [(1, 2880), (2, 128), (7, 2048), (64, 5376)])
def test_add_rmsnorm_matches_oracle(ffai_lib, oracle_mod, rows, n):
    import torch
    rng = np.random.default_rng(rows * 31 + n)
    a = synth.f32_to_bf16(rng.standard_normal((rows, n)).astype(np.float32) * 3)
    b = synth.f32_to_bf16(rng.standard_normal((rows, n)).astype(np.float32))
    w = synth.f32_to_bf16((1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32))
    da, db, dw = to_dev(a.reshape(-1)), to_dev(b.reshape(-1)), to_dev(w)
    res = torch.zeros(rows * n, dtype=torch.int16, device="cuda")
    nrm = torch.zeros(rows * n, dtype=torch.int16, device="cuda")
    capi.check(ffai_lib.ffai_op_add_rmsnorm(da.data_ptr(), db.data_ptr(), dw.data_ptr(), 1e-6, rows, n, res.data_ptr(), nrm.data_ptr(), None),
               "ffai_op_add_rmsnorm")
    torch.cuda.synchronize()
    ores, onrm, onf = oracle_mod.add_rmsnorm(a, b, w, 1e-6)
    assert np.array_equal(from_dev(res, np.uint16).reshape(rows, n), ores)          # the sum is exact in fp32: same bits
    got = synth.bf16_to_f32(from_dev(nrm, np.uint16)).reshape(rows, n)
    # the sum of squares is reduced in another order: at most one bf16 step from the fp32 oracle value
    assert np.all(np.abs(got - onf) <= 2.0 ** -7 * np.abs(onf) + 1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,n", [(1, 2816), (33, 2048)])
def test_plain_rmsnorm_matches_oracle(ffai_lib, oracle_mod, rows, n):
    """b = NULL: the row-wise RMSNorm in front of a Gemma 4 router and its experts; no residual output needed."""
    import torch
    rng = np.random.default_rng(rows + n)
    a = synth.f32_to_bf16(rng.standard_normal((rows, n)).astype(np.float32) * 2)
    w = synth.f32_to_bf16((1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32))
    da, dw = to_dev(a.reshape(-1)), to_dev(w)
    nrm = torch.zeros(rows * n, dtype=torch.int16, device="cuda")
    capi.check(ffai_lib.ffai_op_add_rmsnorm(da.data_ptr(), None, dw.data_ptr(), 1e-6, rows, n, None, nrm.data_ptr(), None),
               "ffai_op_add_rmsnorm")
    torch.cuda.synchronize()
    _, _, onf = oracle_mod.add_rmsnorm(a, None, w, 1e-6)
    got = synth.bf16_to_f32(from_dev(nrm, np.uint16)).reshape(rows, n)
    assert np.all(np.abs(got - onf) <= 2.0 ** -7 * np.abs(onf) + 1e-6)
    # a second addend without a place for the sum is refused
    assert ffai_lib.ffai_op_add_rmsnorm(da.data_ptr(), da.data_ptr(), dw.data_ptr(), 1e-6, rows, n, None, nrm.data_ptr(), None) == capi.FFAI_ERR_INVALID_ARG
