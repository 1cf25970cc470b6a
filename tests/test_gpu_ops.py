"""Operator-level parity on the GPU, through the C ABI, restating the reference's unit tests:
QuantizedOpsTests (per-bit-width GEMV, expert-indexed GEMV, GPU router), MoEBgemmBm64MppTests
(grouped GEMM integer-hash cases), OpsSpecialPathTests (swiglu, unpermute, chain-8 sum)."""
import ctypes as C

import numpy as np
import pytest

import refcases as rc
from ffai_b200 import capi, synth
from helpers import assert_parity, from_dev, to_dev

pytestmark = pytest.mark.gpu


def _sync():
    import torch
    torch.cuda.synchronize()


def _empty(n, dtype):
    import torch
    return torch.zeros(n, dtype=dtype, device="cuda")


@pytest.mark.parametrize("case", rc.gemv_cases(), ids=lambda c: c.name)
def test_dequant_gemv_cases(ffai_lib, oracle_mod, case):
    import torch
    x, w, s, b = to_dev(case.x), to_dev(case.weight), to_dev(case.scales), to_dev(case.biases)
    out = _empty(case.out_dim, torch.int16)
    rc_ = ffai_lib.ffai_op_dequant_gemv(x.data_ptr(), w.data_ptr(), s.data_ptr(), b.data_ptr(), out.data_ptr(),
                                        case.out_dim, case.in_dim, case.bits, case.gs, None)
    assert rc_ == capi.FFAI_OK
    _sync()
    got = synth.bf16_to_f32(from_dev(out, np.uint16))
    # the reference's own acceptance (QuantizedOpsTests.swift:256-259): max(5 %, 1.0)
    tol_ref = np.maximum(np.abs(case.expected) * 0.05, 1.0)
    assert np.all(np.abs(got - case.expected) < tol_ref)
    # ours: bf16 rounding of an fp32-accumulated result
    orc = oracle_mod.dequant_gemv(rc.bf16_f32(case.x), case.weight, case.scales, case.biases,
                                  case.out_dim, case.in_dim, case.bits, case.gs)
    assert np.all(np.abs(got - orc) <= np.abs(orc) * 2.0 ** -8 + 1e-3)


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
def test_expert_indexed_gemv_equals_per_expert_gemv(ffai_lib, bits):
    """QuantizedOpsTests.swift:935-997: the stacked [E,out,in*bits/32] path picks the same slab."""
    import torch
    rng = np.random.default_rng(bits)
    E, O, K, gs = 4, 24, 256, 64
    q = rng.integers(0, 1 << bits, size=(E, O, K), dtype=np.uint32)
    w = synth.pack_bits(q, bits)
    s = synth.f32_to_bf16(rng.uniform(0.005, 0.02, (E, O, K // gs)).astype(np.float32))
    b = synth.f32_to_bf16(rng.uniform(-0.1, 0.1, (E, O, K // gs)).astype(np.float32))
    x = synth.f32_to_bf16(rng.standard_normal(K).astype(np.float32))
    dx, dw, ds, db = to_dev(x), to_dev(w), to_dev(s), to_dev(b)
    for e in range(E):
        out_a, out_b = _empty(O, torch.int16), _empty(O, torch.int16)
        ei = to_dev(np.array([e], dtype=np.uint32))
        assert ffai_lib.ffai_op_dequant_gemv_expert_indexed(dx.data_ptr(), dw.data_ptr(), ds.data_ptr(), db.data_ptr(),
                                                            ei.data_ptr(), out_a.data_ptr(), E, O, K, bits, gs, None) == 0
        we, se, be = to_dev(w[e]), to_dev(s[e]), to_dev(b[e])
        assert ffai_lib.ffai_op_dequant_gemv(dx.data_ptr(), we.data_ptr(), se.data_ptr(), be.data_ptr(),
                                             out_b.data_ptr(), O, K, bits, gs, None) == 0
        _sync()
        assert np.array_equal(from_dev(out_a, np.uint16), from_dev(out_b, np.uint16))


@pytest.mark.parametrize("case", rc.grouped_cases(), ids=lambda c: c.name)
def test_grouped_gemm_integer_hash_cases(ffai_lib, case):
    import torch
    x, w, s, b, idx = (to_dev(a) for a in (case.x, case.weight, case.scales, case.biases, case.indices))
    out = _empty(case.M * case.N, torch.int16)
    assert ffai_lib.ffai_op_moe_gather_dequant_gemm(x.data_ptr(), w.data_ptr(), s.data_ptr(), b.data_ptr(), idx.data_ptr(),
                                                    out.data_ptr(), case.M, case.N, case.K, case.E, 4, case.gs, None) == 0
    _sync()
    got = synth.bf16_to_f32(from_dev(out, np.uint16)).reshape(case.M, case.N).astype(np.float64)
    exp = case.expected()
    cos = float((got * exp).sum() / (np.linalg.norm(got) * np.linalg.norm(exp) + 1e-12))
    assert cos >= 0.99  # the reference's acceptance, MoEBgemmBm64MppTests.swift:290
    assert_parity(from_dev(out, np.uint16), exp.astype(np.float32), what=case.name)


@pytest.mark.parametrize("case", rc.ROUTER_CASES, ids=[c[0] for c in rc.ROUTER_CASES])
def test_router_known_answers(ffai_lib, oracle_mod, case):
    import torch
    _, logits, k, mode, norm, bias, exp_idx, exp_w, tol, ordered = case
    lg = to_dev(np.array(logits, dtype=np.float32))
    eb = to_dev(np.array(bias, dtype=np.float32)) if bias is not None else None
    idx, w = _empty(k, torch.int32), _empty(k, torch.float32)
    assert ffai_lib.ffai_op_moe_router_topk(lg.data_ptr(), idx.data_ptr(), w.data_ptr(), 1, len(logits), k, mode, norm,
                                            eb.data_ptr() if eb is not None else None, None) == 0
    _sync()
    gi, gw = from_dev(idx, np.uint32), from_dev(w, np.float32)
    oi, ow = oracle_mod.route(logits, k, mode, norm, bias)
    assert gi.tolist() == oi.tolist()          # bit-exact against the oracle, order included
    assert np.array_equal(gw, ow)              # same exp, same operation order: identical bits
    if ordered:
        assert gi.tolist() == exp_idx
    if exp_w is not None:
        assert np.allclose(gw, exp_w, atol=tol)


@pytest.mark.parametrize("E,k,mode,norm,use_bias", [(8, 2, 0, 1, False), (32, 4, 1, 1, False), (128, 8, 0, 1, False),
                                                    (256, 8, 0, 0, False), (64, 6, 0, 1, True), (1000, 32, 0, 0, True),
                                                    (5, 5, 1, 1, False)])
def test_router_random_bit_exact(ffai_lib, oracle_mod, E, k, mode, norm, use_bias):
    import torch
    rng = np.random.default_rng(E * 7 + k)
    T = 257
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[3, :] = 0.25                      # all-equal row: ties go to the lower index
    logits[5, ::2] = logits[5, 1::2][: len(logits[5, ::2])] if E % 2 == 0 else logits[5, ::2]
    logits = synth.bf16_to_f32(synth.f32_to_bf16(logits))   # many exact ties, as bf16 logits have
    bias = (0.02 * rng.standard_normal(E)).astype(np.float32) if use_bias else None
    lg = to_dev(logits)
    eb = to_dev(bias) if use_bias else None
    idx, w = _empty(T * k, torch.int32), _empty(T * k, torch.float32)
    assert ffai_lib.ffai_op_moe_router_topk(lg.data_ptr(), idx.data_ptr(), w.data_ptr(), T, E, k, mode, norm,
                                            eb.data_ptr() if eb is not None else None, None) == 0
    _sync()
    gi, gw = from_dev(idx, np.uint32).reshape(T, k), from_dev(w, np.float32).reshape(T, k)
    for t in range(T):
        oi, ow = oracle_mod.route(logits[t], k, mode, norm, bias)
        assert gi[t].tolist() == oi.tolist(), t
        assert np.array_equal(gw[t], ow), t


@pytest.mark.parametrize("T,k,E", [(1, 8, 128), (16, 2, 8), (64, 4, 32), (300, 8, 128), (2048, 8, 128), (1500, 2, 8), (4096, 8, 256), (4100, 8, 256)])
def test_plan_matches_oracle(ffai_lib, oracle_mod, T, k, E):
    import torch
    rng = np.random.default_rng(T)
    p = 1.0 / np.arange(1, E + 1) ** 1.1
    p /= p.sum()
    idx = np.stack([rng.choice(E, size=k, replace=False, p=p) for _ in range(T)]).astype(np.uint32)
    di = to_dev(idx)
    counts, offsets = _empty(E, torch.int32), _empty(E + 1, torch.int32)
    perm, inv = _empty(T * k, torch.int32), _empty(T * k, torch.int32)
    ws = _empty(max(1, ffai_lib.ffai_op_moe_plan_workspace_bytes(T * k, E) // 4), torch.int32)
    assert ffai_lib.ffai_op_moe_plan(di.data_ptr(), T, k, E, counts.data_ptr(), offsets.data_ptr(), perm.data_ptr(),
                                     inv.data_ptr(), ws.data_ptr(), None) == 0
    _sync()
    oc, oo, op, oi = oracle_mod.plan(idx, T, k, E)
    assert np.array_equal(from_dev(counts, np.uint32), oc)
    assert np.array_equal(from_dev(offsets, np.uint32), oo)
    assert np.array_equal(from_dev(perm, np.uint32), op)
    assert np.array_equal(from_dev(inv, np.uint32), oi)


def test_gather_rows(ffai_lib):
    import torch
    rng = np.random.default_rng(0)
    table = rng.integers(0, 65535, size=(50, 256), dtype=np.uint16)
    ids = rng.integers(0, 50, size=400, dtype=np.uint32)
    dt, di = to_dev(table), to_dev(ids)
    out = _empty(400 * 256, torch.int16)
    assert ffai_lib.ffai_op_gather_rows(dt.data_ptr(), di.data_ptr(), out.data_ptr(), 400, 256, None) == 0
    _sync()
    assert np.array_equal(from_dev(out, np.uint16).reshape(400, 256), table[ids])


def test_swiglu_unpermute_chain8_values(ffai_lib):
    import torch
    # OpsSpecialPathTests.swift:314-330
    g = to_dev(synth.f32_to_bf16(np.array([0, 1, -1, 2], dtype=np.float32)))
    u = to_dev(synth.f32_to_bf16(np.array([3, 5, 7, 11], dtype=np.float32)))
    o = _empty(4, torch.int16)
    assert ffai_lib.ffai_op_glu_activation(g.data_ptr(), u.data_ptr(), o.data_ptr(), 4, capi.ACT_SWIGLU, 0.0, 0.0, None) == 0
    _sync()
    r = synth.bf16_to_f32(from_dev(o, np.uint16))
    exp = np.array([0, 5 / (1 + np.exp(-1)), -7 / (1 + np.exp(1)), 22 / (1 + np.exp(-2))])
    assert np.allclose(r, exp, rtol=2.0 ** -8, atol=1e-5)
    # OpsSpecialPathTests.swift:1081-1124
    eo = to_dev(synth.f32_to_bf16(np.repeat(np.array([1, 2, 3, 4], dtype=np.float32)[:, None], 4, axis=1)))
    inv, w = to_dev(np.arange(4, dtype=np.uint32)), to_dev(np.full(4, 0.5, dtype=np.float32))
    out = _empty(8, torch.int16)
    assert ffai_lib.ffai_op_moe_unpermute(eo.data_ptr(), inv.data_ptr(), w.data_ptr(), out.data_ptr(), 2, 4, 2, None) == 0
    _sync()
    r = synth.bf16_to_f32(from_dev(out, np.uint16)).reshape(2, 4)
    assert np.allclose(r[0], 1.5) and np.allclose(r[1], 3.5)
    # OpsSpecialPathTests.swift:445-472: eight-way weighted sum = (j+1)*204
    eo = to_dev(synth.f32_to_bf16(np.stack([(np.arange(16) + 1) * (i + 1) for i in range(8)]).astype(np.float32)))
    inv, w = to_dev(np.arange(8, dtype=np.uint32)), to_dev((np.arange(8) + 1).astype(np.float32))
    out = _empty(16, torch.int16)
    assert ffai_lib.ffai_op_moe_unpermute(eo.data_ptr(), inv.data_ptr(), w.data_ptr(), out.data_ptr(), 1, 16, 8, None) == 0
    _sync()
    assert np.allclose(synth.bf16_to_f32(from_dev(out, np.uint16)), (np.arange(16) + 1) * 204.0, rtol=2.0 ** -8)


def test_sigmoid_scalar_fma(ffai_lib):
    import torch
    rng = np.random.default_rng(5)
    T, H = 3, 64
    gate = rng.standard_normal(T).astype(np.float32)
    val, base, res = (rng.standard_normal((T, H)).astype(np.float32) for _ in range(3))
    bits = [synth.f32_to_bf16(a) for a in (gate, val, base, res)]
    dg, dv, db, dr = (to_dev(a) for a in bits)
    out = _empty(T * H, torch.int16)
    assert ffai_lib.ffai_op_sigmoid_scalar_fma(dg.data_ptr(), dv.data_ptr(), db.data_ptr(), dr.data_ptr(), out.data_ptr(), T, H, None) == 0
    _sync()
    f = [synth.bf16_to_f32(a).astype(np.float64) for a in bits]
    exp = f[3] + f[2] + (1 / (1 + np.exp(-f[0])))[:, None] * f[1]
    assert np.allclose(synth.bf16_to_f32(from_dev(out, np.uint16)).reshape(T, H), exp, rtol=2.0 ** -7, atol=1e-2)
