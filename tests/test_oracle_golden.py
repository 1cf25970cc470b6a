"""The CPU oracle against every known-answer case the reference's tests hold for the path."""
import math

import numpy as np
import pytest

import refcases as rc
from ffai_b200 import capi, synth


@pytest.mark.parametrize("case", rc.ROUTER_CASES, ids=[c[0] for c in rc.ROUTER_CASES])
def test_router_known_answers(oracle_mod, case):
    _, logits, k, mode, norm, bias, exp_idx, exp_w, tol, ordered = case
    idx, w = oracle_mod.route(logits, k, mode, norm, bias)
    if ordered:
        assert idx.tolist() == exp_idx
    else:
        assert set(idx.tolist()) == set(exp_idx)
    if exp_w is not None:
        assert np.allclose(w, exp_w, atol=tol)
    if norm or mode == capi.GATING_TOPK_THEN_SOFTMAX:
        assert abs(float(w.sum()) - 1.0) < 1e-5


def test_router_specific_claims(oracle_mod):
    # MoELayerTests.swift:58-60: un-normalised weights sum below 0.9
    _, w = oracle_mod.route([1, 3, 2, 0], 2, 0, 0)
    assert w.sum() < 0.9
    # QuantizedOpsTests.swift:1018-1025: weight of expert 1 above 0.7
    idx, w = oracle_mod.route([1, 5, 3, 4], 2, 0, 1)
    assert dict(zip(idx.tolist(), w.tolist()))[1] > 0.7
    # LFM2TextTests.swift:131-134: biased weight of expert 1 above expert 0
    idx, w = oracle_mod.route([1, 3, 2, 0], 2, 0, 1, [0.5, 0, 0, 0.5])
    d = dict(zip(idx.tolist(), w.tolist()))
    assert d[1] > d[0]
    # LFM2TextTests.swift:138-150: nil bias leaves the routing unchanged
    a = oracle_mod.route([1, 3, 2, 0], 2, 0, 1, None)
    b = oracle_mod.route([1, 3, 2, 0], 2, 0, 1)
    assert a[0].tolist() == b[0].tolist() and a[1].tolist() == b[1].tolist()


def test_fast_path_equals_general_path(oracle_mod):
    """MoELayer.swift:146-172: softmax→top-k with renormalisation equals top-k→softmax."""
    rng = np.random.default_rng(0)
    for _ in range(200):
        logits = rng.standard_normal(32).astype(np.float32)
        i0, w0 = oracle_mod.route(logits, 4, 0, 1)
        i1, w1 = oracle_mod.route(logits, 4, 1, 1)
        assert i0.tolist() == i1.tolist() and np.array_equal(w0, w1)


def test_expf_matches_libm(oracle_mod):
    L = oracle_mod.lib()
    worst = 0.0
    for x in np.linspace(-80, 5, 4001).astype(np.float32):
        a = L.orc_expf(float(x))
        b = np.float32(math.exp(float(x)))
        worst = max(worst, abs(a - float(b)) / float(np.spacing(b)))
    assert worst <= 2.0
    assert L.orc_expf(0.0) == 1.0 and L.orc_expf(-200.0) == 0.0


def test_bf16_conversion(oracle_mod):
    L = oracle_mod.lib()
    rng = np.random.default_rng(1)
    vals = rng.standard_normal(2000).astype(np.float32) * np.float32(10.0)
    ours = np.array([L.orc_f32_to_bf16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(ours, rc.rne_bf16(vals))
    assert np.array_equal(ours, synth.f32_to_bf16(vals))
    # round-to-nearest-even on a tie: 1 + 2^-8 is halfway between two bf16 values
    assert L.orc_f32_to_bf16(1.0 + 2.0 ** -8) == 0x3F80
    assert L.orc_f32_to_bf16(1.0 + 3 * 2.0 ** -8) == 0x3F82


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_bit_layout_matches_reference_pack_helpers(oracle_mod, bits):
    rng = np.random.default_rng(bits)
    q = rng.integers(0, 1 << bits, size=128, dtype=np.uint32)
    ref_words = rc.ref_pack_row(q, bits)
    assert np.array_equal(oracle_mod.pack(q, bits), ref_words)
    assert np.array_equal(synth.pack_bits(q[None, :], bits)[0], ref_words)
    assert np.array_equal(oracle_mod.unpack(ref_words, bits, 128), q)
    assert np.array_equal(synth.unpack_bits(ref_words[None, :], bits, 128)[0], q)


@pytest.mark.parametrize("case", rc.gemv_cases(), ids=lambda c: c.name)
def test_dequant_gemv_known_answers(oracle_mod, case):
    out = oracle_mod.dequant_gemv(rc.bf16_f32(case.x), case.weight, case.scales, case.biases,
                                  case.out_dim, case.in_dim, case.bits, case.gs)
    assert np.allclose(out, case.expected, rtol=2e-5, atol=2e-4)


@pytest.mark.parametrize("case", rc.grouped_cases(), ids=lambda c: c.name)
def test_grouped_gemm_integer_hash_cases(oracle_mod, case):
    out = oracle_mod.gather_dequant_gemm(rc.bf16_f32(case.x), case.weight, case.scales, case.biases,
                                         case.indices, case.M, case.N, case.K, case.E, 4, case.gs)
    exp = case.expected()
    assert np.allclose(out, exp, rtol=1e-4, atol=1e-5)
    cos = float((out * exp).sum() / (np.linalg.norm(out) * np.linalg.norm(exp) + 1e-12))
    assert cos >= 0.99999  # the reference accepts 0.99 for its kernels (MoEBgemmBm64MppTests.swift:290)


def test_unpermute_two_token_case(oracle_mod):
    # OpsSpecialPathTests.swift:1081-1124
    eo = np.repeat(np.array([1, 2, 3, 4], dtype=np.float32)[:, None], 4, axis=1)
    out = oracle_mod.unpermute(eo, np.arange(4, dtype=np.uint32), np.full(4, 0.5, np.float32), 2, 4, 2)
    assert np.allclose(out[0], 1.5, atol=1e-6) and np.allclose(out[1], 3.5, atol=1e-6)


def test_chain8_accumulate_case(oracle_mod):
    # OpsSpecialPathTests.swift:445-472: sum_k s_k * v_k with s_k = k+1, v_k[j] = (j+1)*k'... = (j+1)*204
    k, hidden = 8, 16
    eo = np.stack([(np.arange(hidden) + 1) * (i + 1) for i in range(k)]).astype(np.float32)
    w = (np.arange(k) + 1).astype(np.float32)
    out = oracle_mod.unpermute(eo, np.arange(k, dtype=np.uint32), w, 1, hidden, k)
    assert np.allclose(out[0], (np.arange(hidden) + 1) * 204.0)


def test_swiglu_values(oracle_mod):
    # OpsSpecialPathTests.swift:314-330
    L = oracle_mod.lib()
    g, u = [0.0, 1.0, -1.0, 2.0], [3.0, 5.0, 7.0, 11.0]
    r = [L.orc_glu(a, b, capi.ACT_SWIGLU, 0.0, 0.0) for a, b in zip(g, u)]
    assert abs(r[0]) < 1e-5
    assert abs(r[1] - 5 / (1 + math.exp(-1))) < 1e-3
    assert abs(r[2] - 7 * (-1 / (1 + math.exp(1)))) < 1e-3
    assert abs(r[3] - 11 * (2 / (1 + math.exp(-2)))) < 1e-3


def test_clamped_swiglu_formula(oracle_mod):
    # GPTOSSText.swift:1421-1431 with L = 7, alpha = 1.702
    L = oracle_mod.lib()
    for g, u in [(0.5, 0.25), (9.0, 3.0), (-3.0, -9.0), (2.0, 8.5)]:
        gc, uc = min(g, 7.0), max(-7.0, min(u, 7.0))
        exp = gc / (1 + math.exp(-1.702 * gc)) * (uc + 1)
        assert abs(L.orc_glu(g, u, capi.ACT_CLAMPED_SWIGLU, 7.0, 1.702) - exp) < 1e-5 * max(1, abs(exp))


@pytest.mark.parametrize("with_shared", [False, True])
def test_four_expert_top2_layer(oracle_mod, with_shared):
    # MoELayerTests.swift:150-265
    arrays, x, expected = rc.four_expert_layer(with_shared)
    spec = synth.LayerSpec("four_expert", 64, 64, 4, 2, router_kind=capi.LINEAR_F32, router_logits_bf16=0,
                           shared_intermediate=64 if with_shared else 0, shared_bits=4, shared_group_size=64)
    layer = synth.HostLayer(spec, arrays)
    r = oracle_mod.moe_forward(layer, synth.f32_to_bf16(x)[None, :])
    assert r.indices[0].tolist() == [1, 2]
    assert np.allclose(r.weights[0], [0.73107, 0.26893], atol=1e-4)
    assert abs(float(r.out_f32[0, 0]) - expected) < 1e-3
    assert np.all(r.out_f32[0, 1:] == 0)


def test_plan_is_stable_sort(oracle_mod):
    rng = np.random.default_rng(3)
    T, k, E = 37, 4, 8
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.uint32)
    counts, offsets, perm, inv = oracle_mod.plan(idx, T, k, E)
    flat = idx.reshape(-1)
    order = np.argsort(flat, kind="stable").astype(np.uint32)
    assert np.array_equal(perm, order)
    assert np.array_equal(inv[perm], np.arange(T * k, dtype=np.uint32))
    assert np.array_equal(counts, np.bincount(flat, minlength=E).astype(np.uint32))
    assert np.array_equal(offsets, np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32))


def test_layer_matches_numpy_float64(oracle_mod):
    """Whole block against an independent float64 numpy evaluation (cfg1 shape)."""
    spec = synth.cfg1_tiny()
    layer = synth.make_layer(spec, 0)
    x = synth.make_tokens(16, spec.hidden, 0)
    r = oracle_mod.moe_forward(layer, x)
    a = layer.arrays
    xf = synth.bf16_to_f32(x).astype(np.float64)

    def deq(p, e, n_in):
        return synth.dequantize(a[p + ".weight"][e], a[p + ".scales"][e], a[p + ".biases"][e], 4, 64, n_in).astype(np.float64)

    out = np.zeros((16, spec.hidden))
    for t in range(16):
        for s in range(spec.top_k):
            e = int(r.indices[t, s])
            g = deq("experts.gate_proj", e, spec.hidden) @ xf[t]
            u = deq("experts.up_proj", e, spec.hidden) @ xf[t]
            inner = g / (1 + np.exp(-g)) * u
            out[t] += float(r.weights[t, s]) * (deq("experts.down_proj", e, spec.intermediate) @ inner)
    rel = np.sqrt(((r.out_f32 - out) ** 2).mean()) / np.sqrt((out ** 2).mean())
    assert rel < 1e-5
    # logits: fixed-order fp32 accumulation stays within fp32 noise of float64
    lg = xf @ a["gate.weight"].astype(np.float64).T
    assert np.allclose(r.logits, lg, atol=1e-4)
    # the stage-rounded variant (bf16 at every tensor boundary, as the reference's
    # per-op path does) stays within the block's output tolerance of the fp32 variant
    r2 = oracle_mod.moe_forward(layer, x, round_stages=True)
    rel2 = np.sqrt(((r2.out_f32 - r.out_f32) ** 2).mean()) / np.sqrt((r.out_f32 ** 2).mean())
    assert rel2 < 5e-3


def test_sigmoid_routing_follows_the_reference_steps(oracle_mod):
    """NemotronH routing (NemotronHText.swift:844-867) restated in numpy float32: sigmoid, selection on
    sigmoid + bias with ties to the lower index, raw sigmoids of the selected over (sum + 1e-20), scaling."""
    from ffai_b200 import capi
    logits = np.array([0.0, 1.0, -1.0, 2.0, 1.0, -3.0], dtype=np.float32)
    bias = np.array([0.5, 0.0, 0.0, -1.0, 0.0, 2.0], dtype=np.float32)
    sig = (np.float32(1) / (np.float32(1) + np.exp(-logits).astype(np.float32))).astype(np.float32)
    sel = sig + bias
    order = sorted(range(len(sel)), key=lambda i: (-sel[i], i))
    for k, norm, scale in ((2, 1, 2.5), (3, 1, 1.0), (3, 0, 0.5), (1, 1, 2.0)):
        want_idx = order[:k]
        w = sig[want_idx].astype(np.float32)
        if k > 1 and norm:
            w = (w / (np.float32(w.sum(dtype=np.float32)) + np.float32(1e-20))).astype(np.float32)
        w = (w * np.float32(scale)).astype(np.float32)
        idx, got = oracle_mod.route(logits, k, capi.GATING_SIGMOID_TOPK, norm, bias, routed_scaling=scale)
        assert list(idx) == want_idx
        assert np.allclose(got, w, rtol=3e-7, atol=0)
    # experts 1 and 4 tie on the selection score: the lower index goes first
    assert order.index(1) < order.index(4) and sel[1] == sel[4]
    # without a bias the selection is on the sigmoid itself
    idx, _ = oracle_mod.route(logits, 2, capi.GATING_SIGMOID_TOPK, 1, None)
    assert list(idx) == [3, 1]


def test_gateless_relu2_expert_matches_a_numpy_restatement(oracle_mod):
    """down(relu(up x)^2) with an always-on shared expert of the same form (NemotronHText.swift:741-763, 885-899),
    against a numpy float64 restatement on a small layer."""
    from ffai_b200 import synth
    spec = synth.nemotronh_style().with_(hidden=128, intermediate=64, n_experts=4, top_k=2, shared_intermediate=64)
    host = synth.make_layer(spec, 3)
    assert "experts.gate_proj.weight" not in host.arrays and "shared_expert.gate_proj.weight" not in host.arrays
    x = synth.make_tokens(5, spec.hidden, 3)
    r = oracle_mod.moe_forward(host, x)
    a = host.arrays
    xf = synth.bf16_to_f32(x).astype(np.float64)

    def deq(name, e, n):
        return synth.dequantize(a[name + ".weight"][e], a[name + ".scales"][e], a[name + ".biases"][e], 4, 64, n).astype(np.float64)

    want = np.zeros((5, spec.hidden))
    for t in range(5):
        for s in range(spec.top_k):
            e = int(r.indices[t, s])
            inner = np.maximum(deq("experts.up_proj", e, spec.hidden) @ xf[t], 0.0) ** 2
            want[t] += float(r.weights[t, s]) * (deq("experts.down_proj", e, spec.intermediate) @ inner)
        inner = np.maximum(deq("shared_expert.up_proj", 0, spec.hidden) @ xf[t], 0.0) ** 2
        want[t] += deq("shared_expert.down_proj", 0, spec.shared_intermediate) @ inner
    assert np.allclose(r.out_f32, want, rtol=2e-4, atol=2e-4 * np.abs(want).max())
