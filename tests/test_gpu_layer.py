"""Whole-block parity on the GPU, through the C ABI, against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

import refcases as rc
from ffai_b200 import capi, synth
from ffai_b200.moe import MoELayer
from helpers import assert_parity, from_dev, parity, to_dev

pytestmark = pytest.mark.gpu


def run_and_check(oracle_mod, spec, T, seed=0, residual=False, max_tokens=None, layer=None, host=None,
                  token_mask=None, rel_rms_tol=5e-3, max_abs_norm_tol=2e-2, path=None, options=None):
    host = host or synth.make_layer(spec, seed)
    x = synth.make_tokens(T, spec.hidden, seed)
    res = synth.make_tokens(T, spec.hidden, seed + 17) if residual else None
    own = layer is None
    layer = layer or MoELayer(host, max_tokens or T)
    try:
        if path is not None:
            layer.set_option("path", path)
        for name, value in (options or {}).items():
            layer.set_option(name, value)
        out, dbg = layer.forward_host(x, residual=res, debug=True)
    finally:
        if own:
            layer.close()
    ref = oracle_mod.moe_forward(host, x, residual=res, token_mask=token_mask)
    # routing: bit-exact
    assert np.array_equal(dbg.logits, ref.logits), "router logits differ"
    assert np.array_equal(dbg.indices, ref.indices), "expert indices differ"
    assert np.array_equal(dbg.weights, ref.weights), "combine weights differ"
    assert np.array_equal(dbg.counts, ref.counts)
    assert np.array_equal(dbg.offsets, ref.offsets)
    assert np.array_equal(dbg.perm, ref.perm)
    assert np.array_equal(dbg.inv_perm, ref.inv_perm)
    if token_mask is not None:
        sel = np.nonzero(token_mask)[0]
        return assert_parity(out[sel], ref.out_f32[sel], rel_rms_tol, max_abs_norm_tol, what=spec.name)
    return assert_parity(out, ref.out_f32, rel_rms_tol, max_abs_norm_tol, what=spec.name)


def test_cfg1_tiny_layer(oracle_mod):
    run_and_check(oracle_mod, synth.cfg1_tiny(), 16)


@pytest.mark.parametrize("T", [1, 8, 32, 64])
def test_cfg2_gptoss_decode_batches(oracle_mod, T):
    run_and_check(oracle_mod, synth.cfg2_gptoss(), T)


def test_cfg2_with_expert_row_biases_and_residual(oracle_mod):
    run_and_check(oracle_mod, synth.cfg2_gptoss().with_(expert_row_bias=1), 5, residual=True)


def test_cfg3_qwen_small_prefill(oracle_mod):
    run_and_check(oracle_mod, synth.cfg3_qwen(), 96)


def test_cfg3_single_token(oracle_mod):
    run_and_check(oracle_mod, synth.cfg3_qwen(), 1)


def test_cfg4_shared_expert_small(oracle_mod):
    run_and_check(oracle_mod, synth.cfg4_shared(), 48)


def test_shared_expert_without_gate(oracle_mod):
    spec = synth.cfg1_tiny().with_(name="granite_style", shared_intermediate=256, shared_bits=4, shared_group_size=64)
    run_and_check(oracle_mod, spec, 7)


@pytest.mark.parametrize("bits", [3, 5, 6, 8])
def test_odd_bit_widths(oracle_mod, bits):
    spec = synth.LayerSpec(f"bits{bits}", 512, 256, 16, 4, expert_bits=bits)
    run_and_check(oracle_mod, spec, 40)


@pytest.mark.parametrize("gs", [32, 128])
def test_group_sizes(oracle_mod, gs):
    spec = synth.LayerSpec(f"gs{gs}", 512, 256, 8, 2, expert_group_size=gs)
    run_and_check(oracle_mod, spec, 9)


def test_softmax_without_renormalisation_and_expert_bias(oracle_mod):
    spec = synth.LayerSpec("raw_softmax", 256, 128, 16, 4, norm_topk_prob=0)
    run_and_check(oracle_mod, spec, 33)
    spec = synth.LayerSpec("lfm2_bias", 256, 128, 16, 4, router_expert_bias=1)
    run_and_check(oracle_mod, spec, 33)


def test_gelu_glu_activation(oracle_mod):
    spec = synth.LayerSpec("gelu", 256, 128, 8, 2, activation=capi.ACT_GELU_GLU, gating_mode=capi.GATING_TOPK_THEN_SOFTMAX)
    run_and_check(oracle_mod, spec, 12)


def test_skewed_routing_layer(oracle_mod):
    spec = synth.LayerSpec("skew", 512, 256, 64, 8, router_has_bias=1, zipf_s=1.1, zipf_strength=1.5)
    p = run_and_check(oracle_mod, spec, 200)
    assert p["ref_rms"] > 0


def test_ragged_token_counts_on_one_handle(oracle_mod):
    """One handle, many batch sizes (empty, 1, odd, max): no state leaks between calls."""
    spec = synth.LayerSpec("ragged", 256, 128, 8, 2)
    host = synth.make_layer(spec, 3)
    layer = MoELayer(host, 70)
    try:
        out, _ = layer.forward_host(np.zeros((0, spec.hidden), dtype=np.uint16))
        assert out.shape == (0, spec.hidden)
        for T in (70, 1, 13, 64, 2, 70):
            run_and_check(oracle_mod, spec, T, seed=T, layer=layer, host=host)
        with pytest.raises(capi.FFAICudaError) as ei:
            layer.forward_host(np.zeros((71, spec.hidden), dtype=np.uint16))
        assert ei.value.status == capi.FFAI_ERR_INVALID_ARG
    finally:
        layer.close()


def test_all_tokens_to_the_same_experts(oracle_mod):
    """Collision extreme: identical rows route every token to the same k experts."""
    spec = synth.LayerSpec("collide", 256, 128, 8, 2)
    host = synth.make_layer(spec, 4)
    x = np.repeat(synth.make_tokens(1, spec.hidden, 4), 50, axis=0)
    ref = oracle_mod.moe_forward(host, x)
    layer = MoELayer(host, 50)
    try:
        # path 1: CUDA-core GEMV (fp32 throughout).  path 2: tcgen05 GEMM, which rounds the
        # dequantised weights and the intermediate to bf16; on this single repeated row the output
        # is small against its intermediates (ref RMS 0.4), so that rounding shows: 2e-2 / 5e-2 there.
        for path, rel_tol, abs_tol in ((1, 5e-3, 2e-2), (2, 2e-2, 5e-2)):
            layer.set_option("path", path)
            out, dbg = layer.forward_host(x, debug=True)
            assert np.array_equal(dbg.indices, ref.indices) and np.array_equal(dbg.perm, ref.perm)
            assert (dbg.counts > 0).sum() == 2
            assert_parity(out, ref.out_f32, rel_tol, abs_tol, what=f"path {path}")
            assert np.all(out == out[0])  # identical rows give identical outputs: the reduction order is fixed
    finally:
        layer.close()


@pytest.mark.parametrize("with_shared", [False, True])
def test_reference_four_expert_layer(oracle_mod, with_shared):
    """MoELayerTests.swift:150-265 through the C ABI."""
    arrays, x, expected = rc.four_expert_layer(with_shared)
    spec = synth.LayerSpec("four_expert", 64, 64, 4, 2, router_kind=capi.LINEAR_F32, router_logits_bf16=0,
                           shared_intermediate=64 if with_shared else 0, shared_bits=4, shared_group_size=64)
    host = synth.HostLayer(spec, arrays)
    layer = MoELayer(host, 1)
    try:
        out, dbg = layer.forward_host(synth.f32_to_bf16(x)[None, :], debug=True)
    finally:
        layer.close()
    assert dbg.indices[0].tolist() == [1, 2]
    assert np.allclose(dbg.weights[0], [0.73107, 0.26893], atol=1e-4)
    got = float(synth.bf16_to_f32(out)[0, 0])
    assert abs(got - expected) <= abs(expected) * 2.0 ** -8 + 1e-3


def test_device_pointer_forward_matches_host_forward(oracle_mod):
    import torch
    spec = synth.cfg1_tiny()
    host = synth.make_layer(spec, 0)
    x = synth.make_tokens(16, spec.hidden, 0)
    layer = MoELayer(host, 16)
    try:
        out_h, _ = layer.forward_host(x)
        dx = to_dev(x)
        dout = torch.zeros(16 * spec.hidden, dtype=torch.int16, device="cuda")
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            layer.forward_ptr(dx.data_ptr(), 16, dout.data_ptr(), stream=st.cuda_stream)
        st.synchronize()
        assert layer.launch_count() > 0
        assert np.array_equal(from_dev(dout, np.uint16).reshape(16, -1), out_h)
    finally:
        layer.close()


def test_forward_is_deterministic(oracle_mod):
    spec = synth.cfg2_gptoss()
    host = synth.make_layer(spec, 0)
    x = synth.make_tokens(32, spec.hidden, 0)
    layer = MoELayer(host, 32)
    try:
        a, _ = layer.forward_host(x)
        b, _ = layer.forward_host(x)
    finally:
        layer.close()
    assert np.array_equal(a, b)


def test_cfg3_full_prefill_sampled_tokens(oracle_mod):
    """Full 2048-token prefill: routing checked for every token, outputs for a token sample."""
    spec = synth.cfg3_qwen()
    mask = np.zeros(2048, dtype=np.uint8)
    mask[np.random.default_rng(0).choice(2048, size=64, replace=False)] = 1
    run_and_check(oracle_mod, spec, 2048, token_mask=mask)


# ── the tcgen05 grouped-GEMM path (forced), same oracle, same tolerances ──

TC = 2  # option "path": tensor-core grouped GEMM whenever possible


@pytest.mark.parametrize("T", [1, 16, 17, 300])
def test_tc_cfg1_shape(oracle_mod, T):
    run_and_check(oracle_mod, synth.cfg1_tiny(), T, path=TC)


@pytest.mark.parametrize("T", [8, 64])
def test_tc_cfg2_decode(oracle_mod, T):
    run_and_check(oracle_mod, synth.cfg2_gptoss(), T, path=TC)


def test_tc_cfg2_row_bias_residual(oracle_mod):
    run_and_check(oracle_mod, synth.cfg2_gptoss().with_(expert_row_bias=1), 40, residual=True, path=TC)


def test_tc_cfg3_small(oracle_mod):
    run_and_check(oracle_mod, synth.cfg3_qwen(), 200, path=TC)


def test_tc_cfg3_full_prefill_sampled(oracle_mod):
    mask = np.zeros(2048, dtype=np.uint8)
    mask[np.random.default_rng(1).choice(2048, size=64, replace=False)] = 1
    run_and_check(oracle_mod, synth.cfg3_qwen(), 2048, token_mask=mask, path=TC)


@pytest.mark.parametrize("tc_weights", [1, 2])
def test_tc_cfg3_full_prefill_one_weight_source(oracle_mod, tc_weights):
    """The same prefill with both grouped GEMMs dequantising the packed weights themselves (1) or both reading
    the bf16 weight cache (2); the automatic choice at this size is packed gate/up and cached down."""
    mask = np.zeros(2048, dtype=np.uint8)
    mask[np.random.default_rng(2).choice(2048, size=64, replace=False)] = 1
    run_and_check(oracle_mod, synth.cfg3_qwen(), 2048, token_mask=mask, path=TC, options={"tc_weights": tc_weights})


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
def test_tc_bf16_weight_cache_any_bit_width(oracle_mod, bits):
    """With the cache the tensor-core path takes every bit width: the experts are expanded once."""
    spec = synth.LayerSpec(f"cache_bits{bits}", 512, 256, 16, 4, expert_bits=bits, prefill_weight_cache=2)
    run_and_check(oracle_mod, spec, 300, path=TC)
    run_and_check(oracle_mod, spec, 300)          # automatic choice


def test_tc_weight_cache_with_ragged_row_blocks(oracle_mod):
    """2880 output rows are 22.5 blocks of 128: the tile-major cache pads the last block of gate/up with zero
    rows and gives down an even block count; both weight sources must still give the same bits."""
    spec = synth.cfg2_gptoss().with_(prefill_weight_cache=2, expert_row_bias=1)
    host = synth.make_layer(spec, 9)
    x = synth.make_tokens(600, spec.hidden, 9)
    layer = MoELayer(host, 600)
    try:
        layer.set_option("path", TC)
        layer.set_option("tc_weights", 2)
        cached, _ = layer.forward_host(x)
        layer.set_option("tc_weights", 1)
        packed, _ = layer.forward_host(x)
    finally:
        layer.close()
    assert np.array_equal(cached, packed)
    run_and_check(oracle_mod, spec, 600, seed=9, host=host, path=TC, options={"tc_weights": 2})


def test_tc_cache_and_packed_weights_agree(oracle_mod):
    spec = synth.LayerSpec("cache_vs_packed", 512, 256, 16, 4, prefill_weight_cache=2)
    host = synth.make_layer(spec, 3)
    x = synth.make_tokens(400, spec.hidden, 3)
    layer = MoELayer(host, 400)
    try:
        layer.set_option("path", TC)
        layer.set_option("tc_weights", 2)
        a, _ = layer.forward_host(x)
        layer.set_option("tc_weights", 1)
        b, _ = layer.forward_host(x)
        layer.set_option("tc_weights", 0)   # automatic: packed gate/up, cached down at this size
        c, _ = layer.forward_host(x)
    finally:
        layer.close()
    # both round fma(q, scale, bias) to bf16 once and run the same MMA sequence
    assert np.array_equal(a, b)
    assert np.array_equal(a, c)


def test_host_entry_in_chunks_gives_the_same_bits(oracle_mod):
    """A large batch through the host entry point is cut into chunks whose copies overlap the compute; tokens
    are independent, so the output equals the uncut call bit for bit (with a residual and the router's own rows
    too), and a sample of tokens agrees with the oracle."""
    spec = synth.LayerSpec("host_chunks", 512, 256, 16, 4, prefill_weight_cache=2)
    host = synth.make_layer(spec, 5)
    T = 4608 + 77                      # two chunks, the second one ragged
    x = synth.make_tokens(T, spec.hidden, 5)
    res = synth.make_tokens(T, spec.hidden, 6)
    layer = MoELayer(host, T)
    try:
        cut, _ = layer.forward_host(x, residual=res)
        cut_split, _ = layer.forward_host(x, residual=res, x_router=x)
        layer.set_option("host_chunks", 1)
        whole, _ = layer.forward_host(x, residual=res)
    finally:
        layer.close()
    assert np.array_equal(cut, whole)
    assert np.array_equal(cut_split, whole)
    mask = np.zeros(T, dtype=np.uint8)
    mask[np.random.default_rng(3).choice(T, size=48, replace=False)] = 1
    ref = oracle_mod.moe_forward(host, x, residual=res, token_mask=mask)
    sel = np.nonzero(mask)[0]
    assert_parity(cut[sel], ref.out_f32[sel], 5e-3, 2e-2, what=spec.name)


@pytest.mark.parametrize("gs", [32, 128])
def test_tc_group_sizes(oracle_mod, gs):
    run_and_check(oracle_mod, synth.LayerSpec(f"tc_gs{gs}", 512, 256, 8, 2, expert_group_size=gs), 150, path=TC)


def test_tc_skewed_many_token_tiles(oracle_mod):
    """One hot expert receives several 128-row token tiles; cold experts receive none."""
    spec = synth.LayerSpec("tc_skew", 512, 256, 64, 8, router_has_bias=1, zipf_s=1.1, zipf_strength=2.0)
    run_and_check(oracle_mod, spec, 700, path=TC)


def test_tc_shared_expert_4bit(oracle_mod):
    spec = synth.LayerSpec("tc_shared", 512, 256, 16, 4, shared_intermediate=256, shared_bits=4, shared_group_size=64,
                           shared_gate_kind=capi.LINEAR_BF16)
    run_and_check(oracle_mod, spec, 130, path=TC)
    run_and_check(oracle_mod, spec, 9, path=TC)


def test_tc_and_gemv_paths_agree_on_routing_and_nearly_on_values(oracle_mod):
    spec = synth.cfg3_qwen()
    host = synth.make_layer(spec, 0)
    x = synth.make_tokens(64, spec.hidden, 0)
    layer = MoELayer(host, 64)
    try:
        layer.set_option("path", 1)
        a, da = layer.forward_host(x, debug=True)
        layer.set_option("path", 2)
        b, db = layer.forward_host(x, debug=True)
        c, _ = layer.forward_host(x)
    finally:
        layer.close()
    assert np.array_equal(da.indices, db.indices) and np.array_equal(da.perm, db.perm)
    assert np.array_equal(b, c)                       # the tensor-core path is deterministic too
    fa, fb = synth.bf16_to_f32(a).astype(np.float64), synth.bf16_to_f32(b).astype(np.float64)
    assert np.sqrt(((fa - fb) ** 2).mean()) / np.sqrt((fa ** 2).mean()) < 5e-3


# ── the register-streaming decode kernels (forced), same oracle, same tolerances ──

MMA = 3  # option "path": per-warp streaming mma.sync kernels


@pytest.mark.parametrize("T", [1, 2, 8, 9, 32, 64])
def test_mma_cfg2_decode(oracle_mod, T):
    run_and_check(oracle_mod, synth.cfg2_gptoss(), T, path=MMA)


def test_mma_cfg2_row_bias_residual(oracle_mod):
    run_and_check(oracle_mod, synth.cfg2_gptoss().with_(expert_row_bias=1), 21, residual=True, path=MMA)


@pytest.mark.parametrize("T", [1, 16, 40])
def test_mma_cfg1_and_cfg3_shapes(oracle_mod, T):
    run_and_check(oracle_mod, synth.cfg1_tiny(), T, path=MMA)
    run_and_check(oracle_mod, synth.cfg3_qwen(), T, path=MMA)


def test_mma_group_size_128_and_many_rows_per_expert(oracle_mod):
    # 70 tokens over 8 experts: several passes of 8/16 activation rows per expert
    run_and_check(oracle_mod, synth.LayerSpec("mma_gs128", 512, 256, 8, 2, expert_group_size=128), 70, path=MMA)
    run_and_check(oracle_mod, synth.LayerSpec("mma_small", 64, 64, 4, 2), 5, path=MMA)


@pytest.mark.parametrize("T", [1, 4, 8, 20, 64])
def test_mma_group_size_32_gptoss_as_transcoded(oracle_mod, T):
    """GPT-OSS experts as the MXFP4 transcode leaves them: 4-bit, group 32, row biases; both pass widths."""
    spec = synth.cfg2_gptoss().with_(name="gptoss_gs32", expert_group_size=32, expert_row_bias=1)
    run_and_check(oracle_mod, spec, T, path=MMA)
    run_and_check(oracle_mod, spec, T)                      # the automatic choice takes the same kernels


def test_mma_group_size_32_small_shapes(oracle_mod):
    run_and_check(oracle_mod, synth.LayerSpec("mma_gs32", 512, 256, 8, 2, expert_group_size=32), 70, path=MMA)
    run_and_check(oracle_mod, synth.LayerSpec("mma_gs32_small", 64, 64, 4, 2, expert_group_size=32), 5, path=MMA)
    run_and_check(oracle_mod, synth.LayerSpec("mma_gs32_odd_runs", 320, 192, 4, 2, expert_group_size=32), 11, path=MMA)


@pytest.mark.parametrize("ksplit", [1, 2, 4])
@pytest.mark.parametrize("gs", [32, 64])
def test_mma_every_reduction_split(oracle_mod, ksplit, gs):
    """The reduction axis cut into 1, 2 or 4 slices per 16-row block (the automatic choice only splits the
    smallest batches), for both scale layouts, with one and with several rows per expert."""
    spec = synth.cfg2_gptoss().with_(name=f"split{ksplit}_gs{gs}", expert_group_size=gs)
    for T in (1, 3, 24):
        run_and_check(oracle_mod, spec, T, path=MMA, options={"ksplit": ksplit})


def test_auto_path_is_deterministic_and_matches_forced_paths(oracle_mod):
    spec = synth.cfg2_gptoss()
    host = synth.make_layer(spec, 0)
    x = synth.make_tokens(8, spec.hidden, 0)
    layer = MoELayer(host, 8)
    try:
        a, _ = layer.forward_host(x)
        b, _ = layer.forward_host(x)
        layer.set_option("path", MMA)
        c, _ = layer.forward_host(x)
    finally:
        layer.close()
    assert np.array_equal(a, b) and np.array_equal(a, c)   # small batches take the streaming kernels


# ── Gemma-4-style routing: scaled logits, per-expert combine scale, GELU-GLU, the router's own input ──

@pytest.mark.parametrize("T,path", [(1, None), (6, None), (40, None), (150, None), (300, 2), (9, 1)])
def test_gemma4_style_block(oracle_mod, T, path):
    spec = synth.gemma4_style()
    host = synth.make_layer(spec, 4)
    x = synth.make_tokens(T, spec.hidden, 4)
    xr = synth.make_tokens(T, spec.hidden, 40)          # stands for rmsNorm(h, router.scale)
    layer = MoELayer(host, T)
    try:
        if path is not None:
            layer.set_option("path", path)
        out, dbg = layer.forward_host(x, debug=True, x_router=xr)
        same, _ = layer.forward_host(x, x_router=xr)
        plain, pdbg = layer.forward_host(x, debug=True)           # router reading x: a different routing
    finally:
        layer.close()
    ref = oracle_mod.moe_forward(host, x, x_router=xr)
    assert np.array_equal(dbg.indices, ref.indices) and np.array_equal(dbg.weights, ref.weights)
    assert np.array_equal(dbg.perm, ref.perm) and np.array_equal(out, same)
    assert_parity(out, ref.out_f32, what=spec.name)
    ref_plain = oracle_mod.moe_forward(host, x)
    assert np.array_equal(pdbg.indices, ref_plain.indices) and np.array_equal(pdbg.weights, ref_plain.weights)
    # the per-expert scale really is in the weights: they no longer sum to one
    assert np.abs(ref.weights.sum(axis=1) - 1.0).max() > 1e-2


# ── the remaining benchmark configurations at their full sizes (outputs on a token sample: the oracle is scalar) ──

def test_cfg4_full_prefill_sampled(oracle_mod):
    """256 experts, top-8, sigmoid-gated 8-bit shared expert, 8-bit router, 2048 tokens: routing and
    the plan for every token, outputs for 48 sampled tokens."""
    mask = np.zeros(2048, dtype=np.uint8)
    mask[np.random.default_rng(4).choice(2048, size=48, replace=False)] = 1
    run_and_check(oracle_mod, synth.cfg4_shared(), 2048, token_mask=mask)


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
def test_cfg5_skewed_routing_every_bit_width(oracle_mod, bits):
    """cfg3 shape with a Zipf(1.1) router bias (a few hot experts with many token tiles, most experts
    nearly empty) at every bit width; 1024 tokens, outputs for 32 sampled tokens."""
    mask = np.zeros(1024, dtype=np.uint8)
    mask[np.random.default_rng(bits).choice(1024, size=32, replace=False)] = 1
    run_and_check(oracle_mod, synth.cfg5_skewed(bits), 1024, token_mask=mask)


def test_cfg4_at_its_full_size(oracle_mod):
    """The 256-expert configuration at its 8192 tokens (65536 routed rows: the dispatch plan takes its
    count / scan / scatter form): routing and plan for every token, outputs for 32 sampled tokens."""
    mask = np.zeros(8192, dtype=np.uint8)
    mask[np.random.default_rng(44).choice(8192, size=32, replace=False)] = 1
    run_and_check(oracle_mod, synth.cfg4_shared(), 8192, token_mask=mask)


def test_cfg5_at_its_full_size_with_requantized_experts(oracle_mod):
    """The skewed configuration as it is described: the 4-bit layer of the cfg3 shape, its experts
    re-quantised at another width (5 bits here) from their dequantised values, Zipf router bias, 16384
    tokens (131072 routed rows); routing and plan for every token, outputs for 32 sampled tokens."""
    base = synth.make_layer(synth.cfg5_skewed(4), 0)
    host = synth.requantize_experts(base, 5)
    assert host.spec.expert_bits == 5
    mask = np.zeros(16384, dtype=np.uint8)
    mask[np.random.default_rng(55).choice(16384, size=32, replace=False)] = 1
    run_and_check(oracle_mod, host.spec, 16384, host=host, token_mask=mask)


# ── NemotronH-style block: sigmoid routing with selection bias and scaling factor, experts without a gate projection ──

@pytest.mark.parametrize("T", [1, 7, 64, 300])
def test_nemotronh_style_block(oracle_mod, T):
    spec = synth.nemotronh_style()
    run_and_check(oracle_mod, spec, T, seed=6, residual=(T == 7))


def test_nemotronh_style_block_other_widths(oracle_mod):
    run_and_check(oracle_mod, synth.nemotronh_style().with_(name="nemotronh_8bit", expert_bits=8, shared_bits=8, norm_topk_prob=0), 33)
    run_and_check(oracle_mod, synth.nemotronh_style().with_(name="nemotronh_no_shared", shared_intermediate=0, top_k=1), 20)
