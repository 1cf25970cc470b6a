"""The committed vectors of tests/golden/moe_golden.npz: the oracle must reproduce them bit for bit
(CPU), and the CUDA path must meet them through the C ABI (GPU): routing and the plan exactly, outputs
within the parity gate, weight preparation exactly."""
import importlib.util
import os

import numpy as np
import pytest

from ffai_b200 import capi, synth
from helpers import assert_parity, from_dev, to_dev

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)


@pytest.fixture(scope="module")
def golden():
    return dict(np.load(os.path.join(HERE, "golden", "moe_golden.npz")))


def test_oracle_reproduces_the_committed_vectors(oracle_mod, golden):
    fresh = make_golden.build()
    assert sorted(fresh) == sorted(golden)
    for k in golden:
        assert golden[k].dtype == fresh[k].dtype and np.array_equal(golden[k], fresh[k]), k


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(make_golden.cases()))
def test_cuda_layer_meets_the_committed_vectors(ffai_lib, golden, name):
    from ffai_b200.moe import MoELayer
    spec, T, seed, with_res = make_golden.cases()[name]
    host = synth.make_layer(spec, seed)
    x = synth.make_tokens(T, spec.hidden, seed)
    res = synth.make_tokens(T, spec.hidden, seed + 17) if with_res else None
    xr = synth.make_tokens(T, spec.hidden, seed + 40) if spec.name.startswith("gemma") else None
    layer = MoELayer(host, T)
    try:
        out, dbg = layer.forward_host(x, residual=res, debug=True, x_router=xr)
    finally:
        layer.close()
    assert np.array_equal(dbg.indices, golden[f"{name}/indices"])
    assert np.array_equal(dbg.weights, golden[f"{name}/weights"])
    assert np.array_equal(dbg.logits, golden[f"{name}/logits"])
    assert np.array_equal(dbg.perm, golden[f"{name}/perm"]) and np.array_equal(dbg.offsets, golden[f"{name}/offsets"])
    assert_parity(out, golden[f"{name}/out_f32"], what=name)


@pytest.mark.gpu
def test_cuda_weight_preparation_meets_the_committed_vectors(ffai_lib, golden):
    import torch
    packed, e8m0 = make_golden.mxfp4_case()
    n = e8m0.size
    dp, de = to_dev(packed.reshape(-1)), to_dev(e8m0)
    ow = torch.zeros(n * 16, dtype=torch.uint8, device="cuda")
    osc = torch.zeros(n, dtype=torch.int16, device="cuda")
    obi = torch.zeros(n, dtype=torch.int16, device="cuda")
    capi.check(ffai_lib.ffai_op_mxfp4_to_affine_int4(dp.data_ptr(), de.data_ptr(), n, ow.data_ptr(), osc.data_ptr(), obi.data_ptr(), None), "transcode")
    torch.cuda.synchronize()
    assert np.array_equal(from_dev(ow, np.uint8).reshape(n, 16), golden["mxfp4/codes"])
    assert np.array_equal(from_dev(osc, np.uint16), golden["mxfp4/scales"]) and np.array_equal(from_dev(obi, np.uint16), golden["mxfp4/biases"])
    wq = make_golden.quant_case()
    rows, K = wq.shape
    dwq = to_dev(wq.reshape(-1))
    for bits in (3, 4, 8):
        pw = torch.zeros(rows * K * bits // 32, dtype=torch.int32, device="cuda")
        ps = torch.zeros(rows * K // 64, dtype=torch.int16, device="cuda")
        pb = torch.zeros(rows * K // 64, dtype=torch.int16, device="cuda")
        capi.check(ffai_lib.ffai_op_affine_quantize(dwq.data_ptr(), rows, K, bits, 64, pw.data_ptr(), ps.data_ptr(), pb.data_ptr(), None), "quantize")
        torch.cuda.synchronize()
        assert np.array_equal(from_dev(pw, np.uint32).reshape(golden[f"quant{bits}/codes"].shape), golden[f"quant{bits}/codes"])
        assert np.array_equal(from_dev(ps, np.uint16).reshape(golden[f"quant{bits}/scales"].shape), golden[f"quant{bits}/scales"])
        assert np.array_equal(from_dev(pb, np.uint16).reshape(golden[f"quant{bits}/biases"].shape), golden[f"quant{bits}/biases"])
