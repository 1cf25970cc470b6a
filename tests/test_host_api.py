"""Host-side checks that need no GPU: the library loads, exports every declared symbol,
the ctypes mirror matches the C header, and argument validation maps the reference's
preconditions to status codes."""
import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from ffai_b200 import capi, synth

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "ffai_cuda.h"


def declared_functions():
    text = HEADER.read_text()
    return re.findall(r"FFAI_API\s+[\w\s\*]+?\b(ffai_\w+)\s*\(", text)


def test_header_declares_and_library_exports_the_same_symbols(ffai_lib):
    names = declared_functions()
    assert len(names) >= 20
    assert sorted(names) == sorted(capi.SIGNATURES)
    for n in names:
        assert hasattr(ffai_lib, n), f"{n} is declared in the header but not exported"
    assert ffai_lib.ffai_cuda_abi_version() == 1


def test_struct_layout_matches_header(tmp_path):
    src = tmp_path / "sz.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "ffai_cuda.h"\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu %zu %zu\\n\", sizeof(ffai_moe_config), sizeof(ffai_moe_weights),"
        " sizeof(ffai_moe_debug), offsetof(ffai_moe_config, max_tokens), offsetof(ffai_moe_weights, gate_proj),"
        " offsetof(ffai_moe_weights, shared_gate), offsetof(ffai_moe_config, swiglu_limit));return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", str(HEADER.parent), "-o", str(exe), str(src)], check=True)
    got = list(map(int, subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()))
    want = [C.sizeof(capi.MoEConfig), C.sizeof(capi.MoEWeights), C.sizeof(capi.MoEDebug),
            capi.MoEConfig.max_tokens.offset, capi.MoEWeights.gate_proj.offset,
            capi.MoEWeights.shared_gate.offset, capi.MoEConfig.swiglu_limit.offset]
    assert got == want


def test_header_compiles_as_c_and_cpp(tmp_path):
    for lang, comp in (("c", "gcc"), ("c++", "g++")):
        subprocess.run([comp, "-x", lang, "-fsyntax-only", "-Wall", "-Werror", str(HEADER)], check=True)


def _create(lib, cfg):
    h = C.c_void_p()
    rc = lib.ffai_moe_create(C.byref(cfg), C.byref(h))
    msg = lib.ffai_moe_last_error(h).decode() if h else ""
    if h:
        lib.ffai_moe_destroy(h)
    return rc, msg


@pytest.mark.parametrize("field,value", [
    ("top_k", 0), ("top_k", 9), ("n_experts", 0), ("hidden", 100), ("intermediate", 0),
    ("expert_bits", 7), ("expert_group_size", 48), ("gating_mode", 5), ("max_tokens", 0),
    ("struct_size", 4), ("activation", 9), ("router_kind", 0),
])
def test_create_rejects_what_the_reference_traps_on(ffai_lib, field, value):
    """MoERouter.init preconditions (MoELayer.swift:109-118) and the quantized-op shape
    guards (Ops.swift:4588-4615) become FFAI_ERR_INVALID_ARG, with a message."""
    cfg = synth.cfg1_tiny().to_config(max_tokens=16)
    setattr(cfg, field, value)
    rc, msg = _create(ffai_lib, cfg)
    assert rc == capi.FFAI_ERR_INVALID_ARG
    assert msg


def test_null_arguments(ffai_lib):
    assert ffai_lib.ffai_moe_create(None, None) == capi.FFAI_ERR_INVALID_ARG
    assert ffai_lib.ffai_moe_destroy(None) == capi.FFAI_OK
    assert ffai_lib.ffai_moe_forward(None, None, 1, None, None, None, None) == capi.FFAI_ERR_INVALID_ARG
    assert ffai_lib.ffai_op_dequant_gemv(None, None, None, None, None, 1, 64, 4, 64, None) == capi.FFAI_ERR_INVALID_ARG
    assert ffai_lib.ffai_status_string(capi.FFAI_ERR_INVALID_ARG) == b"invalid argument"


def test_op_shape_guards(ffai_lib):
    one = C.c_void_p(16)  # non-null, never dereferenced: validation fails first
    # in_dim not a multiple of 32 (Ops.swift:4610-4615), bad bit width, bad group size
    assert ffai_lib.ffai_op_dequant_gemv(one, one, one, one, one, 4, 40, 4, 64, None) == capi.FFAI_ERR_INVALID_ARG
    assert ffai_lib.ffai_op_dequant_gemv(one, one, one, one, one, 4, 64, 7, 64, None) == capi.FFAI_ERR_INVALID_ARG
    assert ffai_lib.ffai_op_dequant_gemv(one, one, one, one, one, 4, 64, 4, 48, None) == capi.FFAI_ERR_INVALID_ARG
    assert ffai_lib.ffai_op_moe_router_topk(one, one, one, 1, 4, 5, 0, 1, None, None) == capi.FFAI_ERR_INVALID_ARG
    assert ffai_lib.ffai_op_moe_plan_workspace_bytes(2048, 8) == 2 * 8 * 4


def test_no_cpu_fallback_without_a_device(ffai_lib):
    """Without a CUDA device the product path fails loudly instead of computing on the CPU."""
    if ffai_lib.ffai_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    rc, msg = _create(ffai_lib, synth.cfg1_tiny().to_config(max_tokens=16))
    assert rc == capi.FFAI_ERR_CUDA and "no CPU fallback" in msg
    one = C.c_void_p(16)
    assert ffai_lib.ffai_op_dequant_gemv(one, one, one, one, one, 4, 64, 4, 64, None) == capi.FFAI_ERR_CUDA


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    monkeypatch.setenv("FFAI_CUDA_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(capi, "_lib", None)
    with pytest.raises(FileNotFoundError):
        capi.load()
    monkeypatch.setattr(capi, "_lib", None)


def test_product_package_does_not_touch_the_oracle():
    """Nothing under ffai_b200/ imports, links or opens the oracle."""
    for p in (ROOT / "ffai_b200").rglob("*"):
        if p.suffix in {".py", ".cu", ".cuh", ".h", ".hpp", ".swift"}:
            text = p.read_text()
            assert "moe_oracle" not in text and "import oracle" not in text and "from oracle" not in text, p


def test_synthetic_layer_is_seed_deterministic():
    a = synth.make_layer(synth.cfg1_tiny(), 0).arrays
    b = synth.make_layer(synth.cfg1_tiny(), 0).arrays
    c = synth.make_layer(synth.cfg1_tiny(), 1).arrays
    assert all(np.array_equal(a[k], b[k]) for k in a)
    assert not np.array_equal(a["experts.gate_proj.weight"], c["experts.gate_proj.weight"])
    sc = synth.bf16_to_f32(a["experts.gate_proj.scales"])
    bi = synth.bf16_to_f32(a["experts.gate_proj.biases"])
    assert 0.0049 <= sc.min() and sc.max() <= 0.0201 and -0.101 <= bi.min() and bi.max() <= 0.101


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
def test_minmax_quantizer_round_trip(bits):
    rng = np.random.default_rng(bits)
    w = rng.standard_normal((8, 128)).astype(np.float32) * 0.1
    p, s, b = synth.quantize_minmax(w, bits, 64)
    back = synth.dequantize(p, s, b, bits, 64, 128)
    step = synth.bf16_to_f32(s).max()
    assert np.abs(back - w).max() <= 0.75 * step + 2e-3
