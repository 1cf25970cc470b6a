"""The safetensors -> ffai_moe_weights path of the library (host code), against files written here from
synthetic layers with the tensor names of the reference's checkpoints (Qwen3xText.swift:605-650,
Gemma4Text.swift:540-554)."""
import ctypes as C
import json
import struct

import numpy as np
import pytest

from ffai_b200 import capi, synth

DTYPES = {np.dtype(np.uint32): "U32", np.dtype(np.uint16): "BF16", np.dtype(np.float32): "F32", np.dtype(np.uint8): "U8"}


def write_safetensors(path, tensors, metadata=None):
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, arr in tensors.items():
        a = np.ascontiguousarray(arr)
        header[name] = {"dtype": DTYPES[a.dtype], "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        blobs.append(a.tobytes())
        off += a.nbytes
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def checkpoint_tensors(host, prefix, scheme):
    a = host.arrays
    ex = f"{prefix}.switch_mlp" if scheme == 0 else f"{prefix}.experts.switch_glu"
    router = f"{prefix}.gate" if scheme == 0 else f"{prefix}.router.proj"
    t = {}
    for proj in ("gate_proj", "up_proj", "down_proj"):
        for part in ("weight", "scales", "biases"):
            t[f"{ex}.{proj}.{part}"] = a[f"experts.{proj}.{part}"]
    for part in ("weight", "scales", "biases", "bias"):
        if f"gate.{part}" in a:
            t[f"{router}.{part}"] = a[f"gate.{part}"]
    if "gate.per_expert_scale" in a:
        t[f"{prefix}.router.per_expert_scale"] = a["gate.per_expert_scale"]
    for proj in ("gate_proj", "up_proj", "down_proj"):
        for part in ("weight", "scales", "biases"):
            k = f"shared_expert.{proj}.{part}"
            if k in a:
                t[f"{prefix}.shared_expert.{proj}.{part}"] = a[k][0]     # [out, cols]: not stacked in the file
    for part in ("weight", "scales", "biases"):
        k = f"shared_expert_gate.{part}"
        if k in a:
            t[f"{prefix}.shared_expert_gate.{part}"] = a[k]
    t["model.embed_tokens.weight"] = np.zeros((4, 8), dtype=np.uint16)   # something unrelated in the same file
    return t


def load(lib, path, prefix, scheme, spec):
    h = C.c_void_p()
    assert lib.ffai_st_open(str(path).encode(), C.byref(h)) == capi.FFAI_OK, lib.ffai_st_last_error(h)
    cfg = capi.MoEConfig()
    cfg.expert_group_size = spec.expert_group_size
    cfg.router_group_size = spec.router_group_size
    cfg.shared_group_size = spec.shared_group_size
    cfg.shared_gate_group_size = spec.shared_gate_group_size
    w = capi.MoEWeights()
    rc = lib.ffai_st_moe_weights(h, prefix.encode(), scheme, C.byref(cfg), C.byref(w))
    return h, cfg, w, rc


def bytes_at(ptr, n):
    return C.string_at(ptr, n)


@pytest.mark.parametrize("scheme,spec", [
    (0, synth.cfg4_shared().with_(n_experts=8, hidden=256, intermediate=128, shared_intermediate=128, name="qwen_like")),
    (0, synth.LayerSpec("six_bit", 256, 128, 4, 2, expert_bits=6)),
    (1, synth.gemma4_style().with_(n_experts=8, hidden=256, intermediate=128, name="gemma_like")),
])
def test_moe_weights_from_file(tmp_path, scheme, spec):
    lib = capi.load()
    host = synth.make_layer(spec, 2)
    prefix = "model.layers.3.mlp" if scheme == 0 else "model.layers.3"
    path = tmp_path / "m.safetensors"
    write_safetensors(path, checkpoint_tensors(host, prefix, scheme), metadata={"format": "mlx", "note": "nested {braces} \"quoted\""})
    h, cfg, w, rc = load(lib, path, prefix, scheme, spec)
    try:
        assert rc == capi.FFAI_OK, lib.ffai_st_last_error(h)
        # derived from the shapes alone (Layers.swift:340-363)
        assert (cfg.n_experts, cfg.hidden, cfg.intermediate, cfg.expert_bits) == (spec.n_experts, spec.hidden, spec.intermediate, spec.expert_bits)
        assert (cfg.router_kind, cfg.router_bits) == (spec.router_kind, spec.router_bits)
        assert (cfg.shared_intermediate, cfg.shared_bits) == (spec.shared_intermediate, spec.shared_bits if spec.shared_intermediate else 0)
        assert cfg.shared_gate_kind == spec.shared_gate_kind and cfg.shared_gate_bits == spec.shared_gate_bits
        a = host.arrays
        for proj, q in (("gate_proj", w.gate_proj), ("up_proj", w.up_proj), ("down_proj", w.down_proj)):
            for part, ptr in (("weight", q.weight), ("scales", q.scales), ("biases", q.biases)):
                arr = np.ascontiguousarray(a[f"experts.{proj}.{part}"])
                assert bytes_at(ptr, arr.nbytes) == arr.tobytes(), (proj, part)
        assert bytes_at(w.router.weight, a["gate.weight"].nbytes) == np.ascontiguousarray(a["gate.weight"]).tobytes()
        if spec.router_per_expert_scale:
            assert bytes_at(w.router_per_expert_scale, 4 * spec.n_experts) == a["gate.per_expert_scale"].tobytes()
        if spec.shared_intermediate:
            arr = np.ascontiguousarray(a["shared_expert.down_proj.weight"][0])
            assert bytes_at(w.shared_down_proj.weight, arr.nbytes) == arr.tobytes()
    finally:
        lib.ffai_st_close(h)


def test_tensor_lookup_and_errors(tmp_path):
    lib = capi.load()
    path = tmp_path / "t.safetensors"
    write_safetensors(path, {"a.weight": np.arange(12, dtype=np.float32).reshape(3, 4), "b": np.zeros(5, dtype=np.uint8)})
    h = C.c_void_p()
    assert lib.ffai_st_open(str(path).encode(), C.byref(h)) == capi.FFAI_OK
    data, nbytes, dtype, shape, nd = C.c_void_p(), C.c_uint64(), C.create_string_buffer(8), (C.c_int64 * 8)(), C.c_int32()
    assert lib.ffai_st_tensor(h, b"a.weight", C.byref(data), C.byref(nbytes), dtype, C.byref(shape), C.byref(nd)) == capi.FFAI_OK
    assert (nbytes.value, dtype.value, nd.value, shape[0], shape[1]) == (48, b"F32", 2, 3, 4)
    assert np.frombuffer(bytes_at(data, 48), dtype=np.float32).tolist() == list(range(12))
    assert lib.ffai_st_tensor(h, b"missing", None, None, None, None, None) == capi.FFAI_ERR_INVALID_ARG
    cfg, w = capi.MoEConfig(), capi.MoEWeights()
    cfg.expert_group_size = 64
    assert lib.ffai_st_moe_weights(h, b"model.layers.0.mlp", 0, C.byref(cfg), C.byref(w)) == capi.FFAI_ERR_INVALID_ARG
    assert b"switch_mlp.gate_proj" in lib.ffai_st_last_error(h)
    lib.ffai_st_close(h)
    # truncated file, and a header length that exceeds the file
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    h2 = C.c_void_p()
    assert lib.ffai_st_open(str(bad).encode(), C.byref(h2)) == capi.FFAI_ERR_INVALID_ARG
    lib.ffai_st_close(h2)
    h3 = C.c_void_p()
    assert lib.ffai_st_open(str(tmp_path / "absent.safetensors").encode(), C.byref(h3)) == capi.FFAI_ERR_INVALID_ARG
    lib.ffai_st_close(h3)


def test_derive_bits():
    lib = capi.load()
    # [out, in*bits/32] packed columns against [out, in/gs] scale columns (Layers.swift:348-363)
    for bits in (2, 3, 4, 5, 6, 8):
        for gs in (32, 64, 128):
            assert lib.ffai_st_derive_bits(2048 * bits // 32, 2048 // gs, gs) == bits
    assert lib.ffai_st_derive_bits(100, 3, 64) == 0      # inconsistent shapes
    assert lib.ffai_st_derive_bits(10, 0, 64) == 0


@pytest.mark.gpu
def test_layer_built_from_a_file_matches_the_layer_built_from_arrays(tmp_path, ffai_lib):
    from ffai_b200.moe import MoELayer
    spec = synth.cfg4_shared().with_(n_experts=16, hidden=512, intermediate=256, shared_intermediate=256, name="file_layer")
    host = synth.make_layer(spec, 7)
    x = synth.make_tokens(33, spec.hidden, 7)
    direct = MoELayer(host, 33)
    try:
        want, _ = direct.forward_host(x)
    finally:
        direct.close()
    path = tmp_path / "l.safetensors"
    write_safetensors(path, checkpoint_tensors(host, "model.layers.0.mlp", 0))
    h, cfg, w, rc = load(ffai_lib, path, "model.layers.0.mlp", 0, spec)
    assert rc == capi.FFAI_OK, ffai_lib.ffai_st_last_error(h)
    # what the file cannot say stays the caller's
    cfg.struct_size = C.sizeof(capi.MoEConfig)
    cfg.top_k, cfg.gating_mode, cfg.norm_topk_prob, cfg.activation = spec.top_k, spec.gating_mode, spec.norm_topk_prob, spec.activation
    cfg.router_logits_bf16, cfg.max_tokens, cfg.ep_world = spec.router_logits_bf16, 33, 1
    cfg.swiglu_limit, cfg.swiglu_alpha = spec.swiglu_limit, spec.swiglu_alpha
    layer = C.c_void_p()
    try:
        capi.check(ffai_lib.ffai_moe_create(C.byref(cfg), C.byref(layer)), "create", layer)
        capi.check(ffai_lib.ffai_moe_set_weights(layer, C.byref(w)), "set_weights", layer)
        ffai_lib.ffai_st_close(h)      # set_weights copied everything: the mapping may go
        h = None
        out = np.zeros_like(want)
        capi.check(ffai_lib.ffai_moe_forward_host(layer, x.ctypes.data, 33, out.ctypes.data, None, None), "forward", layer)
        assert np.array_equal(out, want)
    finally:
        if h:
            ffai_lib.ffai_st_close(h)
        if layer:
            ffai_lib.ffai_moe_destroy(layer)


def _open_raw(lib, tmp_path, name, header_bytes, payload=b""):
    path = tmp_path / name
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header_bytes)))
        f.write(header_bytes)
        f.write(payload)
    h = C.c_void_p()
    rc = lib.ffai_st_open(str(path).encode(), C.byref(h))
    msg = lib.ffai_st_last_error(h).decode() if h else ""
    if h:
        lib.ffai_st_close(h)
    return rc, msg


def test_hostile_headers_are_rejected_not_followed(tmp_path):
    """A header may not send a reader past the mapping: a shape larger than its byte range, a negative
    dimension, a number that runs into the end of the file, an escape cut off by it, nesting without end."""
    lib = capi.load()
    # the declared shape needs 4 MiB, the byte range holds 16 bytes
    hdr = json.dumps({"w": {"dtype": "U32", "shape": [64, 128, 128], "data_offsets": [0, 16]}}).encode()
    rc, msg = _open_raw(lib, tmp_path, "short.safetensors", hdr, b"\0" * 16)
    assert rc == capi.FFAI_ERR_INVALID_ARG and "byte range" in msg
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [-4, 2], "data_offsets": [0, 0]}}).encode()
    assert _open_raw(lib, tmp_path, "neg.safetensors", hdr)[0] == capi.FFAI_ERR_INVALID_ARG
    # the header (and the file) ends in the middle of a number
    hdr = b'{"w":{"dtype":"F32","shape":[1],"data_offsets":[0,4'
    assert _open_raw(lib, tmp_path, "digits.safetensors", hdr)[0] == capi.FFAI_ERR_INVALID_ARG
    # ... in the middle of a \u escape inside a name
    assert _open_raw(lib, tmp_path, "escape.safetensors", b'{"w\\u00')[0] == capi.FFAI_ERR_INVALID_ARG
    # ... and metadata nested deeper than any real file
    deep = b'{"__metadata__":' + b"[" * 5000 + b"]" * 5000 + b"}"
    assert _open_raw(lib, tmp_path, "deep.safetensors", deep)[0] == capi.FFAI_ERR_INVALID_ARG
    # a well-formed neighbour still opens
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}).encode()
    assert _open_raw(lib, tmp_path, "fine.safetensors", hdr, b"\0" * 16)[0] == capi.FFAI_OK


def test_truncated_expert_tensor_is_rejected(tmp_path):
    """A stacked projection whose scales tensor was cut short: the file no longer opens."""
    spec = synth.LayerSpec("cut", 256, 128, 4, 2)
    host = synth.make_layer(spec, 1)
    t = checkpoint_tensors(host, "m.mlp", 0)
    path = tmp_path / "cut.safetensors"
    write_safetensors(path, t)
    raw = path.read_bytes()
    hlen = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + hlen])
    name = "m.mlp.switch_mlp.down_proj.scales"
    b, e = header[name]["data_offsets"]
    header[name]["data_offsets"] = [b, b + (e - b) // 2]      # shape unchanged, half the bytes
    hj = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(hj)) + hj + raw[8 + hlen:])
    h = C.c_void_p()
    lib = capi.load()
    assert lib.ffai_st_open(str(path).encode(), C.byref(h)) == capi.FFAI_ERR_INVALID_ARG
    assert name in lib.ffai_st_last_error(h).decode()
    lib.ffai_st_close(h)
