"""ctypes view of ``include/ffai_cuda.h`` and the loader for ``libffai_cuda.so``.

The structures below mirror the C header field for field.  The loader never
substitutes anything for a missing library: if the shared object is absent the
import of :func:`load` raises, and every compute entry point of the library
itself returns ``FFAI_ERR_CUDA`` when no CUDA device is present.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libffai_cuda.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

FFAI_OK = 0
FFAI_ERR_INVALID_ARG = 1
FFAI_ERR_UNSUPPORTED = 2
FFAI_ERR_CUDA = 3
FFAI_ERR_NOT_READY = 4
FFAI_ERR_NCCL = 5
FFAI_ERR_DEVICE_CHECK = 6

GATING_SOFTMAX_THEN_TOPK = 0
GATING_TOPK_THEN_SOFTMAX = 1
GATING_SIGMOID_TOPK = 2

ACT_SWIGLU = 0
ACT_CLAMPED_SWIGLU = 1
ACT_GELU_GLU = 2
ACT_RELU2 = 3

LINEAR_NONE = 0
LINEAR_F32 = 1
LINEAR_BF16 = 2
LINEAR_AFFINE = 3

MEM_HOST = 0
MEM_DEVICE = 1

EP_EXPORT_BYTES = 192
N_STAGES = 8
STAGE_NAMES = ("router", "plan", "gather", "gate_up", "down", "combine", "shared", "exchange")
MAX_TOP_K = 32


class MoEConfig(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("hidden", C.c_int32),
        ("intermediate", C.c_int32),
        ("n_experts", C.c_int32),
        ("top_k", C.c_int32),
        ("gating_mode", C.c_int32),
        ("norm_topk_prob", C.c_int32),
        ("router_expert_bias", C.c_int32),
        ("activation", C.c_int32),
        ("swiglu_limit", C.c_float),
        ("swiglu_alpha", C.c_float),
        ("router_kind", C.c_int32),
        ("router_bits", C.c_int32),
        ("router_group_size", C.c_int32),
        ("router_has_bias", C.c_int32),
        ("router_logits_bf16", C.c_int32),
        ("expert_bits", C.c_int32),
        ("expert_group_size", C.c_int32),
        ("expert_row_bias", C.c_int32),
        ("shared_intermediate", C.c_int32),
        ("shared_bits", C.c_int32),
        ("shared_group_size", C.c_int32),
        ("shared_gate_kind", C.c_int32),
        ("shared_gate_bits", C.c_int32),
        ("shared_gate_group_size", C.c_int32),
        ("max_tokens", C.c_int32),
        ("ep_rank", C.c_int32),
        ("ep_world", C.c_int32),
        ("prefill_weight_cache", C.c_int32),
        ("router_logit_scale", C.c_float),
        ("routed_scaling_factor", C.c_float),
        ("reserved", C.c_int32 * 5),
    ]

    def __init__(self, **kw):
        super().__init__(**kw)
        self.struct_size = C.sizeof(MoEConfig)


class QProj(C.Structure):
    _fields_ = [
        ("weight", C.c_void_p),
        ("scales", C.c_void_p),
        ("biases", C.c_void_p),
        ("row_bias", C.c_void_p),
    ]


class Linear(C.Structure):
    _fields_ = [
        ("weight", C.c_void_p),
        ("scales", C.c_void_p),
        ("biases", C.c_void_p),
        ("bias", C.c_void_p),
    ]


class MoEWeights(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("location", C.c_int32),
        ("router", Linear),
        ("router_expert_bias", C.c_void_p),
        ("gate_proj", QProj),
        ("up_proj", QProj),
        ("down_proj", QProj),
        ("shared_gate_proj", QProj),
        ("shared_up_proj", QProj),
        ("shared_down_proj", QProj),
        ("shared_gate", Linear),
        ("router_per_expert_scale", C.c_void_p),
    ]

    def __init__(self, **kw):
        super().__init__(**kw)
        self.struct_size = C.sizeof(MoEWeights)


class MoEDebug(C.Structure):
    _fields_ = [
        ("indices", C.c_void_p),
        ("weights", C.c_void_p),
        ("logits", C.c_void_p),
        ("counts", C.c_void_p),
        ("offsets", C.c_void_p),
        ("perm", C.c_void_p),
        ("inv_perm", C.c_void_p),
    ]


# name -> (restype, argtypes); the set of names is also what the symbol-export test checks
# against the declarations in include/ffai_cuda.h.
_P = C.c_void_p
_I = C.c_int32
SIGNATURES = {
    "ffai_cuda_abi_version": (C.c_int, []),
    "ffai_cuda_device_count": (C.c_int, []),
    "ffai_status_string": (C.c_char_p, [C.c_int]),
    "ffai_moe_create": (C.c_int, [C.POINTER(MoEConfig), C.POINTER(_P)]),
    "ffai_moe_set_weights": (C.c_int, [_P, C.POINTER(MoEWeights)]),
    "ffai_moe_destroy": (C.c_int, [_P]),
    "ffai_moe_last_error": (C.c_char_p, [_P]),
    "ffai_moe_forward": (C.c_int, [_P, _P, _I, _P, _P, C.POINTER(MoEDebug), _P]),
    "ffai_moe_forward_split": (C.c_int, [_P, _P, _P, _I, _P, _P, _P, _P]),
    "ffai_moe_forward_host_split": (C.c_int, [_P, _P, _P, _I, _P, _P, _P]),
    "ffai_moe_forward_split": (C.c_int, [_P, _P, _P, _I, _P, _P, C.POINTER(MoEDebug), _P]),
    "ffai_moe_forward_host_split": (C.c_int, [_P, _P, _P, _I, _P, _P, C.POINTER(MoEDebug)]),
    "ffai_moe_forward_host": (C.c_int, [_P, _P, _I, _P, _P, C.POINTER(MoEDebug)]),
    "ffai_moe_set_nccl_comm": (C.c_int, [_P, _P]),
    "ffai_moe_ep_export": (C.c_int, [_P, _P]),
    "ffai_moe_ep_import": (C.c_int, [_P, _P]),
    "ffai_moe_ep_release": (C.c_int, [_P]),
    "ffai_moe_ep_skip_step": (C.c_int, [_P]),
    "ffai_ep_peer_layout": (C.c_int, [_P, _I, _I, _I, _P, _P]),
    "ffai_ep_get_unique_id": (C.c_int, [_P]),
    "ffai_ep_comm_create": (C.c_int, [_P, _I, _I, C.POINTER(_P)]),
    "ffai_ep_comm_destroy": (C.c_int, [_P]),
    "ffai_ep_plan_exchange": (C.c_uint32, [_P, _I, _I, _P, _P, _P, _P]),
    "ffai_moe_set_option": (C.c_int, [_P, C.c_char_p, _I]),
    "ffai_moe_check_device_status": (C.c_int, [_P]),
    "ffai_moe_read_timeline": (C.c_int, [_P, C.POINTER(C.c_int64), _I]),
    "ffai_moe_set_stage_timing": (C.c_int, [_P, C.c_int]),
    "ffai_moe_get_stage_ms": (C.c_int, [_P, C.POINTER(C.c_float * N_STAGES)]),
    "ffai_moe_last_launch_count": (C.c_int, [_P]),
    "ffai_op_dequant_gemv": (C.c_int, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "ffai_op_dequant_gemv_expert_indexed": (C.c_int, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "ffai_op_moe_router_topk": (C.c_int, [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "ffai_op_moe_plan_workspace_bytes": (C.c_size_t, [_I, _I]),
    "ffai_op_moe_plan": (C.c_int, [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "ffai_op_moe_plan_static": (C.c_int, [_P, _I, _I, _I, _P, _P, _P, _P, _P]),
    "ffai_op_gather_rows": (C.c_int, [_P, _P, _P, _I, _I, _P]),
    "ffai_op_moe_gather_dequant_gemm": (C.c_int, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "ffai_op_glu_activation": (C.c_int, [_P, _P, _P, C.c_int64, _I, C.c_float, C.c_float, _P]),
    "ffai_op_moe_unpermute": (C.c_int, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "ffai_st_open": (C.c_int, [C.c_char_p, C.POINTER(_P)]),
    "ffai_st_close": (None, [_P]),
    "ffai_st_last_error": (C.c_char_p, [_P]),
    "ffai_st_tensor": (C.c_int, [_P, C.c_char_p, C.POINTER(_P), C.POINTER(C.c_uint64), C.c_char_p, C.POINTER(C.c_int64 * 8), C.POINTER(C.c_int32)]),
    "ffai_st_derive_bits": (C.c_int32, [C.c_int64, C.c_int64, C.c_int32]),
    "ffai_st_moe_weights": (C.c_int, [_P, C.c_char_p, C.c_int32, C.POINTER(MoEConfig), C.POINTER(MoEWeights)]),
    "ffai_op_add_rmsnorm": (C.c_int, [_P, _P, _P, C.c_float, _I, _I, _P, _P, _P]),
    "ffai_op_mxfp4_to_affine_int4": (C.c_int, [_P, _P, C.c_int64, _P, _P, _P, _P]),
    "ffai_op_affine_quantize": (C.c_int, [_P, C.c_int64, _I, _I, _I, _P, _P, _P, _P]),
    "ffai_op_sigmoid_scalar_fma": (C.c_int, [_P, _P, _P, _P, _P, _I, _I, _P]),
}

_lib = None


class FFAICudaError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        super().__init__(f"{where}: status {status}" + (f" ({detail})" if detail else ""))


def load() -> C.CDLL:
    """Load libffai_cuda.so from the package tree and bind every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("FFAI_CUDA_LIB", str(LIB_PATH)))
    if not path.exists():
        raise FileNotFoundError(
            f"{path} is missing: build it with `python -m ffai_b200.build` "
            "(there is no CPU fallback for the MoE block)")
    lib = C.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int, where: str, layer=None) -> None:
    if status == FFAI_OK:
        return
    lib = load()
    detail = lib.ffai_status_string(status).decode()
    if layer:
        msg = lib.ffai_moe_last_error(layer)
        if msg:
            detail += ": " + msg.decode()
    raise FFAICudaError(status, where, detail)
