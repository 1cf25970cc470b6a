"""Python handle over the C ABI of ``libffai_cuda`` (plumbing for tests and the benchmark).

The compute path is entirely inside the shared library; this module only owns the
opaque handle, keeps weight arrays alive and passes pointers.  ``forward_host``
takes numpy arrays (host buffers, copies inside the call); ``forward`` takes
device pointers (e.g. from ``torch.Tensor.data_ptr()``) and a CUDA stream.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import numpy as np

from . import capi
from .synth import HostLayer


class DebugBuffers:
    """Host-side routing/dispatch outputs of one forward call."""

    def __init__(self, n_tokens: int, k: int, n_experts: int):
        self.indices = np.zeros((n_tokens, k), dtype=np.uint32)
        self.weights = np.zeros((n_tokens, k), dtype=np.float32)
        self.logits = np.zeros((n_tokens, n_experts), dtype=np.float32)
        self.counts = np.zeros(n_experts, dtype=np.uint32)
        self.offsets = np.zeros(n_experts + 1, dtype=np.uint32)
        self.perm = np.zeros(n_tokens * k, dtype=np.uint32)
        self.inv_perm = np.zeros(n_tokens * k, dtype=np.uint32)

    def struct(self) -> capi.MoEDebug:
        return capi.MoEDebug(*(a.ctypes.data for a in (self.indices, self.weights, self.logits,
                                                       self.counts, self.offsets, self.perm,
                                                       self.inv_perm)))


class MoELayer:
    """One MoE block on the current CUDA device.

    Mirrors the call surface of FFAI's ``MoELayer`` (``decode`` / ``decodeMany``,
    ``Sources/FFAI/Models/MoELayer.swift:530-534, 677-680``): construct from weights,
    then call forward with ``[T, hidden]`` bf16 rows.
    """

    def __init__(self, host_layer: HostLayer, max_tokens: int, ep_rank: int = 0, ep_world: int = 1,
                 ep_comm: Optional[C.c_void_p] = None):
        """``ep_world > 1`` shards the experts: this rank keeps block ``ep_rank`` of ``E/ep_world``
        experts and ``ep_comm`` (see ``ffai_b200.ep``) carries the two row exchanges."""
        self.lib = capi.load()
        self.spec = host_layer.spec
        self.max_tokens = max_tokens
        self.cfg = self.spec.to_config(max_tokens, ep_rank, ep_world)
        self.handle = C.c_void_p()
        rc = self.lib.ffai_moe_create(C.byref(self.cfg), C.byref(self.handle))
        if rc != capi.FFAI_OK:
            h = self.handle
            self.handle = C.c_void_p()
            try:
                capi.check(rc, "ffai_moe_create", h)
            finally:
                if h:
                    self.lib.ffai_moe_destroy(h)
        w = host_layer.weights_struct(ep_rank, ep_world)
        capi.check(self.lib.ffai_moe_set_weights(self.handle, C.byref(w)), "ffai_moe_set_weights", self.handle)
        if ep_comm is not None:
            capi.check(self.lib.ffai_moe_set_nccl_comm(self.handle, ep_comm), "ffai_moe_set_nccl_comm", self.handle)

    # host buffers in, host buffers out (copies inside the call)
    def forward_host(self, x: np.ndarray, residual: Optional[np.ndarray] = None,
                     debug: bool = False, out: Optional[np.ndarray] = None,
                     x_router: Optional[np.ndarray] = None
                     ) -> Tuple[np.ndarray, Optional[DebugBuffers]]:
        x = np.ascontiguousarray(x, dtype=np.uint16)
        T = int(x.shape[0]) if x.ndim == 2 else 0
        if out is None:
            out = np.zeros((T, self.spec.hidden), dtype=np.uint16)
        dbg = DebugBuffers(T, self.spec.top_k, self.spec.n_experts) if debug else None
        dstruct = dbg.struct() if dbg else None
        res_p = None
        if residual is not None:
            residual = np.ascontiguousarray(residual, dtype=np.uint16)
            res_p = residual.ctypes.data
        if x_router is not None:   # the router reads its own rows (Gemma 4)
            x_router = np.ascontiguousarray(x_router, dtype=np.uint16)
            rc = self.lib.ffai_moe_forward_host_split(self.handle, x.ctypes.data if T else None,
                                                      x_router.ctypes.data if T else None, T,
                                                      out.ctypes.data if T else None, res_p,
                                                      C.byref(dstruct) if dstruct else None)
        else:
            rc = self.lib.ffai_moe_forward_host(self.handle, x.ctypes.data if T else None, T,
                                                out.ctypes.data if T else None, res_p,
                                                C.byref(dstruct) if dstruct else None)
        capi.check(rc, "ffai_moe_forward_host", self.handle)
        return out, dbg

    # device pointers
    def forward_ptr(self, x_ptr: int, n_tokens: int, out_ptr: int, residual_ptr: int = 0,
                    stream: int = 0, debug: Optional[capi.MoEDebug] = None) -> None:
        rc = self.lib.ffai_moe_forward(self.handle, x_ptr, n_tokens, out_ptr, residual_ptr or None,
                                       C.byref(debug) if debug is not None else None, stream or None)
        capi.check(rc, "ffai_moe_forward", self.handle)

    # exchange over peer memory (expert parallelism without NCCL): export, hand every rank's blob to all, import
    def ep_export(self) -> bytes:
        buf = (C.c_uint8 * capi.EP_EXPORT_BYTES)()
        capi.check(self.lib.ffai_moe_ep_export(self.handle, buf), "ffai_moe_ep_export", self.handle)
        return bytes(buf)

    def ep_import(self, blobs) -> None:
        joined = b"".join(blobs)
        buf = (C.c_uint8 * len(joined)).from_buffer_copy(joined)
        capi.check(self.lib.ffai_moe_ep_import(self.handle, buf), "ffai_moe_ep_import", self.handle)

    def ep_release(self) -> None:
        capi.check(self.lib.ffai_moe_ep_release(self.handle), "ffai_moe_ep_release", self.handle)

    def ep_skip_step(self) -> None:
        """This rank sits out one step of the peer-memory exchange (see ``ffai_moe_ep_skip_step``)."""
        capi.check(self.lib.ffai_moe_ep_skip_step(self.handle), "ffai_moe_ep_skip_step", self.handle)

    def set_option(self, name: str, value: int) -> None:
        capi.check(self.lib.ffai_moe_set_option(self.handle, name.encode(), int(value)), "ffai_moe_set_option", self.handle)

    def check_device_status(self) -> None:
        capi.check(self.lib.ffai_moe_check_device_status(self.handle), "ffai_moe_check_device_status", self.handle)

    def set_stage_timing(self, enabled: bool) -> None:
        capi.check(self.lib.ffai_moe_set_stage_timing(self.handle, 1 if enabled else 0), "set_stage_timing", self.handle)

    def stage_ms(self) -> Dict[str, float]:
        arr = (C.c_float * capi.N_STAGES)()
        capi.check(self.lib.ffai_moe_get_stage_ms(self.handle, C.byref(arr)), "get_stage_ms", self.handle)
        return {n: float(arr[i]) for i, n in enumerate(capi.STAGE_NAMES)}

    def launch_count(self) -> int:
        return int(self.lib.ffai_moe_last_launch_count(self.handle))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.ffai_moe_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
