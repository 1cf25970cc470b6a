"""Expert-parallel plumbing over the C ABI: NCCL communicator setup and the host-side exchange plan.

Tokens stay data-parallel; rank ``r`` of ``W`` owns the contiguous experts ``[r*E/W, (r+1)*E/W)``.
The library does the exchange itself (``ffai_moe_forward`` with ``ep_world > 1``); this module only
creates the communicator it needs and exposes the plan function for host-side tests.  FFAI itself
is single-device (its dispatch is a host sort plus one gather, ``MoELayer.swift:752-774``).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict

import numpy as np

from . import capi


def unique_id() -> bytes:
    """128 opaque bytes made on one rank and handed to all (any transport)."""
    buf = (C.c_uint8 * 128)()
    capi.check(capi.load().ffai_ep_get_unique_id(buf), "ffai_ep_get_unique_id")
    return bytes(buf)


def comm_create(uid: bytes, rank: int, world: int) -> C.c_void_p:
    """Collective over all ranks; the calling thread's current CUDA device is the rank's GPU."""
    if len(uid) != 128:
        raise ValueError("unique id must be 128 bytes")
    buf = (C.c_uint8 * 128).from_buffer_copy(uid)
    comm = C.c_void_p()
    capi.check(capi.load().ffai_ep_comm_create(buf, rank, world, C.byref(comm)), "ffai_ep_comm_create")
    return comm


def comm_destroy(comm: C.c_void_p) -> None:
    if comm:
        capi.check(capi.load().ffai_ep_comm_destroy(comm), "ffai_ep_comm_destroy")


def comm_from_store(store, rank: int, world: int, key: str = "ffai_ep_uid") -> C.c_void_p:
    """Communicator whose id travels through a ``torch.distributed`` key-value store."""
    if rank == 0:
        store.set(key, unique_id())
    return comm_create(bytes(store.get(key)), rank, world)


def plan_exchange(recv_counts: np.ndarray) -> Dict[str, np.ndarray]:
    """Plan of one exchange from ``recv_counts[world, e_local]`` (rows per source rank and local
    expert).  Pure integer work inside the library; needs no GPU."""
    rc = np.ascontiguousarray(recv_counts, dtype=np.uint32)
    world, e_local = rc.shape
    rank_offsets = np.zeros(world + 1, dtype=np.uint32)
    local_offsets = np.zeros(e_local + 1, dtype=np.uint32)
    seg_src = np.zeros((world, e_local), dtype=np.uint32)
    seg_dst = np.zeros((world, e_local), dtype=np.uint32)
    n = capi.load().ffai_ep_plan_exchange(rc.ctypes.data, world, e_local, rank_offsets.ctypes.data,
                                          local_offsets.ctypes.data, seg_src.ctypes.data, seg_dst.ctypes.data)
    return {"n_rows": int(n), "rank_offsets": rank_offsets, "local_offsets": local_offsets,
            "seg_src": seg_src, "seg_dst": seg_dst}


def peer_layout(counts_matrix: np.ndarray, rank: int) -> Dict[str, np.ndarray]:
    """Layout of the peer-memory exchange for one rank from ``counts_matrix[world, n_experts]`` (the code the
    device kernel runs, on the host)."""
    m = np.ascontiguousarray(counts_matrix, dtype=np.uint32)
    world, n_experts = m.shape
    local = np.zeros(n_experts // world + 1, dtype=np.uint32)
    base = np.zeros(n_experts, dtype=np.uint32)
    capi.check(capi.load().ffai_ep_peer_layout(m.ctypes.data, world, n_experts, rank, local.ctypes.data, base.ctypes.data),
               "ffai_ep_peer_layout")
    return {"local_offsets": local, "send_base": base}
