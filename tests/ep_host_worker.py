"""One rank of the expert-parallel protocol on the CPU (gloo), as run by test_ep_host.py.

The row exchange, the regrouping plan (``ffai_ep_plan_exchange`` from the library) and the return
path are the ones the CUDA path uses; the expert arithmetic is the oracle's.  Each rank checks its
own tokens against the single-process oracle with all experts.
usage: ep_host_worker.py <rank> <world> <port> <out.json>
"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import oracle
from ffai_b200 import ep, synth


def all_to_all_rows(send: np.ndarray, send_rows, recv_rows, rank, world):
    """send: [n, w] array; send_rows[d] / recv_rows[s] = rows to rank d / from rank s (in rank order)."""
    width = send.shape[1]
    out = np.zeros((int(sum(recv_rows)), width), dtype=send.dtype)
    s_off = np.concatenate([[0], np.cumsum(send_rows)]).astype(int)
    r_off = np.concatenate([[0], np.cumsum(recv_rows)]).astype(int)
    ops, bufs = [], []
    for peer in range(world):
        if peer == rank:
            out[r_off[peer]:r_off[peer + 1]] = send[s_off[peer]:s_off[peer + 1]]
            continue
        if send_rows[peer]:
            t = torch.from_numpy(np.ascontiguousarray(send[s_off[peer]:s_off[peer + 1]]).view(np.uint8).copy())
            ops.append(dist.P2POp(dist.isend, t, peer))
        if recv_rows[peer]:
            t = torch.empty(int(recv_rows[peer]) * width * send.itemsize, dtype=torch.uint8)
            bufs.append((peer, t))
            ops.append(dist.P2POp(dist.irecv, t, peer))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    for peer, t in bufs:
        out[r_off[peer]:r_off[peer + 1]] = t.numpy().view(send.dtype).reshape(-1, width)
    return out


def main():
    rank, world, port, out_path = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    spec = synth.cfg1_tiny()
    layer = synth.make_layer(spec, seed=11)
    a = layer.arrays
    T = 24 + 8 * rank                      # ragged: ranks hold different token counts
    x = synth.make_tokens(T, spec.hidden, seed=100 + rank)
    H, I, E, K = spec.hidden, spec.intermediate, spec.n_experts, spec.top_k
    El = E // world
    ref = oracle.moe_forward(layer, x)

    # local routing and plan: identical to the single-device path
    indices, weights = ref.indices, ref.weights
    counts, offsets, perm, inv_perm = oracle.plan(indices, T, K, E)
    xf = synth.bf16_to_f32(x)
    sorted_rows = xf[perm // K]                                     # [M, H], sorted by (expert, token, slot)

    # 1. counts: every rank learns how many rows each peer sends to each of its experts
    recv_counts = all_to_all_rows(counts.reshape(world * El, 1).astype(np.uint32), [El] * world, [El] * world,
                                  rank, world).reshape(world, El)
    plan = ep.plan_exchange(recv_counts)
    # 2. rows out
    send_rows = [int(offsets[(d + 1) * El] - offsets[d * El]) for d in range(world)]
    recv_rows = [int(plan["rank_offsets"][s + 1] - plan["rank_offsets"][s]) for s in range(world)]
    got = all_to_all_rows(sorted_rows.astype(np.float32), send_rows, recv_rows, rank, world)
    assert got.shape[0] == plan["n_rows"]
    # 3. regroup by local expert, ascending source rank
    grouped = np.zeros_like(got)
    for s in range(world):
        for e in range(El):
            n = int(recv_counts[s, e])
            grouped[plan["seg_dst"][s, e]:plan["seg_dst"][s, e] + n] = got[plan["seg_src"][s, e]:plan["seg_src"][s, e] + n]
    row_expert = np.repeat(np.arange(El, dtype=np.uint32), np.diff(plan["local_offsets"]).astype(int))
    # 4. this rank's experts
    lo, hi = rank * El, (rank + 1) * El
    n = grouped.shape[0]

    def proj(name, rows, n_out, k_in):
        w, s, b = (a[f"experts.{name}.{p}"][lo:hi] for p in ("weight", "scales", "biases"))
        return oracle.gather_dequant_gemm(rows, w, s, b, row_expert, n, n_out, k_in, El, spec.expert_bits,
                                          spec.expert_group_size)

    if n:
        g = proj("gate_proj", grouped, I, H)
        u = proj("up_proj", grouped, I, H)
        inner = (g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u
        y = proj("down_proj", inner, H, I)
    else:
        y = np.zeros((0, H), dtype=np.float32)
    # 5. back along the same segments
    ret = np.zeros_like(y)
    for s in range(world):
        for e in range(El):
            c = int(recv_counts[s, e])
            ret[plan["seg_src"][s, e]:plan["seg_src"][s, e] + c] = y[plan["seg_dst"][s, e]:plan["seg_dst"][s, e] + c]
    home = all_to_all_rows(ret, recv_rows, send_rows, rank, world)   # [M, H] in this rank's sorted order
    out = oracle.unpermute(home, inv_perm, weights, T, H, K)
    err = float(np.abs(out - ref.out_f32).max())
    scale = float(np.abs(ref.out_f32).max())
    dist.barrier()
    dist.destroy_process_group()
    with open(out_path, "w") as f:
        json.dump({"rank": rank, "tokens": T, "rows_received": int(plan["n_rows"]), "max_err": err, "scale": scale,
                   "recv_counts": recv_counts.tolist()}, f)


if __name__ == "__main__":
    main()
