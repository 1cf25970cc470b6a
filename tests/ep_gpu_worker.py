"""One rank of the expert-parallel GPU test, as run by test_gpu_ep.py (one process per GPU).

Every rank holds the same layer (seeded) and its own tokens.  It runs the block with the experts
sharded over the ranks and checks, per case: routing and dispatch plan bit-exact against the oracle,
output within the parity gate against the oracle, and against the same block run with all experts
on this GPU alone.
usage: ep_gpu_worker.py <rank> <world> <port> <out.json>
"""
import json
import os
import sys
import traceback

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import torch
import torch.distributed as dist

import oracle
from ffai_b200 import capi, ep, synth
from ffai_b200.moe import MoELayer
from helpers import parity

CASES = [
    # name, spec, tokens on rank r, forced path (None = automatic)
    ("tiny_fp32_router", synth.cfg1_tiny(), lambda r: 16 + 4 * r, None),
    ("tiny_gemv_forced", synth.cfg1_tiny(), lambda r: 9, 1),
    ("gptoss_decode", synth.cfg2_gptoss(), lambda r: 8, None),
    ("gptoss_decode_one_token", synth.cfg2_gptoss(), lambda r: 1, None),
    ("qwen_prefill_tcgen05", synth.cfg3_qwen().with_(n_experts=32, name="qwen_32e"), lambda r: 192 + 64 * r, None),
    ("six_bit_gemv", synth.LayerSpec("bits6", 512, 256, 16, 4, expert_bits=6), lambda r: 40, None),
    ("shared_expert", synth.cfg4_shared().with_(n_experts=32, name="shared_32e"), lambda r: 24, None),
    ("rank_without_tokens", synth.cfg1_tiny(), lambda r: 0 if r == 1 else 12, None),
    # the 256-expert configuration at its real expert count, 1024 tokens per rank (outputs on a token sample)
    ("cfg4_256_experts", synth.cfg4_shared(), lambda r: 1024, None),
]
SAMPLED = {"cfg4_256_experts": 32}   # cases whose outputs are checked on this many sampled tokens (the oracle is scalar)


def bounded_wait_case(rank, world, store, meet):
    """One rank sits out a step of the peer-memory exchange; the others' barriers must give up within the (short)
    limit and report it through the status call, nothing faults or waits for ever, and the next step that all
    ranks run gives the same bits as the step before the gap.  The gap is made on the host, between steps."""
    spec = synth.cfg3_qwen().with_(n_experts=32, name="qwen_32e_gap")
    host = synth.make_layer(spec, seed=9)
    T = 96
    x = synth.make_tokens(T, spec.hidden, seed=2000 + rank)
    lay = MoELayer(host, T, ep_rank=rank, ep_world=world)
    rec = {"case": "bounded_wait", "tokens": 0, "bounded_wait": True}
    try:
        lay.set_option("ep_wait_ms", 50)
        store.set(f"blob/gap/{rank}", lay.ep_export())
        lay.ep_import([bytes(store.get(f"blob/gap/{r}")) for r in range(world)])
        meet("gap/go0")
        before, _ = lay.forward_host(x)
        meet("gap/go1")
        if rank == world - 1:
            lay.ep_skip_step()                      # this rank sits the step out
            rec["gave_up"] = None
        else:
            t0 = __import__("time").perf_counter()
            try:
                lay.forward_host(x)
                rec["gave_up"] = False
            except capi.FFAICudaError as err:
                rec["gave_up"] = err.status == capi.FFAI_ERR_DEVICE_CHECK
            rec["gave_up_after_s"] = __import__("time").perf_counter() - t0
        meet("gap/go2")                             # everybody has left the void step
        after, _ = lay.forward_host(x)
        lay.check_device_status()
        rec["same_bits_after_gap"] = bool(np.array_equal(before, after))
        meet("gap/done")
        lay.ep_release()
        meet("gap/released")
    finally:
        lay.close()
    return rec


def main():
    rank, world, port, out_path = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    torch.zeros(1, device="cuda")
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=120))
    comm = ep.comm_from_store(store, rank, world)

    def meet(tag):
        store.set(f"{tag}/{rank}", b"1")
        store.wait([f"{tag}/{r}" for r in range(world)])

    results = []
    try:
        for name, spec, tokens_of, path in CASES:
            T = tokens_of(rank)
            max_t = max(tokens_of(r) for r in range(world))
            host = synth.make_layer(spec, seed=5)
            x = synth.make_tokens(T, spec.hidden, seed=1000 + rank) if T else np.zeros((0, spec.hidden), np.uint16)
            lay = MoELayer(host, max_t, ep_rank=rank, ep_world=world, ep_comm=comm)
            one = MoELayer(host, max(max_t, 1))
            rec = {"case": name, "tokens": T}
            try:
                if path is not None:
                    lay.set_option("path", path)
                    one.set_option("path", path)
                out, dbg = lay.forward_host(x, debug=True)
                out2, _ = lay.forward_host(x)                      # a second call reuses every buffer
                lay.check_device_status()
                if T:
                    solo, _ = one.forward_host(x)
                    mask = None
                    if name in SAMPLED:
                        mask = np.zeros(T, dtype=np.uint8)
                        mask[np.random.default_rng(7 + rank).choice(T, size=SAMPLED[name], replace=False)] = 1
                    sel = np.arange(T) if mask is None else np.nonzero(mask)[0]
                    ref = oracle.moe_forward(host, x, token_mask=mask)
                    rec["routing_exact"] = bool(np.array_equal(dbg.indices, ref.indices) and np.array_equal(dbg.weights, ref.weights)
                                                and np.array_equal(dbg.perm, ref.perm) and np.array_equal(dbg.offsets, ref.offsets))
                    pr = parity(out[sel], ref.out_f32[sel])
                    rec["rel_rms"], rec["max_abs_norm"] = pr["rel_rms"], pr["max_abs_norm"]
                    rec["rel_rms_vs_single_gpu"] = parity(out, synth.bf16_to_f32(solo))["rel_rms"]
                    rec["repeatable"] = bool(np.array_equal(out, out2))
                rec["launches"] = lay.launch_count()
                # the same step with the exchange over peer memory (result rows travel as bf16 there)
                if spec.expert_bits == 4 and path != 1:
                    peer = MoELayer(host, max_t, ep_rank=rank, ep_world=world)
                    try:
                        if path is not None:
                            peer.set_option("path", path)
                        store.set(f"blob/{name}/{rank}", peer.ep_export())
                        peer.ep_import([bytes(store.get(f"blob/{name}/{r}")) for r in range(world)])
                        meet(f"go1/{name}")       # the barriers inside a step are time-limited: enter it together
                        pout, pdbg = peer.forward_host(x, debug=True)
                        meet(f"go2/{name}")
                        pout2, _ = peer.forward_host(x)
                        peer.check_device_status()
                        rec["peer_launches"] = peer.launch_count()
                        if T:
                            rec["peer_rel_rms_vs_nccl"] = parity(pout, synth.bf16_to_f32(out))["rel_rms"]
                            ppar = parity(pout[sel], ref.out_f32[sel])
                            rec["peer_rel_rms"], rec["peer_max_abs_norm"] = ppar["rel_rms"], ppar["max_abs_norm"]
                            rec["peer_routing_exact"] = bool(np.array_equal(pdbg.indices, ref.indices) and np.array_equal(pdbg.perm, ref.perm))
                            rec["peer_repeatable"] = bool(np.array_equal(pout, pout2))
                        meet(f"done/{name}")      # nobody unmaps while a peer may still be reading
                        peer.ep_release()
                        meet(f"released/{name}")  # nobody frees while a peer still maps
                    finally:
                        peer.close()
            finally:
                lay.close()
                one.close()
            results.append(rec)
        results.append(bounded_wait_case(rank, world, store, meet))
        status = "ok"
    except Exception:
        status = traceback.format_exc()
    torch.cuda.synchronize()
    store.set(f"done{rank}", b"1")
    for r in range(world):
        store.wait([f"done{r}"])
    ep.comm_destroy(comm)
    with open(out_path, "w") as f:
        json.dump({"rank": rank, "status": status, "cases": results}, f)


if __name__ == "__main__":
    main()
