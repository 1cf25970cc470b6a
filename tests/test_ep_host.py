"""Expert-parallel host logic on the CPU: the exchange plan alone, and the whole protocol as two
gloo ranks checked against the single-process oracle."""
import json
import os
import socket
import subprocess
import sys

import numpy as np

from ffai_b200 import ep, synth

HERE = os.path.dirname(os.path.abspath(__file__))


def test_plan_exchange_layouts():
    rng = np.random.default_rng(3)
    for world, e_local in ((1, 4), (2, 8), (4, 3), (8, 32)):
        rc = rng.integers(0, 7, size=(world, e_local)).astype(np.uint32)
        rc[rng.integers(0, world), :] = 0            # a source that sends nothing
        p = ep.plan_exchange(rc)
        assert p["n_rows"] == int(rc.sum())
        assert np.array_equal(p["rank_offsets"], np.concatenate([[0], np.cumsum(rc.sum(axis=1))]))
        assert np.array_equal(p["local_offsets"], np.concatenate([[0], np.cumsum(rc.sum(axis=0))]))
        # source order: segments of one source are contiguous and ascending by expert
        assert np.array_equal(p["seg_src"].reshape(-1), np.concatenate([[0], np.cumsum(rc.reshape(-1))])[:-1])
        # regrouped order: segments of one expert are contiguous and ascending by source rank
        assert np.array_equal(p["seg_dst"].T.reshape(-1), np.concatenate([[0], np.cumsum(rc.T.reshape(-1))])[:-1])
        # the two layouts are permutations of each other
        src = np.concatenate([np.arange(p["seg_src"][s, e], p["seg_src"][s, e] + rc[s, e]) for s in range(world) for e in range(e_local)] or [np.zeros(0)])
        dst = np.concatenate([np.arange(p["seg_dst"][s, e], p["seg_dst"][s, e] + rc[s, e]) for s in range(world) for e in range(e_local)] or [np.zeros(0)])
        assert sorted(src.tolist()) == list(range(p["n_rows"])) and sorted(dst.tolist()) == list(range(p["n_rows"]))


def test_plan_exchange_empty():
    p = ep.plan_exchange(np.zeros((2, 4), dtype=np.uint32))
    assert p["n_rows"] == 0 and not p["local_offsets"].any() and not p["rank_offsets"].any()


def test_peer_layout_agrees_with_the_exchange_plan():
    """The device-side layout of the peer-memory mode (run here through its host copy) puts every
    (source rank, expert) segment where the NCCL mode's host plan puts it."""
    rng = np.random.default_rng(9)
    for world, e_local in ((2, 4), (4, 8), (8, 32)):
        E = world * e_local
        matrix = rng.integers(0, 9, size=(world, E)).astype(np.uint32)     # matrix[s, e]: rows rank s sends to expert e
        matrix[rng.integers(0, world)] = 0                                   # a rank without tokens
        for d in range(world):                                               # d: the rank that owns the experts
            plan = ep.plan_exchange(matrix[:, d * e_local:(d + 1) * e_local])
            mine = ep.peer_layout(matrix, d)
            assert np.array_equal(mine["local_offsets"], plan["local_offsets"])
            for s in range(world):
                theirs = ep.peer_layout(matrix, s)["send_base"][d * e_local:(d + 1) * e_local]
                assert np.array_equal(theirs, plan["seg_dst"][s])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_rank_protocol_matches_single_process_oracle(tmp_path, oracle_mod):
    port = _free_port()
    procs = []
    for r in range(2):
        out = tmp_path / f"r{r}.json"
        procs.append((out, subprocess.Popen([sys.executable, os.path.join(HERE, "ep_host_worker.py"), str(r), "2", str(port), str(out)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    for out, p in procs:
        try:
            log, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            raise
        assert p.returncode == 0, log.decode()[-2000:]
    res = [json.loads(out.read_text()) for out, _ in procs]
    # every routed row lands on exactly one rank
    assert sum(r["rows_received"] for r in res) == sum(r["tokens"] for r in res) * synth.cfg1_tiny().top_k
    for r in res:
        assert r["max_err"] <= 2e-5 * max(1.0, r["scale"]), r
