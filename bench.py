#!/usr/bin/env python
"""Benchmark of the MoE block: tokens/s of one layer forward, with the kernel roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (seeded synthetic weights and activations, shapes of the benchmark configurations):
    cfg4 (default)                           256-expert layer with the gated shared expert, 8192 tokens in
                                             total.  With N ranks the experts are sharded 256/N per rank and
                                             every rank holds 8192/N of the tokens (strong scaling); rows travel
                                             to their experts and back over peer memory (or NCCL, --ep-exchange).
                                             N = 1 is the same layer with all experts on one GPU.
    cfg3                                     Qwen3-30B-A3B-shaped 2048-token prefill (same sharding rule)
    cfg5_b3, cfg5_b5, cfg5_b6, cfg5_b8       the cfg3 shape with Zipf-skewed routing and experts re-quantised at
                                             that bit width, 16384 tokens in total (same sharding rule)
    cfg2_b64, cfg2_b1, cfg2_b8, cfg2_b32     GPT-OSS-20B-shaped decode batches (does not shard: N replicas)
    cfg2g32_b64, ...                         the same with group-32 experts and row biases (transcoded checkpoints)
    cfg4_ep, cfg3_ep                         2048 tokens per rank (weak scaling) of the sharded layers
    cfg1                                     tiny layer
    prep_mxfp4, prep_quant4                  load-time weight preparation kernels (own metric: bytes/s)

A step is one forward of the layer over one batch.  Each step is timed on the device with a CUDA-event
pair on the launching stream; between steps a 256 MiB buffer is overwritten so the next step finds none
of its weights in L2 (the flush is not timed).  Time is the max over ranks.

One JSON line is printed by rank 0.  `value` is device-resident throughput, `e2e` the same metric through
the host-buffer entry point of the C ABI (pinned-memory copies inside the timed region), `roofline`
describes the dominant kernel, `cpu_baseline` is the scalar CPU oracle on this host.  When no workload is
named, rank 0 afterwards times the decode sweep (cfg2, 1 / 8 / 32 / 64 tokens) and the cfg3 prefill on its
own GPU and attaches them under `workloads`, each with its own roofline.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np

from ffai_b200 import capi, synth

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
DEFAULT_WORKLOAD = "cfg4"
SWEEP = ("cfg2_b1", "cfg2_b8", "cfg2_b32", "cfg2_b64", "cfg3")
N_BATCHES = 8
L2_NOTE = "256 MiB buffer overwritten between steps (not timed)"


def workload(name: str):
    """-> (spec builder, tokens per step over all ranks, regime, sharding).
    sharding: "strong" (experts and tokens split over the ranks), "weak" (experts split, tokens per rank
    fixed), None (the layer does not shard: every rank runs a replica)."""
    if name == "cfg4":
        return synth.cfg4_shared, 8192, "prefill", "strong"
    if name == "cfg3":
        return synth.cfg3_qwen, 2048, "prefill", "strong"
    if name.startswith("cfg5_b"):
        bits = int(name.split("_b")[1])
        return (lambda: cfg5_layer_spec(bits)), 16384, "prefill", "strong"
    if name == "cfg4_ep":
        return synth.cfg4_shared, 2048, "prefill", "weak"
    if name == "cfg3_ep":
        return synth.cfg3_qwen, 2048, "prefill", "weak"
    if name.startswith("cfg2g32"):   # GPT-OSS experts as the MXFP4 transcode leaves them: group 32, row biases
        b = int(name.split("_b")[1]) if "_b" in name else 64
        return (lambda: synth.cfg2_gptoss().with_(name="cfg2_gptoss20b_gs32", expert_group_size=32, expert_row_bias=1)), b, "decode", None
    if name.startswith("cfg2"):
        b = int(name.split("_b")[1]) if "_b" in name else 64
        return synth.cfg2_gptoss, b, "decode", None
    if name == "cfg1":
        return synth.cfg1_tiny, 16, "decode", None
    raise SystemExit(f"unknown workload {name}")


def cfg5_layer_spec(bits: int):
    return synth.cfg5_skewed(bits)


def make_host_layer(name: str, spec, seed: int):
    """Host arrays of a workload's layer.  The skewed sweep re-quantises the experts of the 4-bit layer of
    the same shape at the requested width, as the configuration describes."""
    if name.startswith("cfg5_b"):
        base = synth.make_layer(spec.with_(expert_bits=4), seed)
        return base if spec.expert_bits == 4 else synth.requantize_experts(base, spec.expert_bits)
    return synth.make_layer(spec, seed)


def tokens_per_rank(total: int, sharding, world: int) -> int:
    if sharding == "strong":
        if total % world:
            raise SystemExit(f"{total} tokens do not divide over {world} ranks")
        return total // world
    return total


def describe(name: str, spec, total_tokens: int, regime: str, sharding, world: int, exchange: str):
    """The `config` object.  Built from the command line alone, so both arms print the same one."""
    if sharding and world > 1:
        par = (f"ep{world}: experts sharded {spec.n_experts // world} per rank, "
               + (f"{total_tokens // world} of {total_tokens} tokens per rank" if sharding == "strong"
                  else f"{total_tokens} tokens per rank") + f", row exchange over {exchange}")
    elif world > 1:
        par = f"replicas: the layer does not shard, {world} independent copies"
    else:
        par = "single GPU, all experts"
    n_step = total_tokens if (sharding == "strong" or world == 1) else total_tokens * world
    return {"workload": name, "layer": spec.name, "tokens_per_step": n_step, "regime": regime,
            "hidden": spec.hidden, "intermediate": spec.intermediate, "experts": spec.n_experts,
            "top_k": spec.top_k, "bits": spec.expert_bits, "group_size": spec.expert_group_size,
            "shared_intermediate": spec.shared_intermediate, "input_batches_rotated": N_BATCHES,
            "l2": L2_NOTE, "parallelism": par}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def ncu_traffic(name: str):
    """DRAM bytes (read + written) of one launch of the workload's dominant kernel, from the ncu capture
    summarised under profiles/ (the figures file sits beside the summaries); None without a capture."""
    p = ROOT / "profiles" / "ncu_traffic.json"
    if not p.exists():
        return None
    rec = json.loads(p.read_text()).get(name)
    return None if rec is None else float(rec["dram_bytes_per_launch"])


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(host, n_tokens: int, seed: int, min_seconds: float, single_thread: bool = True):
    """The scalar CPU oracle on this host's cores, on a bounded sample of the workload: all the cores the
    process may use (experts of a token batch in parallel), and one thread beside it."""
    import oracle
    oracle.build()
    spec = host.spec
    sample_tokens = min(n_tokens, 64)
    x = synth.make_tokens(sample_tokens, spec.hidden, seed)
    # every core this process may run on, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for its ranks)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.moe_forward(host, x[:1], n_threads=threads)  # touch the weights once
    t0 = time.perf_counter()
    reps = 0
    while True:
        oracle.moe_forward(host, x, n_threads=threads)
        reps += 1
        if time.perf_counter() - t0 >= min_seconds or reps >= 50:
            break
    dt = time.perf_counter() - t0
    out = {"value": sample_tokens * reps / dt, "unit": UNIT, "cores": threads, "kind": "port",
           "sample": f"{reps} forward(s) of {sample_tokens} tokens of {spec.name} ({dt:.1f} s), "
                     f"expert-parallel over {threads} host threads"}
    if single_thread:
        n1 = min(sample_tokens, 8)
        t1 = time.perf_counter()
        oracle.moe_forward(host, x[:n1], n_threads=1)
        d1 = time.perf_counter() - t1
        out["single_thread"] = {"value": n1 / d1, "unit": UNIT, "cores": 1,
                                "sample": f"one forward of {n1} tokens ({d1:.1f} s)"}
    return out, dt / reps


def run_reference(args, name, rank, world):
    """--impl reference: the reference's CPU arithmetic (the oracle port; the Swift/Metal
    reference cannot be built on this box) on the host cores, same config and metric."""
    if rank != 0:
        return
    make_spec, total, regime, sharding = workload(name)
    spec = make_spec()
    host = make_host_layer(name, spec, args.seed)
    per_step_s = []
    base = None
    for i in range(args.warmup + args.steps):
        base, sec = cpu_baseline(host, total, args.seed, min_seconds=0.0, single_thread=False)
        if i >= args.warmup:
            per_step_s.append(sec)
        if sum(per_step_s) > 120:
            break
    sample_tokens = min(total, 64)
    ms = 1e3 * statistics.mean(per_step_s)
    value = sample_tokens / (ms / 1e3)
    base["value"] = value
    line = {"metric": METRIC, "value": value, "unit": UNIT, "impl": "reference", "n_gpus": world,
            "steps": len(per_step_s), "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if sharding == "strong" else "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic (seeded)",
            "config": describe(name, spec, total, regime, sharding, world, args.ep_exchange),
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_prep(args):
    """--workload prep_mxfp4 | prep_quant4: the load-time weight preparation kernels on one GPT-OSS-20B-sized
    stacked projection (32 x 2880 x 2880), GB/s against the HBM roofline (bytes read + written)."""
    import torch
    lib = capi.load()
    if lib.ffai_cuda_device_count() <= 0:
        raise SystemExit("bench.py needs a CUDA device: libffai_cuda has no CPU fallback")
    rows, K = 32 * 2880, 2880
    g = torch.Generator(device="cuda").manual_seed(args.seed)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    if args.workload == "prep_mxfp4":
        n_groups = rows * K // 32
        src = torch.randint(0, 256, (n_groups * 16,), dtype=torch.uint8, device="cuda", generator=g)
        e8 = torch.randint(110, 130, (n_groups,), dtype=torch.uint8, device="cuda", generator=g)
        ow = torch.empty_like(src)
        osc = torch.empty(n_groups, dtype=torch.int16, device="cuda")
        obi = torch.empty(n_groups, dtype=torch.int16, device="cuda")
        nbytes = n_groups * (16 + 1 + 16 + 4)
        call = lambda: lib.ffai_op_mxfp4_to_affine_int4(src.data_ptr(), e8.data_ptr(), n_groups, ow.data_ptr(), osc.data_ptr(),
                                                        obi.data_ptr(), torch.cuda.current_stream().cuda_stream)
        kernel = "mxfp4_to_affine4_kernel"
    else:
        w = torch.randn(rows * K, device="cuda", generator=g).to(torch.bfloat16)
        ow = torch.empty(rows * K // 8, dtype=torch.int32, device="cuda")
        osc = torch.empty(rows * K // 64, dtype=torch.int16, device="cuda")
        obi = torch.empty(rows * K // 64, dtype=torch.int16, device="cuda")
        nbytes = rows * K * 2 + rows * K // 2 + rows * K // 64 * 4
        call = lambda: lib.ffai_op_affine_quantize(w.data_ptr(), rows, K, 4, 64, ow.data_ptr(), osc.data_ptr(), obi.data_ptr(),
                                                   torch.cuda.current_stream().cuda_stream)
        kernel = "affine_quantize_kernel<4>"
    times = []
    for i in range(args.warmup + args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        capi.check(call(), kernel)
        e1.record()
        e1.synchronize()
        if i >= args.warmup:
            times.append(e0.elapsed_time(e1))
    ms = statistics.mean(times)
    peaks = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "weight_prep_bytes_per_s", "value": gbs * 1e9, "unit": "bytes/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "u4 codes, bf16 scales", "data": "synthetic (seeded)",
                      "config": {"workload": args.workload, "rows": rows, "in_dim": K, "l2": L2_NOTE},
                      "gpu_launches": args.steps + args.warmup,
                      "roofline": {"bound": "hbm", "kernel": kernel, "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                   "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"], "traffic": None,
                                   "algorithmic_bytes_per_launch": nbytes, "kernel_ms": ms}}), flush=True)


def measure(name, args, rank, local_rank, world, dist, steps, with_clocks):
    """Times one workload on this process's GPU (with `world` > 1 and a sharding rule: together with the
    other ranks).  Returns the result record on rank 0, None elsewhere."""
    import torch
    from ffai_b200.moe import MoELayer

    make_spec, total, regime, sharding = workload(name)
    spec = make_spec()
    host = make_host_layer(name, spec, args.seed)
    n_tokens = tokens_per_rank(total, sharding, world)
    ep_mode = sharding is not None and world > 1
    ep_comm = None
    if ep_mode:
        from ffai_b200 import ep
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        if args.ep_exchange == "nccl":
            uid = [ep.unique_id() if rank == 0 else None]
            dist.broadcast_object_list(uid, src=0)
            ep_comm = ep.comm_create(uid[0], rank, world)
            layer = MoELayer(host, n_tokens, ep_rank=rank, ep_world=world, ep_comm=ep_comm)
        else:
            layer = MoELayer(host, n_tokens, ep_rank=rank, ep_world=world)
            blobs = [None] * world
            dist.all_gather_object(blobs, layer.ep_export())
            layer.ep_import(blobs)
    else:
        layer = MoELayer(host, n_tokens)
    layer.set_stage_timing(False)
    for ov in args.option:
        oname, value = ov.split("=")
        layer.set_option(oname, int(value))
    H = spec.hidden
    # host batches live in page-locked memory (the end-to-end pass copies from and to pinned buffers);
    # a rank's batches differ from every other rank's
    seed0 = args.seed + 100 * rank
    xs_pin = [torch.from_numpy(synth.make_tokens(n_tokens, H, seed0 + i).view(np.int16)).pin_memory()
              for i in range(N_BATCHES)]
    xs_host = [t.numpy().view(np.uint16) for t in xs_pin]
    out_pin = torch.zeros(n_tokens, H, dtype=torch.int16).pin_memory()
    out_host = out_pin.numpy().view(np.uint16)
    xs_dev = [t.cuda() for t in xs_pin]
    out_dev = torch.zeros(n_tokens * H, dtype=torch.int16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # distinct experts selected per batch (for the algorithmic decode bytes)
    distinct = []
    for x in xs_host:
        if ep_mode:
            sync_all()      # ranks enter every exchange together
        _, dbg = layer.forward_host(x, debug=True)
        distinct.append(int((dbg.counts > 0).sum()))

    def step(i, timed):
        flush.zero_()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        layer.forward_ptr(xs_dev[i % N_BATCHES].data_ptr(), n_tokens, out_dev.data_ptr(), stream=stream.cuda_stream)
        ev1.record(stream)
        if timed:
            ev1.synchronize()
            return ev0.elapsed_time(ev1), layer.stage_ms(), layer.launch_count()
        return None

    for i in range(args.warmup):
        step(i, False)
        if ep_mode:
            sync_all()
    sync_all()
    sampler = ClockSampler(local_rank) if (with_clocks and rank == 0) else None
    if sampler:
        sampler.start()
    times, stages, launches = [], [], 0
    for i in range(steps):
        ms, _, nl = step(i, True)
        times.append(ms); launches += nl
        if ep_mode:
            sync_all()
    sync_all()
    clocks = sampler.stop() if sampler else None

    # per-kernel durations for the roofline: a second pass with the library's stage events switched on
    # (the event records cost a few microseconds per stage, so they stay out of the headline pass)
    layer.set_stage_timing(True)
    for i in range(min(steps, 20)):
        _, st, nl = step(i, True)
        stages.append(st); launches += nl
        if ep_mode:
            sync_all()
    layer.set_stage_timing(False)

    # end to end through the host-buffer entry point (copies inside the timed region)
    e2e_times = []
    e2e_steps = 3 + min(steps, 50)
    for i in range(e2e_steps):
        flush.zero_()
        if ep_mode:
            sync_all()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        layer.forward_host(xs_host[i % N_BATCHES], out=out_host)
        dt = time.perf_counter() - t0
        if i >= 3:
            e2e_times.append(dt * 1e3)
            launches += layer.launch_count()

    ms_step = statistics.mean(times)
    e2e_ms = statistics.mean(e2e_times)
    if world > 1:
        t = torch.tensor([ms_step, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, e2e_ms = float(t[0]), float(t[1])
        lt = torch.tensor([launches], device="cuda", dtype=torch.int64)
        dist.all_reduce(lt)
        launches = int(lt[0])

    rec = None
    if rank == 0:
        peaks = measured_peaks()
        used = [distinct[i % N_BATCHES] for i in range(steps)]
        mean_distinct = statistics.mean(used)
        stage_mean = {k: statistics.mean(s[k] for s in stages) for k in stages[0]}
        bpw = spec.bytes_per_weight()
        step_tokens = n_tokens * world if (ep_mode or sharding is None) else n_tokens
        if regime == "decode":
            # dominant kernel: the fused gate/up product (2 of the 3 projections' bytes)
            kernel, kms = "gate_up", stage_mean["gate_up"]
            alg_bytes = mean_distinct * 2.0 * spec.hidden * spec.intermediate * bpw + n_tokens * H * 2.0
            achieved = alg_bytes / (kms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peaks["hbm_gbs"],
                        "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                        "traffic": ncu_traffic(name), "algorithmic_bytes_per_launch": alg_bytes, "kernel_ms": kms}
            down_bytes = mean_distinct * spec.hidden * spec.intermediate * bpw + n_tokens * spec.top_k * (spec.intermediate * 2.0 + H * 4.0)
            roofline["down"] = {"kernel_ms": stage_mean["down"], "algorithmic_bytes_per_launch": down_bytes,
                                "frac": down_bytes / (stage_mean["down"] * 1e-3) / 1e9 / peaks["hbm_gbs"]}
            layer_bytes = spec.decode_bytes(n_tokens, mean_distinct)
            layer_frac = layer_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]
        else:
            # per-rank share of the routed FLOPs (uniform routing: every rank's experts see 1/world of the rows)
            fl = spec.prefill_flops(total if sharding == "strong" else n_tokens * (world if ep_mode else 1))
            share = 1.0 / world if ep_mode else 1.0
            kernel, kms = "gate_up", stage_mean["gate_up"]
            alg = fl["routed"] * 2.0 / 3.0 * share
            achieved = alg / (kms * 1e-3) / 1e12
            roofline = {"bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": peaks["bf16_tflops"],
                        "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "peak_source": peaks["source"],
                        "peak_kind": "burst (the kernel is timed alone between stage events)",
                        "traffic": ncu_traffic(name), "algorithmic_flops_per_launch": alg, "kernel_ms": kms}
            roofline["down"] = {"kernel_ms": stage_mean["down"], "algorithmic_flops_per_launch": alg / 2.0,
                                "frac": alg / 2.0 / (stage_mean["down"] * 1e-3) / 1e12 / peaks["bf16_tflops"]}
            # a rank's own work: its share of the routed rows, its own tokens through the shared expert and the router
            layer_flops = fl["routed"] * share + (fl["shared"] + fl["router"]) * share
            layer_frac = layer_flops / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"]
        rec = {"workload": name, "config": describe(name, spec, total, regime, sharding, world, args.ep_exchange),
               "tokens_per_step": step_tokens, "tokens_per_rank": n_tokens, "ms_per_step": ms_step,
               "value": step_tokens / (ms_step * 1e-3), "sharding": sharding, "ep_mode": ep_mode,
               "e2e": {"value": step_tokens / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": step_tokens * H * 2, "d2h_bytes_per_step": step_tokens * H * 2},
               "gpu_launches": launches, "roofline": roofline, "layer_roofline_frac": layer_frac,
               "stage_ms": stage_mean, "distinct_experts_per_step": mean_distinct, "clocks": clocks,
               "host": host}
        if ep_mode:
            rows = n_tokens * spec.top_k
            off_rank = (world - 1) / world      # share of a rank's rows whose expert lives on another rank (uniform routing)
            ret_bytes = 2 if args.ep_exchange == "peer" else 4   # result rows travel as bf16 over peer memory, fp32 over NCCL
            rec["ep"] = {"exchange_ms": stage_mean["exchange"], "rows_per_rank": rows,
                         "dispatch_bytes_per_rank": rows * H * 2 * off_rank, "return_bytes_per_rank": rows * H * ret_bytes * off_rank,
                         "transport": ("peer memory over NVLink (CUDA IPC): gather fused with dispatch, combine fused with "
                                       "return, flag barriers, no host synchronisation" if args.ep_exchange == "peer"
                                       else "NCCL send/recv groups over NVLink, one host sync per step for the sizes")}
    if ep_mode and ep_comm is None:
        sync_all()
        layer.ep_release()
        sync_all()
    layer.close()
    if ep_comm is not None:
        from ffai_b200 import ep
        sync_all()
        ep.comm_destroy(ep_comm)
    del xs_dev, out_dev, flush
    torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="default workload only: skip the decode / prefill sweep")
    ap.add_argument("--option", action="append", default=[], help="name=value execution option (experiments)")
    ap.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                    help="sharded workloads: row exchange over peer memory (CUDA IPC, fused into gather and combine) or NCCL send/recv")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    sweep = args.workload is None and not args.no_sweep
    name = args.workload or DEFAULT_WORKLOAD
    args.workload = name
    if name.startswith("prep_"):
        if rank == 0:
            run_prep(args)
        return
    if args.impl == "reference":
        run_reference(args, name, rank, world)
        return

    import torch
    import torch.distributed as dist

    lib = capi.load()
    if lib.ffai_cuda_device_count() <= 0:
        raise SystemExit("bench.py needs a CUDA device: libffai_cuda has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # before any communicator exists: plain peer transports only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    head = measure(name, args, rank, local_rank, world, dist, args.steps, with_clocks=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()
    if rank != 0:
        return

    host = head.pop("host")
    line = {
        "metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
        "scaling": "strong" if head["sharding"] == "strong" else "weak", "vs_baseline": None,
        "dtype": f"u{host.spec.expert_bits} weights, bf16 activations, f32 accumulate",
        "data": "synthetic (seeded Philox; shapes and value distributions of the benchmark configuration)",
        "config": head["config"],
        "e2e": head["e2e"],
        "gpu_launches": head["gpu_launches"],
        "roofline": head["roofline"],
        "layer_roofline_frac": head["layer_roofline_frac"],
        "stage_ms": head["stage_ms"],
        "distinct_experts_per_step": head["distinct_experts_per_step"],
        "clocks": head["clocks"],
    }
    if "ep" in head:
        line["ep"] = head["ep"]
    if sweep:
        # the other halves of the metric, on rank 0's GPU alone: decode batches against the HBM roofline,
        # the 2048-token prefill against the tensor-core roofline
        one = argparse.Namespace(**vars(args))
        line["workloads"] = {}
        for wn in SWEEP:
            r = measure(wn, one, 0, local_rank, 1, None, min(args.steps, 100), with_clocks=False)
            r.pop("host"); r.pop("clocks"); r.pop("sharding"); r.pop("ep_mode"); r.pop("config")
            line["workloads"][wn] = r
    if not args.no_cpu_baseline:
        make_spec, total, _, _ = workload(name)
        line["cpu_baseline"], _ = cpu_baseline(host, total, args.seed, args.cpu_seconds)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
