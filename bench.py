#!/usr/bin/env python
"""Benchmark of the MoE block: tokens/s of one layer forward, with the kernel roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (seeded synthetic weights and activations, shapes of the benchmark configurations):
    cfg2_b64 (default), cfg2_b1, cfg2_b8, cfg2_b32   GPT-OSS-20B-shaped decode batches
    cfg2g32_b64, cfg2g32_b1, ...                     the same with group-32 experts and row biases (transcoded checkpoints)
    cfg3                                            Qwen3-30B-A3B-shaped 2048-token prefill
    cfg1                                            tiny layer
    prep_mxfp4, prep_quant4                         load-time weight preparation kernels (own metric: bytes/s)
    cfg4_ep, cfg3_ep                                256- / 128-expert layers, 2048 tokens per rank, experts
                                                    sharded over the N ranks (expert parallelism: two NCCL
                                                    all-to-all exchanges inside the timed step); N = 1 runs
                                                    the same layer with all experts on one GPU

A step is one forward of the layer over one batch.  Each step is timed on the device with a
CUDA-event pair on the launching stream; between steps a 256 MiB buffer is overwritten so the
next step finds none of its weights in L2 (the flush is not timed).  With N > 1 every rank runs
its own replica of the layer on its own batch (decode does not shard); time is the max over ranks.
The *_ep workloads instead shard the experts over the ranks and keep the tokens per rank fixed.

One JSON line is printed by rank 0.  `value` is device-resident throughput, `e2e` the same metric
through the host-buffer entry point of the C ABI (pinned-memory copies inside the timed region),
`roofline` describes the dominant kernel, `cpu_baseline` is the scalar CPU oracle on this host.
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

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu captures
# summarised in profiles/ (same workload, same command); None where no capture exists
NCU_TRAFFIC_BYTES = {"cfg2_b64": 306.2e6 + 5.1e6, "cfg3": 883.0e6 + 24.4e6}

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


def workload(name: str):
    """-> (spec, tokens per step and rank, regime)"""
    if name == "cfg4_ep":
        return synth.cfg4_shared(), 2048, "prefill"
    if name == "cfg3_ep":
        return synth.cfg3_qwen(), 2048, "prefill"
    if name.startswith("cfg2g32"):   # GPT-OSS experts as the MXFP4 transcode leaves them: group 32, row biases
        b = int(name.split("_b")[1]) if "_b" in name else 64
        return synth.cfg2_gptoss().with_(name="cfg2_gptoss20b_gs32", expert_group_size=32, expert_row_bias=1), b, "decode"
    if name.startswith("cfg2"):
        b = int(name.split("_b")[1]) if "_b" in name else 64
        return synth.cfg2_gptoss(), b, "decode"
    if name == "cfg3":
        return synth.cfg3_qwen(), 2048, "prefill"
    if name == "cfg1":
        return synth.cfg1_tiny(), 16, "decode"
    raise SystemExit(f"unknown workload {name}")


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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


def cpu_baseline(spec, n_tokens: int, seed: int, min_seconds: float, impl_line: bool = False):
    """The scalar CPU oracle on this host's cores, on a bounded sample of the workload."""
    import oracle
    oracle.build()
    host = synth.make_layer(spec, seed)
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
    return {"value": sample_tokens * reps / dt, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{reps} forward(s) of {sample_tokens} tokens of {spec.name} ({dt:.1f} s), "
                      f"expert-parallel over {threads} host threads"}, dt / reps


def run_reference(args, spec, n_tokens, rank, world):
    """--impl reference: the reference's CPU arithmetic (the oracle port; the Swift/Metal
    reference cannot be built on this box) on the host cores, same config and metric."""
    if rank != 0:
        return
    per_step_s = []
    base = None
    for i in range(args.warmup + args.steps):
        base, sec = cpu_baseline(spec, n_tokens, args.seed, min_seconds=0.0)
        if i >= args.warmup:
            per_step_s.append(sec)
        if sum(per_step_s) > 120:
            break
    sample_tokens = min(n_tokens, 64)
    ms = 1e3 * statistics.mean(per_step_s)
    value = sample_tokens / (ms / 1e3)
    base["value"] = value
    line = {"metric": METRIC, "value": value, "unit": UNIT, "impl": "reference", "n_gpus": world,
            "steps": len(per_step_s), "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
            "config": {"workload": args.workload, "layer": spec.name, "tokens_per_step": sample_tokens},
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
                      "config": {"workload": args.workload, "rows": rows, "in_dim": K, "l2": "256 MiB buffer overwritten between steps (not timed)"},
                      "gpu_launches": args.steps + args.warmup,
                      "roofline": {"bound": "hbm", "kernel": kernel, "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                   "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"], "traffic": None,
                                   "algorithmic_bytes_per_launch": nbytes, "kernel_ms": ms}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg2_b64")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--option", action="append", default=[], help="name=value execution option (experiments)")
    ap.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                    help="*_ep workloads: row exchange over peer memory (CUDA IPC, fused into gather and combine) or NCCL send/recv")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload.startswith("prep_"):
        if rank == 0:
            run_prep(args)
        return
    spec, n_tokens, regime = workload(args.workload)

    if args.impl == "reference":
        run_reference(args, spec, n_tokens, rank, world)
        return

    import torch
    import torch.distributed as dist
    from ffai_b200.moe import MoELayer

    lib = capi.load()
    if lib.ffai_cuda_device_count() <= 0:
        raise SystemExit("bench.py needs a CUDA device: libffai_cuda has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    host = synth.make_layer(spec, args.seed)
    ep_mode = args.workload.endswith("_ep") and world > 1
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
        name, value = ov.split("=")
        layer.set_option(name, int(value))
    H = spec.hidden
    n_batches = 8
    # host batches live in page-locked memory (the end-to-end pass copies from and to pinned buffers)
    xs_pin = [torch.from_numpy(synth.make_tokens(n_tokens, H, args.seed + 100 * rank + i).view(np.int16)).pin_memory()
              for i in range(n_batches)]
    xs_host = [t.numpy().view(np.uint16) for t in xs_pin]
    out_pin = torch.zeros(n_tokens, H, dtype=torch.int16).pin_memory()
    out_host = out_pin.numpy().view(np.uint16)
    xs_dev = [t.cuda() for t in xs_pin]
    out_dev = torch.zeros(n_tokens * H, dtype=torch.int16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()

    # distinct experts selected per batch (for the algorithmic decode bytes)
    distinct = []
    for x in xs_host:
        _, dbg = layer.forward_host(x, debug=True)
        distinct.append(int((dbg.counts > 0).sum()))

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def step(i, timed):
        flush.zero_()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        layer.forward_ptr(xs_dev[i % n_batches].data_ptr(), n_tokens, out_dev.data_ptr(), stream=stream.cuda_stream)
        ev1.record(stream)
        if timed:
            ev1.synchronize()
            return ev0.elapsed_time(ev1), layer.stage_ms(), layer.launch_count()
        return None

    for i in range(args.warmup):
        step(i, False)
        if ep_mode:
            sync_all()      # ranks enter every exchange together
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    times, stages, launches = [], [], 0
    for i in range(args.steps):
        ms, _, nl = step(i, True)
        times.append(ms); launches += nl
        if ep_mode:
            sync_all()
    sync_all()
    clocks = sampler.stop() if rank == 0 else None

    # per-kernel durations for the roofline: a second pass with the library's stage events switched on
    # (the event records cost a few microseconds per stage, so they stay out of the headline pass)
    layer.set_stage_timing(True)
    for i in range(min(args.steps, 20)):
        _, st, nl = step(i, True)
        stages.append(st); launches += nl
    layer.set_stage_timing(False)

    # end to end through the host-buffer entry point (copies inside the timed region)
    e2e_times = []
    for i in range(3 + args.steps):
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        layer.forward_host(xs_host[i % n_batches], out=out_host)
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

    if rank == 0:
        peaks = measured_peaks()
        used = [distinct[i % n_batches] for i in range(args.steps)]
        mean_distinct = statistics.mean(used)
        stage_mean = {k: statistics.mean(s[k] for s in stages) for k in stages[0]}
        bpw = spec.bytes_per_weight()
        if regime == "decode":
            # dominant kernel: the fused gate/up product (2 of the 3 projections' bytes)
            kernel, kms = "gate_up", stage_mean["gate_up"]
            alg_bytes = mean_distinct * 2.0 * spec.hidden * spec.intermediate * bpw + n_tokens * H * 2.0
            achieved = alg_bytes / (kms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peaks["hbm_gbs"],
                        "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                        "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "algorithmic_bytes_per_launch": alg_bytes, "kernel_ms": kms}
            layer_bytes = spec.decode_bytes(n_tokens, mean_distinct)
            layer_frac = layer_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]
        else:
            fl = spec.prefill_flops(n_tokens)
            kernel, kms = "gate_up", stage_mean["gate_up"]
            alg = fl["routed"] * 2.0 / 3.0
            achieved = alg / (kms * 1e-3) / 1e12
            roofline = {"bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": peaks["bf16_tflops"],
                        "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "peak_source": peaks["source"],
                        "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "algorithmic_flops_per_launch": alg, "kernel_ms": kms}
            layer_frac = (fl["routed"] + fl["shared"] + fl["router"]) / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"]
        line = {
            "metric": METRIC, "value": world * n_tokens / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u4 weights, bf16 activations, f32 accumulate",
            "data": "synthetic (seeded Philox; shapes and value distributions of the benchmark configuration)",
            "config": {"workload": args.workload, "layer": spec.name, "tokens_per_step": n_tokens, "regime": regime,
                       "hidden": spec.hidden, "intermediate": spec.intermediate, "experts": spec.n_experts,
                       "top_k": spec.top_k, "bits": spec.expert_bits, "group_size": spec.expert_group_size,
                       "distinct_experts_per_step": mean_distinct, "input_batches_rotated": n_batches,
                       "l2": "256 MiB buffer overwritten between steps (not timed)",
                       "parallelism": (f"ep{world}: experts sharded, tokens per rank fixed" if ep_mode else
                                       "replicas" if world > 1 else "single")},
            "e2e": {"value": world * n_tokens / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": n_tokens * H * 2, "d2h_bytes_per_step": n_tokens * H * 2},
            "gpu_launches": launches,
            "roofline": roofline,
            "layer_roofline_frac": layer_frac,
            "stage_ms": stage_mean,
            "clocks": clocks,
        }
        if ep_mode:
            rows = n_tokens * spec.top_k
            off_rank = (world - 1) / world      # share of a rank's rows whose expert lives on another rank (uniform routing)
            line["ep"] = {"exchange_ms": stage_mean["exchange"], "rows_per_rank": rows,
                          "dispatch_bytes_per_rank": rows * H * 2 * off_rank, "return_bytes_per_rank": rows * H * 4 * off_rank,
                          "transport": ("peer memory over NVLink (CUDA IPC): gather fused with dispatch, combine fused with "
                                        "return, three flag barriers, no host synchronisation" if args.ep_exchange == "peer"
                                        else "NCCL send/recv groups over NVLink, one host sync per step for the sizes")}
        if not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_baseline(spec, n_tokens, args.seed, args.cpu_seconds)
        print(json.dumps(line), flush=True)
    if ep_mode and ep_comm is None:
        sync_all()
        layer.ep_release()
        sync_all()
    layer.close()
    if ep_comm is not None:
        sync_all()
        ep.comm_destroy(ep_comm)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
