"""Benchmark of the paged decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

One step is one decode call (one launch of the streaming decode kernel, which merges its own
partial results) over one
synthetic batch of the named workload.  At N GPUs every rank holds its own batch of the
same shape (requests shard across ranks with no communication: weak scaling), except
workload c4, whose KV range is sharded across ranks and merged after an all-gather
(strong scaling).  The metric is HBM GB/s over the algorithmic KV bytes of the batch
(2 * sum(seq_lens) * Hkv * D * elem + scale bytes), with microseconds per call beside it.

Rank 0 prints ONE JSON line.  `value` is timed with CUDA events on the launching stream
with everything resident in HBM; `e2e` goes through the host-buffer entry point
(pd_decode_host) with q, block table and lengths copied from pinned host memory and the
result copied back inside the timed region; `roofline` relates the decode step to the
measured copy bandwidth of this pool; `cpu_baseline` times the CPU port of the reference's
algorithm on this box's cores.  `--impl reference` times only that CPU port.
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode_attn_hbm_gbs"
# DRAM bytes moved per algorithmic byte, from one ncu capture of the streaming kernel per
# workload shape (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic KV bytes of
# the captured case; see profiles/).  Traffic grows in proportion to the tokens processed, so
# the ratio scales a full launch.
NCU_TRAFFIC_RATIO = {"c2": 1.0136, "c3": 1.024, "c4": 1.015, "c5": 1.025}
L2_BYTES = 126 << 20
FALLBACK_HBM_GBS = 6650.0


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, enabled: bool = True):
        self.gpu = gpu_index
        self.enabled = enabled  # only the reporting rank samples
        self.lines: list[str] = []
        self.proc = None

    def __enter__(self):
        if not self.enabled:
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def _sample_rows(lens, budget_tokens: int) -> list[int]:
    """Indices of a prefix of requests holding about `budget_tokens` tokens (at least one)."""
    rows, total = [], 0
    for i, n in enumerate(lens):
        if rows and total + n > budget_tokens:
            break
        rows.append(i)
        total += int(n)
    return rows


def cpu_port_timing(cache, q, steps: int, warmup: int, budget_tokens: int):
    """Times the CPU ports of the reference's path on a bounded sample of the batch."""
    import torch

    from oracle import adapters, c_oracle, torch_port
    from paged_decode_attention_b200 import synth

    lens = cache.seq_lens.cpu().tolist()
    rows = _sample_rows(lens, budget_tokens)
    sub = synth.take_requests(cache, rows)
    oc = adapters.from_torch_cache(sub)
    qf = adapters.q_to_f32(q[rows])
    nbytes = oc.bytes_read_per_decode_step()
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)

    def timed(fn):
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(steps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return ts

    t_torch = timed(lambda: torch_port.decode(qf, oc))
    t_c = timed(lambda: c_oracle.decode(qf, oc, num_threads=threads))
    sample = (f"{len(rows)} of {len(lens)} requests of the batch, {sum(lens[i] for i in rows)} tokens, "
              f"{nbytes / 1e6:.1f} MB of KV; torch-on-CPU restatement of reference_decode "
              f"(gather + fp32 attention), {steps} timed passes after {warmup} warm-up")
    return {
        "torch_s": statistics.mean(t_torch), "c_s": statistics.mean(t_c), "bytes": nbytes,
        "threads": threads, "torch_threads": torch.get_num_threads(),
        "c_threads": c_oracle.max_threads(), "sample": sample, "rows": len(rows),
    }


def run_reference(args) -> None:
    """--impl reference: the CPU port of the reference's path, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    from paged_decode_attention_b200 import synth

    w = synth.WORKLOADS[args.workload]
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    # a bounded draw: the sample is cut from the same seeded batch the GPU arm uses when a
    # GPU is present, from a smaller draw of the same distribution otherwise
    if dev == "cpu":
        q, cache = synth.make(args.workload, device="cpu", seed=args.seed, batch=min(w.batch, 8))
    else:
        q, cache = synth.make(args.workload, device=dev, seed=args.seed)
    r = cpu_port_timing(cache, q, steps=args.steps, warmup=args.warmup, budget_tokens=args.cpu_tokens)
    gbs = r["bytes"] / r["torch_s"] / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["torch_s"] * 1e3,
        "us_per_call": r["torch_s"] * 1e6, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {w.description}", "seed": args.seed,
                   "note": "CPU port on a bounded sample; value = sample KV bytes / pass time"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": r["torch_threads"], "kind": "port",
                         "sample": r["sample"]},
        "cpu_port_c": {"value": r["bytes"] / r["c_s"] / 1e9, "unit": "GB/s", "cores": r["c_threads"],
                       "note": "fused C/OpenMP restatement on the same sample"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import paged_decode_attention_b200 as pda
    from paged_decode_attention_b200 import decode as pdec, sharding, synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime

        # a rank that dies must not leave the others waiting for NCCL's ten-minute default
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=args.pg_timeout))

    w = synth.WORKLOADS[args.workload]
    kv_sharded = args.workload == "c4" and world > 1
    if kv_sharded:
        q, cache = sharding.make_kv_range_shard(args.workload, rank, world, dev, seed=args.seed)
        runner = sharding.KVRangeShardedDecoder(q, cache, group=dist.group.WORLD, kernel=args.kernel,
                                                exchange=args.exchange)
        for _ in range(2):
            runner.step()
        if not args.no_graph:
            runner.capture()  # decode + all-gather + merge replayed as one CUDA graph
        step = runner.step
        launches_per_step = runner.launches_per_step
    else:
        q, cache = synth.make(args.workload, device=dev, seed=args.seed + rank,
                              batch=args.batch or None, seq_len=args.seq_len or None)
        out = torch.empty_like(q)
        dargs = pdec.build_args(q, cache, out, kernel=args.kernel,
                                num_splits=args.num_splits if args.num_splits else None)
        kernel_used = pdec.selected_kernel(dargs)

        prepared = pda.DecodeStep(q, cache, out, kernel=args.kernel,
                                  num_splits=args.num_splits if args.num_splits else None)
        step = prepared.step

        launches_per_step = 1 if (kernel_used == "stream" or pdec.workspace_bytes(dargs) == 0) else 2
    my_bytes = cache.bytes_read_per_decode_step()
    resident = sum(t.numel() * t.element_size() for t in (cache.k_cache, cache.v_cache))

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()

    # optional: the same steps replayed from a CUDA graph, to see GPU time without host launch gaps
    graph_us = None
    if args.graph_steps > 0 and not kv_sharded:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(args.graph_steps):
                step()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(1, args.steps // args.graph_steps)
        g0.record()
        for _ in range(reps):
            graph.replay()
        g1.record()
        torch.cuda.synchronize()
        graph_us = g0.elapsed_time(g1) * 1e3 / (reps * args.graph_steps)

    # ---- device-timed region: K steps, CUDA events on the launching stream -------------
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(local, enabled=rank == 0) as clocks:
        t_wall0 = time.perf_counter()
        for i in range(args.steps):
            starts[i].record()
            step()
            stops[i].record()
        sync_all()
        t_wall = time.perf_counter() - t_wall0
        # keep the sampler alive long enough to see the GPU under load for short regions
        if t_wall < 0.5:
            # the same number of extra steps on every rank: a step may contain a collective
            extra = torch.tensor([int(0.6 / max(t_wall / args.steps, 1e-6))], device=dev, dtype=torch.int64)
            if world > 1:
                dist.all_reduce(extra, op=dist.ReduceOp.MAX)
            for _ in range(min(int(extra.item()), 20000)):
                step()
            torch.cuda.synchronize()
    per_step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    total_ms = starts[0].elapsed_time(stops[-1])
    t = torch.tensor([total_ms, statistics.median(per_step_ms), min(per_step_ms)], device=dev,
                     dtype=torch.float64)
    tot_bytes = torch.tensor([float(my_bytes)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot_bytes, op=dist.ReduceOp.SUM)
    total_ms, med_ms, min_ms = (float(x) for x in t.tolist())
    job_bytes = float(tot_bytes.item())
    ms_per_step = total_ms / args.steps
    value = job_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the host-buffer entry point -------------------------------
    e2e = None
    if not kv_sharded:
        host = pda.HostDecoder(cache, kernel=args.kernel)
        q_h = q.cpu().pin_memory()
        bt_h = cache.block_table.cpu().pin_memory()
        sl_h = cache.seq_lens.cpu().pin_memory()
        out_h = torch.empty(q.shape, dtype=q.dtype).pin_memory()
        for _ in range(3):
            host.step(q_h, bt_h, sl_h, out_h)
        sync_all()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            host.step(q_h, bt_h, sl_h, out_h)
        torch.cuda.synchronize()
        e2e_s = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
        e2e_step = float(e2e_s.item()) / args.steps
        e2e = {"value": job_bytes / e2e_step / 1e9, "unit": "GB/s", "us_per_call": e2e_step * 1e6,
               "h2d_bytes_per_step": host.h2d_bytes, "d2h_bytes_per_step": host.d2h_bytes,
               "note": "pd_decode_host: q, block table and lengths from pinned host memory, result "
                       "copied back; the KV pages are device state and stay in HBM"}
    else:
        e2e = {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "note": "KV-range-sharded run has no host-buffer entry point; same as value"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = _peaks()
    per_gpu_gbs = my_bytes / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "us_per_call": ms_per_step * 1e3,
        "us_per_call_median": med_ms * 1e3, "us_per_call_min": min_ms * 1e3,
        "higher_is_better": True, "scaling": "strong" if kv_sharded else "weak",
        "vs_baseline": None, "dtype": "f16 tensor-core tiles, f32 softmax and accumulation",
        "data": "synthetic",
        "pct_of_8tbs": 100.0 * value / world / 8000.0,
        "config": {"workload": f"{args.workload}: {w.description}", "seed": args.seed,
                   "kernel": args.kernel, "batch": int(q.shape[0]), "kv_bytes_per_gpu": my_bytes, "kv_bytes_job": job_bytes,
                   "resident_pool_bytes_per_gpu": resident,
                   "l2": f"inputs ({resident / 1e6:.0f} MB per GPU) exceed the {L2_BYTES >> 20} MB L2"
                         if resident > 2 * L2_BYTES else "inputs fit in L2: latency-bound, no HBM claim",
                   "parallelism": (f"kv-range sharding + {args.exchange} exchange + merge" if kv_sharded
                                   else f"request sharding x{world}, no communication")},
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s",
                     "frac": per_gpu_gbs / peak, "peak_kind": f"of {peak_kind}",
                     "traffic": (my_bytes * NCU_TRAFFIC_RATIO[args.workload]
                                 if args.workload in NCU_TRAFFIC_RATIO and not args.batch else None),
                     "note": "achieved = algorithmic KV bytes of rank 0 / mean step time (memset + the one "
                             "decode launch); traffic = DRAM bytes per launch, scaled from the ncu "
                             "capture of a smaller batch of the same shape (profiles/)"},
        "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
        "api": "DecodeStep.step (paged_decode prepared once; same C-ABI call pd_decode)",
    }
    if graph_us is not None:
        line["us_per_call_cuda_graph"] = graph_us
    if world == 1 and not args.no_cpu:
        r = cpu_port_timing(cache, q, steps=2, warmup=1, budget_tokens=args.cpu_tokens)
        line["cpu_baseline"] = {"value": r["bytes"] / r["torch_s"] / 1e9, "unit": "GB/s",
                                "cores": r["torch_threads"], "kind": "port", "sample": r["sample"],
                                "s_per_pass": r["torch_s"]}
        line["cpu_port_c"] = {"value": r["bytes"] / r["c_s"] / 1e9, "unit": "GB/s",
                              "cores": r["c_threads"], "s_per_pass": r["c_s"],
                              "note": "fused C/OpenMP restatement on the same sample"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=("c1", "c2", "c3", "c4", "c5"), default="c2")
    ap.add_argument("--kernel", choices=("auto", "simple", "stream"), default="auto")
    ap.add_argument("--num-splits", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--batch", type=int, default=0,
                    help="shrink the workload to this many requests (profiling captures)")
    ap.add_argument("--seq-len", type=int, default=0, help="force one length for every request")
    ap.add_argument("--cpu-tokens", type=int, default=40000,
                    help="size of the CPU sample in tokens")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--exchange", choices=("nccl", "peer"), default="nccl",
                    help="KV-range-sharded runs: NCCL all-gather + merge, or direct peer stores + merge")
    ap.add_argument("--no-graph", action="store_true",
                    help="KV-range-sharded runs: issue the step from the host instead of a CUDA graph")
    ap.add_argument("--pg-timeout", type=int, default=120, help="process-group timeout in seconds")
    ap.add_argument("--graph-steps", type=int, default=0,
                    help="also time this many steps per CUDA-graph replay (GPU time without host gaps)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
