"""Benchmark of the paged decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

One step is one decode call (one launch of the streaming decode kernel, which merges its own
partial results) over one synthetic batch of the named workload.  The headline line is
workload c2 (the Llama-3-8B-shaped batch the target is quoted on).  The metric is HBM GB/s
over the algorithmic KV bytes of the batch (2 * sum(seq_lens) * Hkv * D * elem + scale
bytes), with microseconds per call beside it.

Rank 0 prints ONE JSON line.  `value` is timed with CUDA events on the launching stream with
everything resident in HBM; `e2e` goes through the host-buffer entry point (pd_decode_host)
with q, block table and lengths copied from pinned host memory and the result copied back
inside the timed region; `roofline` relates the decode step to the measured copy bandwidth
of this pool; `cpu_baseline` times the CPU port of the reference's algorithm on this box's
cores over the same full batch.  `--impl reference` times only that CPU port.

Beside the headline the line carries, when the headline workload is c2:
  * at one GPU, `workloads`: the other four configurations (c1, c3, c4, c5) measured the
    same way (events, CUDA graph, end to end, roofline, clocks);
  * at N > 1 GPUs (one process per GPU), the headline is weak scaling (every rank decodes
    its own batch, nothing is exchanged), `kv_range_sharded` is the long-context workload c4
    with its KV range cut over the ranks and the partial results merged across GPUs (strong
    scaling, the one path with cross-GPU traffic) together with a parity figure of a small
    sharded case, and `workloads.c5` is ONE seeded ragged batch whose requests are dealt to
    the ranks by the token-balancing partitioner (strong scaling, no communication).
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
# the exchange buffers of the KV-range-sharded block are written with plain peer stores only:
# keep torch's symmetric memory from binding them to an NVLink multicast object (read when it
# first allocates, so set before torch is imported)
os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"

METRIC = "decode_attn_hbm_gbs"
# DRAM bytes moved per algorithmic byte, from one ncu capture of the streaming kernel per
# workload shape (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic KV bytes of
# the captured case; see profiles/).  Traffic grows in proportion to the tokens processed, so
# the ratio scales a full launch.
NCU_TRAFFIC_RATIO = {"c2": 1.013, "c3": 1.021, "c4": 1.013, "c5": 1.022}
L2_BYTES = 126 << 20
FALLBACK_HBM_GBS = 6650.0
CPU_SUB_BATCH = 8  # requests per call of the CPU port: bounds its dense [b, Hkv, S_max, D] temporaries


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
        # the idle samples before the first step would drag the median down: keep the upper half
        busy = sorted(sm)[len(sm) // 2:] if len(sm) > 3 else sm
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# the CPU port (reference arm and cpu_baseline leg)
# ------------------------------------------------------------------------------------------------
def cpu_port_timing(cache, q, steps: int, warmup: int, budget_tokens: int = 0):
    """Times the CPU ports of the reference's path.

    With ``budget_tokens == 0`` a pass is the WHOLE batch, fed to the port ``CPU_SUB_BATCH``
    requests at a time (the port gathers dense [b, Hkv, S_max, D] tensors like the reference
    does; sub-batching bounds them and changes results by rounding only).  With a budget a
    pass is a prefix of the batch holding about that many tokens.
    """
    import torch

    from oracle import adapters, c_oracle, torch_port
    from paged_decode_attention_b200 import synth

    lens = cache.seq_lens.cpu().tolist()
    rows_all = list(range(len(lens)))
    if budget_tokens > 0:
        rows_all, total = [], 0
        for i, n in enumerate(lens):
            if rows_all and total + n > budget_tokens:
                break
            rows_all.append(i)
            total += int(n)
    groups = [rows_all[i:i + CPU_SUB_BATCH] for i in range(0, len(rows_all), CPU_SUB_BATCH)]
    subs = []
    nbytes = 0
    for rows in groups:
        oc = adapters.from_torch_cache(synth.take_requests(cache, rows))
        subs.append((adapters.q_to_f32(q[rows]), oc))
        nbytes += oc.bytes_read_per_decode_step()
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

    t_torch = timed(lambda: [torch_port.decode(qf, oc) for qf, oc in subs])
    t_c = timed(lambda: [c_oracle.decode(qf, oc, num_threads=threads) for qf, oc in subs])
    whole = len(rows_all) == len(lens)
    sample = (f"{'the whole batch: ' if whole else ''}{len(rows_all)} of {len(lens)} requests, "
              f"{sum(lens[i] for i in rows_all)} tokens, {nbytes / 1e6:.1f} MB of KV, in calls of "
              f"{CPU_SUB_BATCH} requests; torch-on-CPU restatement of reference_decode (gather + fp32 "
              f"attention), {steps} timed passes after {warmup} warm-up")
    return {
        "torch_s": statistics.mean(t_torch), "c_s": statistics.mean(t_c), "bytes": nbytes,
        "threads": threads, "torch_threads": torch.get_num_threads(),
        "c_threads": c_oracle.max_threads(), "sample": sample, "rows": len(rows_all), "whole": whole,
    }


def _config(workload: str, seed: int, batch: int, job_bytes: float) -> dict:
    """The workload description both arms print (identical for the same batch)."""
    from paged_decode_attention_b200 import synth

    return {"workload": f"{workload}: {synth.WORKLOADS[workload].description}", "seed": seed,
            "batch": batch, "kv_bytes_job": float(job_bytes)}


def run_reference(args) -> None:
    """--impl reference: the CPU port of the reference's path over the same batch, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    from paged_decode_attention_b200 import synth

    w = synth.WORKLOADS[args.workload]
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    # the same seeded batch as the GPU arm when a GPU is present (pages are drawn on the
    # device); a smaller draw of the same distribution on a box without one
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
        "config": _config(args.workload, args.seed, int(q.shape[0]), float(cache.bytes_read_per_decode_step())),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": r["torch_threads"], "kind": "port",
                         "sample": r["sample"]},
        "cpu_port_c": {"value": r["bytes"] / r["c_s"] / 1e9, "unit": "GB/s", "cores": r["c_threads"],
                       "note": "fused C/OpenMP restatement over the same requests"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# the GPU arm
# ------------------------------------------------------------------------------------------------
class Env:
    """Rank, device and the collective helpers of one bench process."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.args = torch, dist, args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}; launch with torch.distributed.run")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import datetime

            # a rank that dies must not leave the others waiting for NCCL's ten-minute default
            dist.init_process_group("nccl", device_id=self.dev,
                                    timeout=datetime.timedelta(seconds=args.pg_timeout))

    def sync_all(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def reduce(self, values, op: str):
        """max or sum over ranks of a list of floats."""
        t = self.torch.tensor([float(v) for v in values], device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.SUM)
        return [float(x) for x in t.tolist()]


def timed_steps(env: Env, step, steps: int, warmup: int, graph_steps: int = 0, collective: bool = False):
    """Device-timed region: `steps` calls of `step` between CUDA events on the launching stream.

    Returns (ms per step over the whole region, median ms, min ms, µs per step replayed from a
    CUDA graph or None, clock summary), each time the max over ranks.
    """
    torch = env.torch
    for _ in range(max(warmup, 3)):
        step()
    env.sync_all()
    graph_us = None
    if graph_steps > 0 and not collective:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(graph_steps):
                step()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(1, steps // graph_steps)
        g0.record()
        for _ in range(reps):
            graph.replay()
        g1.record()
        torch.cuda.synchronize()
        graph_us = g0.elapsed_time(g1) * 1e3 / (reps * graph_steps)
        del graph
        env.sync_all()
    # The timed region: exactly `steps` calls between ONE pair of events (events between the calls
    # would put two more stream operations into every step).  A second pass with an event pair
    # per call gives the spread (median, minimum); it is not part of the headline figure.
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    with ClockSampler(env.local, enabled=env.rank == 0) as clocks:
        t_wall0 = time.perf_counter()
        t0.record()
        for i in range(steps):
            step()
        t1.record()
        env.sync_all()
        t_wall = time.perf_counter() - t_wall0
        for i in range(steps):
            starts[i].record()
            step()
            stops[i].record()
        env.sync_all()
        # keep the sampler alive long enough to see the GPU under load for short regions
        if t_wall < 0.5:
            # the same number of extra steps on every rank: a step may contain a collective
            extra = int(env.reduce([0.6 / max(t_wall / steps, 1e-6)], "max")[0])
            for _ in range(min(extra, 20000)):
                step()
            torch.cuda.synchronize()
    per_step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    total_ms = t0.elapsed_time(t1)
    total_ms, med_ms, min_ms = env.reduce([total_ms, statistics.median(per_step_ms), min(per_step_ms)], "max")
    if graph_us is not None:
        graph_us = env.reduce([graph_us], "max")[0]
    return total_ms / steps, med_ms, min_ms, graph_us, clocks.summary()


def e2e_steps(env: Env, cache, q, kernel: str, steps: int, job_bytes: float) -> dict:
    """The same call through pd_decode_host: inputs in pinned host memory, result into pinned host memory.

    Timed twice: the way `--e2e-direct` names (default: the kernels use the caller's buffers in
    place where that pays) and, for comparison, with every buffer staged through a device copy
    by cudaMemcpyAsync ahead of and behind the kernel."""
    import paged_decode_attention_b200 as pda

    torch = env.torch
    q_h = q.cpu().pin_memory()
    bt_h = cache.block_table.cpu().pin_memory()
    sl_h = cache.seq_lens.cpu().pin_memory()
    out_h = torch.empty(q.shape, dtype=q.dtype).pin_memory()

    def timed(host) -> float:
        # Warm-up by time as well as by count: pinning the host copies above leaves the GPU idle
        # for milliseconds, and the first steps after that run while its clocks are still coming
        # back up.
        warm_until, n = time.perf_counter() + 0.05, 0
        while n < max(3, env.args.warmup) or time.perf_counter() < warm_until:
            host.step(q_h, bt_h, sl_h, out_h)
            n += 1
        env.sync_all()
        t0 = time.perf_counter()
        for _ in range(steps):
            host.step(q_h, bt_h, sl_h, out_h)
        torch.cuda.synchronize()
        return env.reduce([time.perf_counter() - t0], "max")[0] / steps

    host = pda.HostDecoder(cache, kernel=kernel, direct=env.args.e2e_direct)
    e2e_step = timed(host)
    parts = host.direct.replace("both", "out+q").split("+")
    res = {"value": job_bytes / e2e_step / 1e9, "unit": "GB/s", "us_per_call": e2e_step * 1e6,
           "h2d_bytes_per_step": host.h2d_bytes, "d2h_bytes_per_step": host.d2h_bytes,
           "note": "pd_decode_host, every step: lengths copied from pinned host memory; query rows "
                   f"{'read by the kernel from the pinned host buffer (PD_FLAG_HOST_DIRECT_Q)' if 'q' in parts else 'copied likewise'}; block-table entries "
                   f"{'read by the kernel from the pinned host table (PD_FLAG_HOST_DIRECT_BT)' if 'bt' in parts else 'copied likewise'}; "
                   f"result rows {'written by the kernel into the pinned host buffer (PD_FLAG_HOST_DIRECT_OUT)' if 'out' in parts else 'copied back'}; "
                   "h2d/d2h bytes count the buffers' full sizes; the KV pages are device state and stay in HBM",
           "direct": host.direct}
    if parts != ["none"]:
        staged = timed(pda.HostDecoder(cache, kernel=kernel, direct="none"))
        res["all_buffers_staged"] = {"us_per_call": staged * 1e6, "value": job_bytes / staged / 1e9, "unit": "GB/s",
                                     "note": "the same steps with q, block table and lengths copied in and the result "
                                             "copied back by cudaMemcpyAsync around the kernel"}
    return res


def measure_request_sharded(env: Env, name: str, strong: bool) -> dict:
    """One workload whose requests shard with no communication.

    weak (`strong` false): every rank draws its own batch of the workload's shape.
    strong: ONE seeded batch; its requests are dealt to the ranks by partition_requests and
    each rank builds only the pages of its own requests.
    """
    import paged_decode_attention_b200 as pda
    from paged_decode_attention_b200 import decode as pdec, sharding, synth

    torch, args = env.torch, env.args
    w = synth.WORKLOADS[name]
    extra = {}
    if strong and env.world > 1:
        lens = synth.draw_lengths(name, torch.Generator().manual_seed(args.seed))
        shards = sharding.partition_requests(lens.tolist(), env.world)
        mine = shards[env.rank]
        q, cache = synth.make(name, device=env.dev, seed=args.seed + 1 + env.rank, lengths=lens[mine])
        loads = [int(lens[s].sum()) for s in shards]
        extra["token_imbalance_max_over_mean"] = max(loads) / (sum(loads) / len(loads))
        extra["requests_per_rank"] = [len(s) for s in shards]
    else:
        q, cache = synth.make(name, device=env.dev, seed=args.seed + env.rank,
                              batch=args.batch or None, seq_len=args.seq_len or None)
    out = torch.empty_like(q)
    ns = args.num_splits if args.num_splits else None
    kernel_used = pdec.selected_kernel(pdec.build_args(q, cache, out, kernel=args.kernel, num_splits=ns))
    prepared = pda.DecodeStep(q, cache, out, kernel=args.kernel, num_splits=ns, equal_tile_shares=args.equal_tile_shares)
    launches = 1 if (kernel_used == "stream" or pdec.workspace_bytes(prepared.args) == 0) else 2
    my_bytes = cache.bytes_read_per_decode_step()
    resident = sum(t.numel() * t.element_size() for t in (cache.k_cache, cache.v_cache))
    ms, med_ms, min_ms, graph_us, clocks = timed_steps(env, prepared.step, args.steps, args.warmup,
                                                       graph_steps=args.graph_steps)
    job_bytes = env.reduce([my_bytes], "sum")[0]
    e2e = e2e_steps(env, cache, q, args.kernel, args.steps, job_bytes)
    peak, peak_kind = _peaks()
    l2_resident = resident <= 2 * L2_BYTES
    per_gpu = my_bytes / (ms * 1e-3) / 1e9
    per_gpu_max = env.reduce([per_gpu], "max")[0]
    res = {
        "workload": f"{name}: {w.description}", "batch": int(q.shape[0]), "kernel": kernel_used,
        "scaling": "strong" if (strong and env.world > 1) else "weak",
        "us_per_call": ms * 1e3, "us_per_call_median": med_ms * 1e3, "us_per_call_min": min_ms * 1e3,
        "us_per_call_cuda_graph": graph_us,
        "value": job_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
        "kv_bytes_job": job_bytes, "kv_bytes_rank0": my_bytes, "resident_pool_bytes_rank0": resident,
        "l2": ("inputs fit in L2: latency-bound, microseconds only, no HBM claim" if resident <= L2_BYTES
               else f"inputs ({resident / 1e6:.0f} MB per GPU) are less than twice the {L2_BYTES >> 20} MB L2: "
                    "part of a step may be served from it, no HBM fraction claimed" if l2_resident
               else f"inputs ({resident / 1e6:.0f} MB per GPU) exceed the {L2_BYTES >> 20} MB L2"),
        "roofline": None if l2_resident else {
            "bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
            "peak_kind": f"of {peak_kind}", "best_rank_frac": per_gpu_max / peak,
            "traffic": (my_bytes * NCU_TRAFFIC_RATIO[name] if name in NCU_TRAFFIC_RATIO and not args.batch
                        else None)},
        "e2e": e2e, "clocks": clocks, "gpu_launches": launches * args.steps,
        "_objects": (q, cache),
    }
    if l2_resident:
        # Host cost of issuing a call (no device wait inside the loop; the kernel is shorter than
        # the host path, so the wall time per call is what the host spends): the one-shot entry
        # point that re-reads every tensor each call, and the prepared step.
        def host_us(fn, calls=300):
            for _ in range(20):
                fn()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(calls):
                fn()
            dt = time.perf_counter() - t0
            torch.cuda.synchronize()
            return dt / calls * 1e6

        res["host_us_per_call"] = {"paged_decode_one_shot": host_us(lambda: pda.paged_decode(q, cache, out=out)),
                                   "decode_step_prepared": host_us(prepared.step)}
    res.update(extra)
    return res


def measure_kv_range_sharded(env: Env) -> dict:
    """Workload c4 with its KV range cut over the ranks (strong scaling) + a parity figure."""
    import dataclasses

    import paged_decode_attention_b200 as pda
    from paged_decode_attention_b200 import sharding

    torch, dist, args = env.torch, env.dist, env.args
    status = torch.zeros(1, dtype=torch.int32, device=env.dev)

    # ---- parity on a small sharded case: merged result vs one decode of the whole sequence ----
    q, cache = sharding.make_kv_range_shard("c4", env.rank, env.world, env.dev, seed=3, batch=2, seq_len=8192)
    dec = sharding.KVRangeShardedDecoder(q, cache, group=dist.group.WORLD, kernel=args.kernel,
                                         exchange=args.exchange, status=status)
    for _ in range(3):
        got = dec.step().clone()
    dec.capture()
    replayed = dec.step().clone()
    torch.cuda.synchronize()
    dec.close()
    caches = [sharding.make_kv_range_shard("c4", r, env.world, env.dev, seed=3, batch=2, seq_len=8192)[1]
              for r in range(env.world)]
    cat8 = lambda ts: torch.cat([t.view(torch.uint8) for t in ts]).view(ts[0].dtype)
    first, at = caches[0], 0
    tables = []
    for c in caches:
        tables.append(c.block_table + at)
        at += c.num_blocks
    whole = dataclasses.replace(
        first, k_cache=cat8([c.k_cache for c in caches]), v_cache=cat8([c.v_cache for c in caches]),
        k_scale=torch.cat([c.k_scale for c in caches]), v_scale=torch.cat([c.v_scale for c in caches]),
        block_table=torch.cat(tables, dim=1), seq_lens=sum(c.seq_lens for c in caches))
    f32 = torch.empty(q.shape, dtype=torch.float32, device=env.dev)
    lse = torch.empty(q.shape[:2], dtype=torch.float32, device=env.dev)
    pda.paged_decode(q, whole, result_f32=f32, result_lse=lse, kernel=args.kernel)
    parity = float((got.float() - f32).abs().max())
    graph_equal = bool(torch.equal(got, replayed))
    parity, = env.reduce([parity], "max")
    del caches, whole, dec

    # ---- the full-size step, replayed from one CUDA graph ---------------------------------------
    q, cache = sharding.make_kv_range_shard("c4", env.rank, env.world, env.dev, seed=args.seed)
    runner = sharding.KVRangeShardedDecoder(q, cache, group=dist.group.WORLD, kernel=args.kernel,
                                            exchange=args.exchange, status=status)
    for _ in range(2):
        runner.step()
    # Several steps per graph: the device time of a step, without one graph launch per step (in a
    # serving engine the step sits inside the graph of a whole model step).
    per_replay = 1 if args.no_graph else max(1, args.graph_steps)
    if not args.no_graph:
        runner.capture(steps=per_replay)
    my_bytes = cache.bytes_read_per_decode_step()
    ms, med_ms, min_ms, _, clocks = timed_steps(env, runner.step, max(args.steps, 20), args.warmup, collective=True)
    ms, med_ms, min_ms = ms / per_replay, med_ms / per_replay, min_ms / per_replay
    torch.cuda.synchronize()
    job_bytes = env.reduce([my_bytes], "sum")[0]
    status_word = int(env.reduce([int(status.item())], "max")[0])
    runner.close()
    peak, peak_kind = _peaks()
    per_gpu = my_bytes / (med_ms * 1e-3) / 1e9
    return {
        "workload": "c4: long-context scaled fp8_e5m2 decode B4 x 131072, KV range cut over the ranks, "
                    "partial results merged across GPUs",
        "scaling": "strong", "exchange": args.exchange, "cuda_graph": not args.no_graph,
        "steps_per_graph_replay": per_replay,
        "us_per_call": ms * 1e3, "us_per_call_median": med_ms * 1e3, "us_per_call_min": min_ms * 1e3,
        "value": job_bytes / (med_ms * 1e-3) / 1e9, "unit": "GB/s", "value_is": "job bytes / median step",
        "kv_bytes_job": job_bytes, "kv_bytes_rank0": my_bytes,
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                     "peak_kind": f"of {peak_kind}",
                     "note": "per rank: this rank's slice of the KV bytes / median step time; the step "
                             "also holds the exchange and the cross-rank merge"},
        "clocks": clocks, "gpu_launches_per_step": runner.launches_per_step, "status_word": status_word,
        "parity_max_abs": parity, "parity_case": "B2 x 8192 tokens sharded over the ranks vs one decode of the "
                                                 "whole sequence on each rank (fp32 result)",
        "graph_replay_equals_host_issued": graph_equal,
    }


def _public(d: dict) -> dict:
    return {k: v for k, v in d.items() if not k.startswith("_")}


def run_ours(args) -> None:
    env = Env(args)
    torch, dist = env.torch, env.dist
    head = measure_request_sharded(env, args.workload, strong=args.scaling == "strong")
    q, cache = head["_objects"]
    line = {
        "metric": METRIC, "value": head["value"], "unit": "GB/s", "n_gpus": env.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": head["us_per_call"] / 1e3,
        "us_per_call": head["us_per_call"], "us_per_call_median": head["us_per_call_median"],
        "us_per_call_min": head["us_per_call_min"],
        "higher_is_better": True, "scaling": head["scaling"],
        "vs_baseline": None, "dtype": "f16 tensor-core tiles, f32 softmax and accumulation",
        "data": "synthetic",
        "pct_of_8tbs": 100.0 * head["value"] / env.world / 8000.0,
        "config": _config(args.workload, args.seed, head["batch"], head["kv_bytes_job"]),
        "details": {"kernel": head["kernel"], "kv_bytes_rank0": head["kv_bytes_rank0"],
                    "resident_pool_bytes_rank0": head["resident_pool_bytes_rank0"], "l2": head["l2"],
                    "parallelism": f"request sharding x{env.world}, no communication"},
        "roofline": head["roofline"] or {"bound": "hbm", "achieved": None, "peak": _peaks()[0], "unit": "GB/s",
                                         "frac": None, "traffic": None, "note": head["l2"]},
        "e2e": head["e2e"],
        "gpu_launches": head["gpu_launches"],
        "clocks": head["clocks"],
        "api": "DecodeStep.step (paged_decode prepared once; same C-ABI call pd_decode)",
    }
    if line["roofline"].get("frac") is not None:
        line["roofline"]["note"] = ("achieved = algorithmic KV bytes of rank 0 / mean step time (the one decode "
                                    "launch); traffic = DRAM bytes per launch, scaled from the ncu capture of a "
                                    "smaller batch of the same shape (profiles/)")
    if head["us_per_call_cuda_graph"] is not None:
        line["us_per_call_cuda_graph"] = head["us_per_call_cuda_graph"]
    for k in ("token_imbalance_max_over_mean", "requests_per_rank"):
        if k in head:
            line[k] = head[k]

    if env.world == 1 and not args.no_cpu:
        r = cpu_port_timing(cache, q, steps=1, warmup=1, budget_tokens=args.cpu_tokens)
        line["cpu_baseline"] = {"value": r["bytes"] / r["torch_s"] / 1e9, "unit": "GB/s",
                                "cores": r["torch_threads"], "kind": "port", "sample": r["sample"],
                                "s_per_pass": r["torch_s"]}
        line["cpu_port_c"] = {"value": r["bytes"] / r["c_s"] / 1e9, "unit": "GB/s",
                              "cores": r["c_threads"], "s_per_pass": r["c_s"],
                              "note": "fused C/OpenMP restatement over the same requests"}
    del q, cache, head
    torch.cuda.empty_cache()

    # the other configurations ride along with the default headline only
    if args.workload == "c2" and not args.only_headline and not args.batch and not args.seq_len:
        others = {}
        if env.world == 1:
            for name in ("c1", "c3", "c4", "c5"):
                others[name] = _public(measure_request_sharded(env, name, strong=False))
                torch.cuda.empty_cache()
        else:
            others["c5"] = _public(measure_request_sharded(env, "c5", strong=True))
            torch.cuda.empty_cache()
            line["kv_range_sharded"] = measure_kv_range_sharded(env)
        line["workloads"] = others
        line["gpu_launches_all_workloads"] = line["gpu_launches"] + sum(o["gpu_launches"] for o in others.values())

    # every rank has released its captured graphs and finished its work before any rank tears
    # the process group down
    env.sync_all()
    if env.rank == 0:
        print(json.dumps(line))
        sys.stdout.flush()
    if env.world > 1:
        dist.barrier()
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
    ap.add_argument("--cpu-tokens", type=int, default=0,
                    help="bound the CPU pass to a prefix of about this many tokens (0 = the whole batch)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--only-headline", action="store_true",
                    help="skip the other configurations and the KV-range-sharded block")
    ap.add_argument("--scaling", choices=("weak", "strong"), default="weak",
                    help="N > 1: every rank its own batch (weak) or one batch dealt to the ranks (strong)")
    ap.add_argument("--exchange", choices=("fused", "peer", "nccl"), default="fused",
                    help="KV-range-sharded block: the decode kernel stores its units into the peers' buffers "
                         "(fused), a push kernel does (peer), or NCCL all-gather + merge (nccl)")
    ap.add_argument("--equal-tile-shares", action="store_true",
                    help="streaming kernel: equal tile counts per worker instead of equal estimated times (A/B)")
    ap.add_argument("--e2e-direct", choices=("auto", "out+bt", "out", "none", "q", "both", "out+bt+q"), default="auto",
                    help="e2e: which pinned host buffers the kernels use in place instead of a staging copy "
                         "(PD_FLAG_HOST_DIRECT_OUT / _BT / _Q); none = every buffer staged (A/B)")
    ap.add_argument("--no-graph", action="store_true",
                    help="KV-range-sharded block: issue the step from the host instead of a CUDA graph")
    ap.add_argument("--pg-timeout", type=int, default=120, help="process-group timeout in seconds")
    ap.add_argument("--graph-steps", type=int, default=10,
                    help="also time this many steps per CUDA-graph replay (GPU time without host gaps)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
