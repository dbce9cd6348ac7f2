"""Multi-GPU partitioning of the decode path: one process per GPU.

Two schemes, neither present in the reference (a single-GPU kernel):

* **Request sharding** — every (request, kv head) is independent
  (pagedattn/triton_decode.py:10-12), so a ragged batch is split across ranks by
  request, balanced by token count; each rank decodes the requests whose pages it holds
  and nothing is exchanged.  ``partition_requests`` computes the assignment on the host.

* **KV-range sharding** — for few, very long requests each rank holds a contiguous slice
  of every request's tokens in its own page pool, decodes it to a normalised fp32 partial
  plus its base-2 log-sum-exp, the ranks all-gather the partials (``B*Hq*(D+1)`` floats
  per rank over NCCL/NVLink) and every rank merges them with the log-sum-exp merge kernel
  — the same arithmetic that merges split-KV partials inside one GPU
  (pagedattn/triton_decode.py:221-240).
"""

from __future__ import annotations

import heapq
from typing import Callable, Sequence

import torch
import torch.distributed as dist

from . import synth
from .cache import PagedKVCache


def partition_requests(seq_lens: Sequence[int], world: int) -> list[list[int]]:
    """Token-balanced assignment of request indices to ``world`` ranks.

    Longest-first greedy: the next longest request goes to the rank with the fewest
    tokens so far (ties to the lower rank).  Deterministic; every request appears once.
    """
    if world <= 0:
        raise ValueError("world must be positive")
    heap = [(0, r) for r in range(world)]
    heapq.heapify(heap)
    shards: list[list[int]] = [[] for _ in range(world)]
    for idx in sorted(range(len(seq_lens)), key=lambda i: (-int(seq_lens[i]), i)):
        load, r = heapq.heappop(heap)
        shards[r].append(idx)
        heapq.heappush(heap, (load + int(seq_lens[idx]), r))
    for s in shards:
        s.sort()
    return shards


def token_ranges(seq_len: int, world: int, align: int) -> list[tuple[int, int]]:
    """Contiguous [lo, hi) token slices of one request for ``world`` ranks.

    Boundaries are multiples of ``align`` (the page size) so a page never straddles two
    ranks; trailing ranks may get an empty slice when the request is short.
    """
    pages = -(-seq_len // align)
    per = -(-pages // world)
    out = []
    for r in range(world):
        lo = min(r * per * align, seq_len)
        hi = min((r + 1) * per * align, seq_len)
        out.append((lo, hi))
    return out


def make_kv_range_shard(name: str, rank: int, world: int, device, seed: int = 0,
                        batch: int | None = None, seq_len: int | None = None):
    """This rank's slice of a KV-range-sharded synthetic workload.

    All ranks share q (drawn from ``seed``); rank r's pool holds tokens
    ``token_ranges(seq_len, world, page)[r]`` of every request, drawn from ``seed + 1 + r``.
    """
    w = synth.WORKLOADS[name]
    full = int(synth.draw_lengths(name, torch.Generator().manual_seed(seed), batch, seq_len)[0])
    lo, hi = token_ranges(full, world, w.page)[rank]
    q, _ = synth.make(name, device=device, seed=seed, batch=batch, seq_len=w.page)
    _, cache = synth.make(name, device=device, seed=seed + 1 + rank, batch=batch, seq_len=max(hi - lo, 0))
    return q, cache


class PeerExchange:
    """Cross-rank merge of decode partials by direct peer stores.

    Every rank owns one exchange buffer in torch symmetric memory, mapped into all peers.  A
    step stores this rank's partial (fp32 results then lses) into every rank's buffer over
    NVLink (every value as a word that carries the step's mark, so nothing is fenced or
    flagged) and merges the partials that arrive in its own buffer.  Two
    forms: ``step()`` pushes a finished flat partial with a small kernel and merges
    (``pd_exchange_step``); ``fused_step(decode_args)`` lets the streaming decode kernel store
    each finished (request, kv head) unit itself and launches the merge behind it as a
    programmatic dependent (``pd_decode_exchange``).  Plain peer stores only — no multicast,
    nothing is loaded from a peer's memory — and the wait for the words is bounded
    (``PD_DEV_TIMEOUT`` in ``status`` after one second).
    """

    def __init__(self, local: torch.Tensor | None, out: torch.Tensor, group, status: torch.Tensor | None = None):
        import ctypes
        import os

        # the exchange buffer must be reachable by plain stores only: no NVLink multicast binding
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
        import torch.distributed._symmetric_memory as symm_mem

        from . import _cabi

        b, hq, d = out.shape
        if local is not None and (local.numel() != b * hq * (d + 1) or local.dtype != torch.float32
                                  or not local.is_contiguous()):
            raise ValueError("local must be the flat fp32 partial: B*Hq*D results then B*Hq lses")
        if not out.is_contiguous():
            raise ValueError("out must be contiguous")
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        nbytes = int(_cabi.load().pd_exchange_bytes(self.world, b * hq, d))
        if nbytes == 0:
            raise ValueError("exchange supports at most 16 ranks")
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=out.device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group)
        if int(getattr(self.handle, "multicast_ptr", 0) or 0) != 0:
            raise RuntimeError("the exchange buffer was bound to an NVLink multicast object; "
                               "set TORCH_SYMM_MEM_DISABLE_MULTICAST=1 before torch initialises symmetric memory")
        torch.cuda.synchronize(out.device)
        dist.barrier(group)  # every buffer is zero before anybody pushes
        self._ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self.handle.buffer_ptrs])
        a = _cabi.PdExchangeArgs()
        a.peer_bufs = ctypes.cast(self._ptrs, ctypes.POINTER(ctypes.c_void_p))
        a.world, a.rank = self.world, self.rank
        if local is not None:
            a.local = local.data_ptr()
        a.rows, a.head_dim, a.rows_per_batch = b * hq, d, hq
        a.out, a.out_stride_b, a.out_stride_h = out.data_ptr(), hq * d, d
        a.io_dtype = _cabi.IO_CODE[out.dtype]
        if status is not None:
            a.status = status.data_ptr()
        self._keep = (local, out, status)
        self.args, self._ref = a, ctypes.byref(a)
        self._step, self._fused = _cabi.load().pd_exchange_step, _cabi.load().pd_decode_exchange
        self.device = out.device

    def step(self) -> None:
        from . import _cabi

        self.args.stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._step(self._ref)
        if rc != 0:
            _cabi.check(rc, "pd_exchange_step")

    def fused_step(self, decode_args) -> None:
        """Decode + push + merge in two launches; ``decode_args`` is a prepared ``PdDecodeArgs``."""
        import ctypes

        from . import _cabi

        stream = torch.cuda.current_stream(self.device).cuda_stream
        self.args.stream = decode_args.stream = stream
        rc = self._fused(ctypes.byref(decode_args), self._ref)
        if rc != 0:
            _cabi.check(rc, "pd_decode_exchange")


class KVRangeShardedDecoder:
    """Decode step of one rank of a KV-range-sharded group.

    ``step()`` = local decode to (fp32 partial, lse) -> exchange -> merge of ``world`` partials
    into ``out``.  ``exchange`` picks how the partials travel: ``"nccl"`` (one all-gather of the
    flat partial through the group's backend, then the merge kernel; the default, and the only
    one for CPU stand-ins over gloo), ``"peer"`` (a push kernel stores it into every rank's
    buffer, a merge kernel waits for it), ``"fused"`` (the decode kernel stores each
    finished unit itself; the merge is launched behind it as a programmatic dependent).
    ``decode_fn``/``merge_fn`` default to the CUDA library; host-side tests inject CPU
    stand-ins to exercise the plumbing over gloo.

    Call ``close()`` on every rank before ``destroy_process_group``: a captured step that
    contains an NCCL all-gather keeps a reference on the communicator, and tearing the
    communicator down while that graph is alive waits for it for ever.
    """

    def __init__(self, q: torch.Tensor, cache: PagedKVCache, group=None, kernel: str = "auto",
                 decode_fn: Callable | None = None, merge_fn: Callable | None = None,
                 exchange: str = "nccl", status: torch.Tensor | None = None):
        if exchange not in ("nccl", "peer", "fused"):
            raise ValueError("exchange must be 'nccl' (all-gather + merge), 'peer' (push kernel + merge) "
                             "or 'fused' (the decode kernel pushes)")
        self.q, self.cache, self.group, self.kernel = q, cache, group, kernel
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.exchange = exchange
        b, hq, d = q.shape
        self.n_o = b * hq * d
        self.local = torch.empty(self.n_o + b * hq, dtype=torch.float32, device=q.device)
        self.f32 = self.local[: self.n_o].view(b, hq, d)
        self.lse = self.local[self.n_o:].view(b, hq)
        self.gathered = torch.empty((self.world, self.local.numel()), dtype=torch.float32, device=q.device)
        self.parts = self.gathered[:, : self.n_o].view(self.world, b, hq, d)
        self.lses = self.gathered[:, self.n_o:].view(self.world, b, hq)
        self.out = torch.empty_like(q)
        self.graph = None
        self.steps_per_replay = 1
        self._decode_step = None
        if decode_fn is None:
            from .decode import DecodeStep, MergeStep

            fused = exchange == "fused" and dist.is_initialized()
            self._decode_step = DecodeStep(q, cache, None, kernel=kernel, status=status, no_output=True) if fused \
                else DecodeStep(q, cache, None, result_f32=self.f32, result_lse=self.lse, kernel=kernel)
            merge_step = MergeStep(self.parts, self.lses, self.out)
            decode_fn = lambda *_: self._decode_step.step()
            merge_fn = lambda *_: merge_step.step()
        self.decode_fn, self.merge_fn = decode_fn, merge_fn
        self.launches_per_step = 2  # decode (merges its own splits), the cross-rank merge
        self.peer = None
        if exchange in ("peer", "fused") and dist.is_initialized():
            self.peer = PeerExchange(None if exchange == "fused" else self.local, self.out, group, status=status)
            self.launches_per_step = 2 if exchange == "fused" else 3  # decode, [push,] wait-and-merge

    def _run(self) -> None:
        if self.peer is not None and self.exchange == "fused" and self._decode_step is not None:
            self.peer.fused_step(self._decode_step.args)
            return
        self.decode_fn(self.q, self.cache, self.f32, self.lse, self.kernel)
        if self.peer is not None:
            self.peer.step()
            return
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered.view(-1), self.local, group=self.group)
        else:
            self.gathered[0].copy_(self.local)
        self.merge_fn(self.parts, self.lses, self.out)

    def capture(self, steps: int = 1) -> None:
        """Record the whole step into one CUDA graph; ``step`` then replays it.

        ``steps`` > 1 records that many consecutive steps into the one graph (a serving engine's
        graph holds a whole model step with one decode per layer; a measurement wants the device
        time of a step without one graph launch per step); ``steps_per_replay`` says how many
        steps a ``step()`` call then runs.

        At eight ranks a rank's slice of a long request decodes in a few tens of
        microseconds, less than the host needs to issue the operations; replaying a graph
        takes the host out of the step.  Every rank of the group must call this at the same
        point (an all-gather is captured collectively), after at least one plain step.
        """
        side = torch.cuda.Stream(device=self.q.device)
        side.wait_stream(torch.cuda.current_stream(self.q.device))
        with torch.cuda.stream(side):
            self._run()
        torch.cuda.current_stream(self.q.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(max(1, int(steps))):
                self._run()
        self.graph = graph
        self.steps_per_replay = max(1, int(steps))

    def step(self) -> torch.Tensor:
        if self.graph is not None:
            self.graph.replay()
        else:
            self._run()
        return self.out

    def close(self) -> None:
        """Waits for this rank's work and releases the captured graph.

        Collective in effect, not in form: every rank must have called it before any rank
        destroys the process group (a barrier between the two is the caller's).  Safe to call
        twice; ``step`` falls back to host-issued launches afterwards.
        """
        if self.q.is_cuda:
            torch.cuda.synchronize(self.q.device)
        graph, self.graph = self.graph, None
        self.steps_per_replay = 1
        if graph is not None:
            graph.reset()
            del graph
        if self.q.is_cuda:
            torch.cuda.synchronize(self.q.device)
