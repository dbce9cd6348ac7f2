"""Python entry point of the decode path.

``paged_decode`` keeps the call shape of the reference's launcher
(``pagedattn/triton_decode.py:285-295``): ``(q, cache, out=None, block_n=64,
num_splits=None, per_page_bt=True, num_warps=4, num_stages=3, sm_scale=None)``; it is
also exported as ``paged_decode_triton`` so existing call sites keep working.  What it
keeps of the reference's behaviour:

* writes into ``out`` when given and returns it; allocates ``[B, Hq, D]`` in q's dtype
  otherwise (``:309-310``);
* ``sm_scale`` overrides ``head_dim ** -0.5`` and is never re-derived (``:298-299, 328``);
* asserts ``q.shape[-1] == cache.shape.head_dim`` and ``block_n % block_size == 0``
  (``:306-307``);
* runs on torch's current CUDA stream, no autograd;
* an explicit ``num_splits`` cuts every request's KV range by the reference's rule
  (``:78-82``) and merges the partial results by log-sum-exp.

What differs: ``num_splits=None`` never synchronises with the device (the reference
calls ``seq_lens.max().item()``, ``:320-326``); ``per_page_bt``, ``num_warps`` and
``num_stages`` are accepted and ignored (pages are always resolved once per page, and
the CUDA kernels fix their own warp and stage counts); the split scratch is cached per
(device, stream), not per shape.  All compute happens in the CUDA library behind the C
ABI; there is no CPU or PyTorch fallback.
"""

from __future__ import annotations

import ctypes
import threading

import torch

from . import _cabi
from .cache import PagedKVCache

_ws_lock = threading.Lock()
_ws_cache: dict[tuple[int, int], torch.Tensor] = {}
# Buffers handed out while a CUDA graph was being captured: the graph's nodes hold their raw
# address, so they stay referenced here for the life of the process even when a larger request
# later replaces them in the cache.
_ws_captured: list[torch.Tensor] = []

STATS = {"decode_launches": 0}


def pick_num_splits(batch: int, num_kv_heads: int, max_seq_len: int, sm_count: int, block_n: int) -> int:
    """Split count for the one-CTA-per-(request, kv head, split) kernel.

    Same signature and role as ``pagedattn/triton_decode.py:248-263``.  The policy is
    re-derived for a 148-SM part (see ``pd_pick_num_splits`` in the C ABI); the streaming
    kernel balances work by itself and does not need it.
    """
    return int(_cabi.load().pd_pick_num_splits(int(batch), int(num_kv_heads), int(max_seq_len),
                                               int(sm_count), int(block_n)))


def _workspace(device: torch.device, nbytes: int, stream: int | None = None) -> torch.Tensor | None:
    if nbytes == 0:
        return None
    if stream is None:
        stream = torch.cuda.current_stream(device).cuda_stream
    key = (device.index, stream)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        with _ws_lock:
            buf = _ws_cache.get(key)
            if buf is None or buf.numel() < nbytes:
                buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
                _ws_cache[key] = buf
    if torch.cuda.is_current_stream_capturing() and not any(buf is t for t in _ws_captured):
        with _ws_lock:
            _ws_captured.append(buf)
    return buf


def _call_on_device(device: torch.device, fn, *fn_args) -> int:
    """Runs a native entry point with `device` current (switching only when it is not)."""
    if device.index is None or torch.cuda.current_device() == device.index:
        return fn(*fn_args)
    with torch.cuda.device(device):
        return fn(*fn_args)


def build_args(q: torch.Tensor, cache: PagedKVCache, out: torch.Tensor | None, *, block_n: int = 64,
               num_splits: int | None = None, sm_scale: float | None = None, kernel: str = "auto",
               result_f32: torch.Tensor | None = None, result_lse: torch.Tensor | None = None,
               status: torch.Tensor | None = None, max_seq_len: int = 0,
               sm_count: int = 0, no_output: bool = False, equal_tile_shares: bool = False) -> _cabi.PdDecodeArgs:
    """Validated argument block for ``pd_decode`` (no workspace attached yet).

    ``no_output`` leaves ``out`` unset: only ``pd_decode_exchange`` takes such a block (its
    result leaves through the exchange buffers).  ``equal_tile_shares`` makes the streaming kernel
    cut the work into equal tile counts instead of equal estimated times (for A/B measurements).
    """
    if q.dim() != 3:
        raise ValueError("q must be [batch, num_q_heads, head_dim]")
    b, hq, d = q.shape
    assert d == cache.shape.head_dim, f"q head_dim {d} != cache head_dim {cache.shape.head_dim}"
    assert block_n % cache.block_size == 0, "BLOCK_N must be a multiple of the page size"
    if hq != cache.shape.num_q_heads:
        raise ValueError(f"q has {hq} heads, cache.shape says {cache.shape.num_q_heads}")
    if q.dtype not in _cabi.IO_CODE:
        raise ValueError(f"q dtype {q.dtype} not supported (fp16 or bf16)")
    if q.stride(2) != 1:
        raise ValueError("head_dim must be contiguous in q")
    if b != cache.batch:
        raise ValueError(f"q batch {b} != block_table rows {cache.batch}")
    if kernel not in _cabi.KERNEL_CODE:
        raise ValueError(f"kernel must be one of {sorted(_cabi.KERNEL_CODE)}")
    args = _cabi.PdDecodeArgs()
    _cabi.fill_cache_fields(args, cache)
    if args.num_kv_heads != cache.shape.num_kv_heads or args.block_size != cache.block_size:
        raise ValueError("cache tensors disagree with cache.shape / cache.block_size")
    args.q = q.data_ptr()
    args.q_stride_b, args.q_stride_h = q.stride(0), q.stride(1)
    if out is not None and not no_output:
        if out.shape != q.shape or out.dtype != q.dtype or out.stride(2) != 1:
            raise ValueError("out must match q in shape and dtype with head_dim contiguous")
        args.out = out.data_ptr()
        args.out_stride_b, args.out_stride_h = out.stride(0), out.stride(1)
    args.io_dtype = _cabi.IO_CODE[q.dtype]
    args.sm_scale = float(cache.shape.softmax_scale if sm_scale is None else sm_scale)
    args.num_splits = 0 if num_splits is None else int(num_splits)
    if args.num_splits < 0:
        raise ValueError("num_splits must be positive or None")
    args.block_n = int(block_n)
    args.kernel = _cabi.KERNEL_CODE[kernel]
    args.sm_count = int(sm_count)
    args.max_seq_len = int(max_seq_len)
    if equal_tile_shares:
        args.flags |= _cabi.FLAG_EQUAL_TILE_SHARES
    if (result_f32 is None) != (result_lse is None):
        raise ValueError("result_f32 and result_lse go together")
    if result_f32 is not None:
        if (result_f32.dtype != torch.float32 or result_lse.dtype != torch.float32
                or tuple(result_f32.shape) != (b, hq, d) or tuple(result_lse.shape) != (b, hq)
                or not result_f32.is_contiguous() or not result_lse.is_contiguous()):
            raise ValueError("result_f32 [B,Hq,D] and result_lse [B,Hq] must be contiguous fp32")
        args.result_f32, args.result_lse = result_f32.data_ptr(), result_lse.data_ptr()
    if status is not None:
        if status.dtype != torch.int32 or status.numel() < 1:
            raise ValueError("status must be an int32 tensor")
        args.status = status.data_ptr()
    return args


def workspace_bytes(args: _cabi.PdDecodeArgs) -> int:
    n = ctypes.c_uint64(0)
    _cabi.check(_cabi.load().pd_workspace_bytes(ctypes.byref(args), ctypes.byref(n)), "pd_workspace_bytes")
    return int(n.value)


def selected_kernel(args: _cabi.PdDecodeArgs) -> str:
    rc = _cabi.load().pd_select_kernel(ctypes.byref(args))
    if rc < 0:
        _cabi.check(rc, "pd_select_kernel")
    return _cabi.KERNEL_NAME[rc]


def paged_decode(
    q: torch.Tensor,
    cache: PagedKVCache,
    out: torch.Tensor | None = None,
    block_n: int = 64,
    num_splits: int | None = None,
    per_page_bt: bool = True,
    num_warps: int = 4,
    num_stages: int = 3,
    sm_scale: float | None = None,
    *,
    kernel: str = "auto",
    result_f32: torch.Tensor | None = None,
    result_lse: torch.Tensor | None = None,
    status: torch.Tensor | None = None,
    max_seq_len: int = 0,
) -> torch.Tensor:
    """Paged GQA decode attention: q ``[B, Hq, D]`` (fp16/bf16) -> ``[B, Hq, D]``.

    Keyword-only extras: ``kernel`` ("auto", "simple", "stream") pins the CUDA kernel;
    ``result_f32``/``result_lse`` additionally receive the fp32 result and its base-2
    log-sum-exp (what a cross-GPU merge needs); ``status`` is an int32 device word that
    collects the kernels' PD_DEV_* flags; ``max_seq_len`` is an optional host-side bound
    on ``seq_lens`` that refines the automatic split count.
    """
    del per_page_bt, num_warps, num_stages
    if not q.is_cuda:
        raise _cabi.NativeLibraryError("paged_decode runs on CUDA tensors only; there is no CPU path")
    if out is None:
        out = torch.empty((q.shape[0], q.shape[1], q.shape[2]), dtype=q.dtype, device=q.device)
    # A call over the same tensors (same addresses, shapes, strides and options) as an earlier one
    # reuses that call's validated argument block and its scratch size: a serving loop that calls
    # this entry point every step pays for the validation and the size query once.
    key = _call_key(q, cache, out, block_n, num_splits, sm_scale, kernel, result_f32, result_lse, status)
    hit = _args_cache.get(key)
    if hit is None:
        args = build_args(q, cache, out, block_n=block_n, num_splits=num_splits, sm_scale=sm_scale,
                          kernel=kernel, result_f32=result_f32, result_lse=result_lse, status=status,
                          max_seq_len=max_seq_len)
        need = ctypes.c_uint64(0)
        rc = _call_on_device(q.device, _cabi.load().pd_workspace_bytes, ctypes.byref(args), ctypes.byref(need))
        if rc != 0:
            _cabi.check(rc, "pd_workspace_bytes")
        if len(_args_cache) >= _ARGS_CACHE_CAP:
            _args_cache.pop(next(iter(_args_cache)))
        hit = _args_cache[key] = (args, int(need.value), ctypes.byref(args))
    args, need_bytes, ref = hit
    args.stream = torch.cuda.current_stream(q.device).cuda_stream
    args.max_seq_len = int(max_seq_len)
    ws = _workspace(q.device, need_bytes, args.stream)
    if ws is not None:
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
    rc = _call_on_device(q.device, _cabi.load().pd_decode, ref)
    if rc != 0:
        _cabi.check(rc, "pd_decode")
    STATS["decode_launches"] += 1
    return out


_ARGS_CACHE_CAP = 256
_args_cache: dict[tuple, tuple] = {}


def _call_key(q, cache, out, block_n, num_splits, sm_scale, kernel, result_f32, result_lse, status) -> tuple:
    """Everything an argument block is built from, as plain values (addresses, shapes, strides)."""
    k, v, bt, sl, ks, vs = cache.k_cache, cache.v_cache, cache.block_table, cache.seq_lens, cache.k_scale, cache.v_scale
    # the calling thread is part of the key: a cached block is refreshed in place (stream, scratch)
    # on every call, so two threads must not share one
    return (threading.get_ident(), q.data_ptr(), out.data_ptr(), k.data_ptr(), v.data_ptr(), bt.data_ptr(), sl.data_ptr(),
            q.shape, q.stride(), q.dtype, out.shape, out.stride(), out.dtype,
            k.shape, k.stride(), k.dtype, v.shape, v.stride(), v.dtype,
            bt.shape, bt.stride(), bt.dtype, sl.shape, sl.stride(), sl.dtype,
            None if ks is None else (ks.data_ptr(), ks.stride(), ks.dtype),
            None if vs is None else (vs.data_ptr(), vs.stride(), vs.dtype),
            cache.shape, cache.block_size, cache.kv_dtype, q.device,
            block_n, num_splits, sm_scale, kernel,
            None if result_f32 is None else (result_f32.data_ptr(), result_f32.shape, result_f32.stride(), result_f32.dtype),
            None if result_lse is None else (result_lse.data_ptr(), result_lse.shape, result_lse.stride(), result_lse.dtype),
            None if status is None else (status.data_ptr(), status.dtype, status.numel()))


class DecodeStep:
    """A decode call prepared once and replayed: for loops that decode into the same buffers.

    ``paged_decode`` re-reads every pointer, stride and size on each call.  When q, out and
    the cache tensors stay where they are between steps (a serving loop that updates the
    block table and lengths in place), that work can be done once: ``DecodeStep(q, cache,
    out)`` validates and fills the argument block and attaches the scratch, ``step()`` only
    refreshes the stream and crosses the C ABI.  Results are those of ``paged_decode``.
    """

    def __init__(self, q: torch.Tensor, cache: PagedKVCache, out: torch.Tensor | None = None, **kw):
        if not q.is_cuda:
            raise _cabi.NativeLibraryError("DecodeStep runs on CUDA tensors only; there is no CPU path")
        no_output = bool(kw.get("no_output"))
        self.out = None if no_output else (torch.empty_like(q) if out is None else out)
        self.device = q.device
        self._keep = (q, cache, self.out, kw.get("result_f32"), kw.get("result_lse"), kw.get("status"))
        self.args = build_args(q, cache, self.out, **kw)
        need = ctypes.c_uint64(0)
        probe = self.args
        if no_output:  # the size query wants a complete block; sizes do not depend on the pointer
            probe = _cabi.PdDecodeArgs.from_buffer_copy(self.args)
            probe.out = q.data_ptr()
        _cabi.check(_call_on_device(self.device, _cabi.load().pd_workspace_bytes, ctypes.byref(probe),
                                    ctypes.byref(need)), "pd_workspace_bytes")
        # Private scratch, zero-filled once: the step may be replayed on any stream, and since
        # every call leaves the merge counters at zero and nobody else writes here, the per-call
        # clear of the counters is not needed (PD_FLAG_COUNTERS_ZERO).
        self._ws = (torch.zeros(int(need.value), dtype=torch.uint8, device=self.device)
                    if need.value else None)
        if self._ws is not None:
            self.args.workspace, self.args.workspace_bytes = self._ws.data_ptr(), self._ws.numel()
            self.args.flags |= _cabi.FLAG_COUNTERS_ZERO
        self._fn = _cabi.load().pd_decode
        self._ref = ctypes.byref(self.args)

    def step(self) -> torch.Tensor:
        self.args.stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = _call_on_device(self.device, self._fn, self._ref)
        if rc != 0:
            _cabi.check(rc, "pd_decode")
        STATS["decode_launches"] += 1
        return self.out

    __call__ = step

    def step_at(self, q_ptr: int, out_ptr: int, block_table_ptr: int, seq_lens_ptr: int, stream: int,
                max_seq_len: int = 0) -> None:
        """One step with this step's buffers at new addresses, everything else as prepared.

        For a serving engine that hands over fresh views of the same shapes, strides and dtypes
        every step (its padded query and output buffers, its block table and lengths): only the
        five addresses, the stream and the optional length bound are refreshed, nothing is
        re-validated and no tensor object is made.  The caller vouches that the layouts are the
        ones the step was prepared with.
        """
        a = self.args
        a.q, a.out, a.block_table, a.seq_lens, a.stream = q_ptr, out_ptr, block_table_ptr, seq_lens_ptr, stream
        a.max_seq_len = max_seq_len
        rc = self._fn(self._ref)
        if rc != 0:
            _cabi.check(rc, "pd_decode")
        STATS["decode_launches"] += 1


# Drop-in name of the reference's entry point (pagedattn/triton_decode.py:285).
paged_decode_triton = paged_decode


def paged_decode_static(q: torch.Tensor, cache: PagedKVCache, out: torch.Tensor, *, block_n: int = 64,
                        num_splits: int | None = None, sm_scale: float | None = None,
                        status: torch.Tensor | None = None) -> torch.Tensor:
    """``paged_decode`` without any allocation: for callers that may not allocate device memory.

    Meant for code that runs where allocating is off limits — a process whose free HBM all
    went to the KV-page pool, or a plugin on an engine thread that must not touch the
    allocator.  ``out`` is therefore required (nothing is created here), and the kernel's
    scratch is the fixed ``STATIC_SCRATCH_BYTES`` (8 MiB) array inside the library instead
    of a torch buffer.  Requests the streaming kernel does not serve, or that need more
    scratch than that, raise; calls that may overlap on the GPU must be ordered by the
    caller because they share the array.  The first call on a device performs a one-time
    address look-up and should happen before any stream capture.
    """
    if not q.is_cuda:
        raise _cabi.NativeLibraryError("paged_decode_static runs on CUDA tensors only")
    if out is None:
        raise ValueError("paged_decode_static allocates nothing: pass `out`")
    args = build_args(q, cache, out, block_n=block_n, num_splits=num_splits, sm_scale=sm_scale,
                      kernel="stream", status=status)
    _cabi.check(_call_on_device(q.device, _cabi.load().pd_decode_static, ctypes.byref(args)),
                "pd_decode_static")
    return out


def merge_partials(part_out: torch.Tensor, part_lse: torch.Tensor, out: torch.Tensor | None = None,
                   *, io_dtype: torch.dtype = torch.float16, want_f32: bool = False):
    """Merge ``P`` partial results by log-sum-exp on the GPU.

    ``part_out`` is ``[P, B, Hq, D]`` fp32 (each normalised), ``part_lse`` ``[P, B, Hq]``
    fp32 in base 2, ``-inf`` for an empty partial; ``P`` may be splits of one GPU or the
    ranks of a KV-range-sharded group.  Returns ``out`` (``[B, Hq, D]`` in ``io_dtype``),
    or ``(out, merged_f32, merged_lse)`` when ``want_f32``.
    """
    if not part_out.is_cuda:
        raise _cabi.NativeLibraryError("merge_partials runs on CUDA tensors only")
    p, b, hq, d = part_out.shape
    # each partial must be dense; the partials themselves may be any distance apart
    if p and not part_out[0].is_contiguous():
        part_out = part_out.contiguous()
    if p and not part_lse[0].is_contiguous():
        part_lse = part_lse.contiguous()
    if out is None:
        out = torch.empty((b, hq, d), dtype=io_dtype, device=part_out.device)
    if not out.is_contiguous():
        raise ValueError("out must be contiguous")
    m = _cabi.PdMergeArgs()
    m.part_out, m.part_lse = part_out.data_ptr(), part_lse.data_ptr()
    m.out_stride_p, m.out_stride_row = part_out.stride(0), d
    m.lse_stride_p, m.lse_stride_row = part_lse.stride(0), 1
    m.num_parts, m.num_rows, m.head_dim = p, b * hq, d
    m.out, m.dst_stride_row, m.io_dtype = out.data_ptr(), d, _cabi.IO_CODE[out.dtype]
    f32 = lse = None
    if want_f32:
        f32 = torch.empty((b, hq, d), dtype=torch.float32, device=part_out.device)
        lse = torch.empty((b, hq), dtype=torch.float32, device=part_out.device)
        m.result_f32, m.result_lse = f32.data_ptr(), lse.data_ptr()
    m.stream = torch.cuda.current_stream(part_out.device).cuda_stream
    with torch.cuda.device(part_out.device):
        _cabi.check(_cabi.load().pd_merge(ctypes.byref(m)), "pd_merge")
    return (out, f32, lse) if want_f32 else out


class MergeStep:
    """``merge_partials`` prepared once for fixed buffers (see ``DecodeStep``)."""

    def __init__(self, part_out: torch.Tensor, part_lse: torch.Tensor, out: torch.Tensor):
        if not part_out.is_cuda:
            raise _cabi.NativeLibraryError("MergeStep runs on CUDA tensors only")
        p, b, hq, d = part_out.shape
        if not (part_out[0].is_contiguous() and part_lse[0].is_contiguous() and out.is_contiguous()):
            raise ValueError("each partial, each lse block and out must be dense")
        self._keep = (part_out, part_lse, out)
        self.out, self.device = out, part_out.device
        m = _cabi.PdMergeArgs()
        m.part_out, m.part_lse = part_out.data_ptr(), part_lse.data_ptr()
        m.out_stride_p, m.out_stride_row = part_out.stride(0), d
        m.lse_stride_p, m.lse_stride_row = part_lse.stride(0), 1
        m.num_parts, m.num_rows, m.head_dim = p, b * hq, d
        m.out, m.dst_stride_row, m.io_dtype = out.data_ptr(), d, _cabi.IO_CODE[out.dtype]
        self.args, self._ref, self._fn = m, ctypes.byref(m), _cabi.load().pd_merge

    def step(self) -> torch.Tensor:
        self.args.stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = _call_on_device(self.device, self._fn, self._ref)
        if rc != 0:
            _cabi.check(rc, "pd_merge")
        return self.out

    __call__ = step


class HostDecoder:
    """Decode steps for callers whose q, block table, lengths and result live in host memory.

    Owns device staging buffers for the per-step inputs and the output; the KV pages are
    device state and stay on the GPU.  ``step`` goes through ``pd_decode_host``: three
    host-to-device copies, the decode, the result back, one stream wait.  ``direct`` names the
    caller's pinned buffers the kernels use in place instead of a staging copy, joined by "+":
    ``"out"`` (result rows are written across the bus as they are finished, while the KV pages
    still stream: 3 to 13 % off a step of the five bench workloads), ``"bt"`` (the producers
    fetch the block-table entries they need across the bus instead of the whole padded table
    being copied first: up to 5 % more), ``"q"`` (every consumer warp fetches its group's query
    rows across the bus, whole lines into shared memory, when a request starts: 5 to 35 % more
    on batches of many requests, a few per cent worse where a few long requests are cut over all
    workers, which then all want the same rows at once; ``"both"`` = ``"out+q"``) or
    ``"none"``.  Default ``"auto"``: ``"out+bt"``, and ``"q"`` as well from 16 requests upwards.
    Pageable host tensors are always staged.
    """

    def __init__(self, cache: PagedKVCache, io_dtype: torch.dtype = torch.float16,
                 sm_scale: float | None = None, kernel: str = "auto", direct: str = "auto"):
        dev = cache.k_cache.device
        b, hq, d = cache.batch, cache.shape.num_q_heads, cache.shape.head_dim
        self.q_dev = torch.empty((b, hq, d), dtype=io_dtype, device=dev)
        self.out_dev = torch.empty_like(self.q_dev)
        self.cache = cache
        self.args = build_args(self.q_dev, cache, self.out_dev, sm_scale=sm_scale, kernel=kernel)
        # `direct`: which of the caller's pinned buffers the kernels use in place instead of the
        # staging buffers q_dev / out_dev (PD_FLAG_HOST_DIRECT_OUT, PD_FLAG_HOST_DIRECT_Q)
        bits = {"out": _cabi.FLAG_HOST_DIRECT_OUT, "q": _cabi.FLAG_HOST_DIRECT_Q, "bt": _cabi.FLAG_HOST_DIRECT_BT,
                "none": 0, "both": _cabi.FLAG_HOST_DIRECT_OUT | _cabi.FLAG_HOST_DIRECT_Q}
        if direct == "auto":
            direct = "out+bt+q" if b >= 16 else "out+bt"
        self.direct = direct
        for part in direct.split("+"):
            self.args.flags |= bits[part]
        need = ctypes.c_uint64(0)
        _cabi.check(_call_on_device(dev, _cabi.load().pd_workspace_bytes, ctypes.byref(self.args),
                                    ctypes.byref(need)), "pd_workspace_bytes")
        self.ws = torch.empty(int(need.value), dtype=torch.uint8, device=dev) if need.value else None
        if self.ws is not None:
            self.args.workspace, self.args.workspace_bytes = self.ws.data_ptr(), self.ws.numel()
        self._fn, self._ref = _cabi.load().pd_decode_host, ctypes.byref(self.args)
        self._io_key = self._io = self._io_ref = None
        self.h2d_bytes = (self.q_dev.numel() * 2 + cache.block_table.numel() * 4 + cache.seq_lens.numel() * 4)
        self.d2h_bytes = self.out_dev.numel() * 2

    def step(self, q_host: torch.Tensor, block_table_host: torch.Tensor, seq_lens_host: torch.Tensor,
             out_host: torch.Tensor) -> torch.Tensor:
        for t in (q_host, block_table_host, seq_lens_host, out_host):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("host tensors must be contiguous CPU tensors")
        # the same four buffers as the step before (a serving loop refills them in place): the
        # pointer block is reused
        key = (q_host.data_ptr(), block_table_host.data_ptr(), seq_lens_host.data_ptr(), out_host.data_ptr())
        if key != self._io_key:
            self._io = _cabi.PdHostIO(*key)
            self._io_ref, self._io_key = ctypes.byref(self._io), key
        dev = self.q_dev.device
        self.args.stream = torch.cuda.current_stream(dev).cuda_stream
        rc = _call_on_device(dev, self._fn, self._ref, self._io_ref)
        if rc != 0:
            _cabi.check(rc, "pd_decode_host")
        return out_host
