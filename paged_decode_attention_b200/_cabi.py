"""ctypes binding of libpaged_decode_b200.so (the C ABI of include/paged_decode.h).

This is the only place the Python host code crosses into native code.  There is no
fallback: if the shared object is missing or was built for another ABI version, loading
raises, and every public entry point of the package fails with that error.
"""

from __future__ import annotations

import ctypes
import pathlib

import torch

from .config import KV_CODE

_PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = _PKG / "libpaged_decode_b200.so"
ABI_VERSION = 2

KERNEL_CODE = {"auto": 0, "simple": 1, "stream": 2}
KERNEL_NAME = {1: "simple", 2: "stream"}
IO_CODE = {torch.float16: 0, torch.bfloat16: 1}

DEV_BAD_BLOCK = 1
DEV_TIMEOUT = 2

_c_i32, _c_i64, _c_u64, _c_vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_uint64, ctypes.c_void_p


class PdDecodeArgs(ctypes.Structure):
    _fields_ = [
        ("q", _c_vp), ("out", _c_vp),
        ("q_stride_b", _c_i64), ("q_stride_h", _c_i64),
        ("out_stride_b", _c_i64), ("out_stride_h", _c_i64),
        ("k_cache", _c_vp), ("v_cache", _c_vp),
        ("kv_stride_block", _c_i64), ("kv_stride_token", _c_i64), ("kv_stride_head", _c_i64),
        ("k_scale", _c_vp), ("v_scale", _c_vp),
        ("scale_stride_block", _c_i64), ("scale_stride_token", _c_i64),
        ("block_table", _c_vp), ("block_table_stride", _c_i64), ("seq_lens", _c_vp),
        ("batch", _c_i32), ("num_q_heads", _c_i32), ("num_kv_heads", _c_i32), ("head_dim", _c_i32),
        ("block_size", _c_i32), ("num_blocks", _c_i32), ("max_blocks_per_seq", _c_i32),
        ("kv_dtype", _c_i32), ("io_dtype", _c_i32),
        ("sm_scale", ctypes.c_float),
        ("num_splits", _c_i32), ("block_n", _c_i32), ("kernel", _c_i32), ("sm_count", _c_i32),
        ("max_seq_len", _c_i32),
        ("workspace", _c_vp), ("workspace_bytes", _c_u64),
        ("result_f32", _c_vp), ("result_lse", _c_vp),
        ("status", _c_vp), ("stream", _c_vp), ("flags", ctypes.c_uint32),
    ]


class PdHostIO(ctypes.Structure):
    _fields_ = [("q_host", _c_vp), ("block_table_host", _c_vp), ("seq_lens_host", _c_vp),
                ("out_host", _c_vp)]


class PdMergeArgs(ctypes.Structure):
    _fields_ = [
        ("part_out", _c_vp), ("part_lse", _c_vp),
        ("out_stride_p", _c_i64), ("out_stride_row", _c_i64),
        ("lse_stride_p", _c_i64), ("lse_stride_row", _c_i64),
        ("num_parts", _c_i32), ("num_rows", _c_i32), ("head_dim", _c_i32),
        ("out", _c_vp), ("dst_stride_row", _c_i64), ("io_dtype", _c_i32),
        ("result_f32", _c_vp), ("result_lse", _c_vp), ("stream", _c_vp),
    ]


class PdCacheWriteArgs(ctypes.Structure):
    _fields_ = [
        ("key", _c_vp), ("value", _c_vp), ("in_stride_token", _c_i64), ("in_stride_head", _c_i64),
        ("k_cache", _c_vp), ("v_cache", _c_vp),
        ("kv_stride_block", _c_i64), ("kv_stride_token", _c_i64), ("kv_stride_head", _c_i64),
        ("k_scale", _c_vp), ("v_scale", _c_vp),
        ("scale_stride_block", _c_i64), ("scale_stride_token", _c_i64),
        ("slot_mapping", _c_vp),
        ("num_tokens", _c_i32), ("num_kv_heads", _c_i32), ("head_dim", _c_i32),
        ("block_size", _c_i32), ("num_blocks", _c_i32), ("kv_dtype", _c_i32), ("io_dtype", _c_i32),
        ("status", _c_vp), ("stream", _c_vp),
    ]


class PdExchangeArgs(ctypes.Structure):
    _fields_ = [
        ("peer_bufs", ctypes.POINTER(_c_vp)), ("world", _c_i32), ("rank", _c_i32),
        ("local", _c_vp), ("rows", _c_i32), ("head_dim", _c_i32), ("rows_per_batch", _c_i32),
        ("out", _c_vp), ("out_stride_b", _c_i64), ("out_stride_h", _c_i64), ("io_dtype", _c_i32),
        ("result_f32", _c_vp), ("result_lse", _c_vp), ("status", _c_vp), ("stream", _c_vp),
        ("phases", _c_i32), ("wait_limit_ns", _c_u64),
    ]


class PdGatherArgs(ctypes.Structure):
    _fields_ = [("cache", ctypes.POINTER(PdDecodeArgs)), ("k_dense", _c_vp), ("v_dense", _c_vp),
                ("s_max", _c_i32)]


EXPORTS = ("pd_abi_version", "pd_status_string", "pd_decode", "pd_decode_host",
           "pd_workspace_bytes", "pd_select_kernel", "pd_pick_num_splits", "pd_merge", "pd_gather",
           "pd_decode_static", "pd_cache_write", "pd_selftest_bounded_wait", "pd_exchange_bytes",
           "pd_exchange_step", "pd_exchange_part_offset", "pd_decode_exchange", "pd_counter_bytes")

FLAG_COUNTERS_ZERO = 1
FLAG_EQUAL_TILE_SHARES = 2
FLAG_HOST_DIRECT_OUT = 4
FLAG_HOST_DIRECT_Q = 8
FLAG_HOST_DIRECT_BT = 16
FLAG_STAGE_Q = 32
EXCHANGE_SEND, EXCHANGE_MERGE = 1, 2

STATIC_SCRATCH_BYTES = 8 << 20
ERR_TOO_LARGE = -5

_lib = None


class NativeLibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """The loaded library; raises NativeLibraryError when it is absent or mismatched."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise NativeLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m paged_decode_attention_b200.build` "
            "(needs nvcc); this package has no non-CUDA path")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise NativeLibraryError(f"{LIB_PATH} does not export {name}")
    lib.pd_abi_version.restype = ctypes.c_int
    if lib.pd_abi_version() != ABI_VERSION:
        raise NativeLibraryError(f"{LIB_PATH} has ABI {lib.pd_abi_version()}, expected {ABI_VERSION}")
    lib.pd_status_string.restype = ctypes.c_char_p
    lib.pd_status_string.argtypes = [ctypes.c_int]
    for name in ("pd_decode", "pd_select_kernel", "pd_decode_static"):
        getattr(lib, name).restype = ctypes.c_int
        getattr(lib, name).argtypes = [ctypes.POINTER(PdDecodeArgs)]
    lib.pd_decode_host.restype = ctypes.c_int
    lib.pd_decode_host.argtypes = [ctypes.POINTER(PdDecodeArgs), ctypes.POINTER(PdHostIO)]
    lib.pd_workspace_bytes.restype = ctypes.c_int
    lib.pd_workspace_bytes.argtypes = [ctypes.POINTER(PdDecodeArgs), ctypes.POINTER(_c_u64)]
    lib.pd_pick_num_splits.restype = ctypes.c_int
    lib.pd_pick_num_splits.argtypes = [ctypes.c_int] * 5
    lib.pd_merge.restype = ctypes.c_int
    lib.pd_merge.argtypes = [ctypes.POINTER(PdMergeArgs)]
    lib.pd_gather.restype = ctypes.c_int
    lib.pd_gather.argtypes = [ctypes.POINTER(PdGatherArgs)]
    lib.pd_exchange_bytes.restype = _c_u64
    lib.pd_exchange_bytes.argtypes = [_c_i32, _c_i32, _c_i32]
    lib.pd_exchange_part_offset.restype = _c_u64
    lib.pd_exchange_part_offset.argtypes = [_c_i32] * 5
    lib.pd_decode_exchange.restype = ctypes.c_int
    lib.pd_decode_exchange.argtypes = [ctypes.POINTER(PdDecodeArgs), ctypes.POINTER(PdExchangeArgs)]
    lib.pd_counter_bytes.restype = ctypes.c_int
    lib.pd_counter_bytes.argtypes = [ctypes.POINTER(PdDecodeArgs), ctypes.POINTER(_c_u64)]
    lib.pd_exchange_step.restype = ctypes.c_int
    lib.pd_exchange_step.argtypes = [ctypes.POINTER(PdExchangeArgs)]
    lib.pd_selftest_bounded_wait.restype = ctypes.c_int
    lib.pd_selftest_bounded_wait.argtypes = [_c_vp, _c_u64, _c_vp]
    lib.pd_cache_write.restype = ctypes.c_int
    lib.pd_cache_write.argtypes = [ctypes.POINTER(PdCacheWriteArgs)]
    _lib = lib
    return lib


def status_string(rc: int) -> str:
    return load().pd_status_string(int(rc)).decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed: {status_string(rc)} ({rc})")


def _current_stream(device: torch.device):
    if device.type != "cuda":
        return None
    return torch.cuda.current_stream(device).cuda_stream


def fill_cache_fields(args: PdDecodeArgs, cache) -> None:
    """Copies the cache side of a PagedKVCache into an argument block."""
    k, v = cache.k_cache, cache.v_cache
    if k.dim() != 4 or k.shape != v.shape:
        raise ValueError("k_cache and v_cache must be [num_blocks, block_size, H_kv, D] and alike")
    if k.stride() != v.stride():
        raise ValueError("k_cache and v_cache must have equal strides")
    if k.stride(3) != 1:
        raise ValueError("head_dim must be contiguous in the cache")
    if k.dtype != v.dtype:
        raise ValueError("k_cache and v_cache dtypes differ")
    args.k_cache, args.v_cache = k.data_ptr(), v.data_ptr()
    args.kv_stride_block, args.kv_stride_token, args.kv_stride_head = k.stride(0), k.stride(1), k.stride(2)
    ks, vs = cache.k_scale, cache.v_scale
    if (ks is None) != (vs is None):
        raise ValueError("k_scale and v_scale must both be given or both be None")
    if ks is not None:
        if ks.dtype != torch.float16 or vs.dtype != torch.float16:
            raise ValueError("scales must be fp16")
        if ks.stride() != vs.stride() or ks.stride(2) != 1:
            raise ValueError("scales must share strides with the head index contiguous")
        args.k_scale, args.v_scale = ks.data_ptr(), vs.data_ptr()
        args.scale_stride_block, args.scale_stride_token = ks.stride(0), ks.stride(1)
    bt, sl = cache.block_table, cache.seq_lens
    if bt.dtype != torch.int32 or sl.dtype != torch.int32:
        raise ValueError("block_table and seq_lens must be int32")
    if bt.dim() != 2 or bt.stride(1) != 1 or not sl.is_contiguous():
        raise ValueError("block_table rows and seq_lens must be contiguous")
    args.block_table, args.block_table_stride, args.seq_lens = bt.data_ptr(), bt.stride(0), sl.data_ptr()
    args.batch = int(bt.shape[0])
    args.num_q_heads = cache.shape.num_q_heads
    args.num_kv_heads = int(k.shape[2])
    args.head_dim = int(k.shape[3])
    args.block_size = int(k.shape[1])
    args.num_blocks = int(k.shape[0])
    args.max_blocks_per_seq = int(bt.shape[1])
    args.kv_dtype = KV_CODE[cache.kv_dtype]
    args.stream = _current_stream(k.device)


def gather(cache, k_dense: torch.Tensor, v_dense: torch.Tensor, s_max: int) -> None:
    if not cache.k_cache.is_cuda:
        raise NativeLibraryError("the gather kernel runs on CUDA tensors only")
    args = PdDecodeArgs()
    fill_cache_fields(args, cache)
    g = PdGatherArgs(ctypes.pointer(args), k_dense.data_ptr(), v_dense.data_ptr(), int(s_max))
    with torch.cuda.device(cache.k_cache.device):
        check(load().pd_gather(ctypes.byref(g)), "pd_gather")
