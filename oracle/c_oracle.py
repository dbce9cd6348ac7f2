"""ctypes front end of the C oracle (oracle/paged_decode_oracle.c).

TEST INFRASTRUCTURE ONLY — see the header of paged_decode_oracle.py for who may import
this.  ``build()`` compiles the shared object with the Makefile next to this file;
``decode`` and ``gather`` take the same ``OracleCache`` the numpy oracle uses.
"""

from __future__ import annotations

import ctypes
import pathlib
import subprocess

import numpy as np

from .paged_decode_oracle import OracleCache

_HERE = pathlib.Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libpaged_decode_oracle.so"
_KV = {"fp16": 0, "bf16": 1, "fp8_e5m2": 2, "int8": 3}
_lib = None


class _PdoCache(ctypes.Structure):
    _fields_ = [
        ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
        ("k_scale", ctypes.c_void_p), ("v_scale", ctypes.c_void_p),
        ("block_table", ctypes.c_void_p), ("seq_lens", ctypes.c_void_p),
        ("batch", ctypes.c_int32), ("num_q_heads", ctypes.c_int32),
        ("num_kv_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("block_size", ctypes.c_int32), ("num_blocks", ctypes.c_int32),
        ("max_blocks", ctypes.c_int32), ("kv_dtype", ctypes.c_int32),
    ]


def build(force: bool = False) -> pathlib.Path:
    src = _HERE / "paged_decode_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True,
                       capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(str(_LIB_PATH))
        lib.pdo_decode.restype = ctypes.c_int
        lib.pdo_decode.argtypes = [ctypes.POINTER(_PdoCache), ctypes.c_void_p, ctypes.c_float,
                                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                   ctypes.c_void_p, ctypes.c_int]
        lib.pdo_gather.restype = ctypes.c_int
        lib.pdo_gather.argtypes = [ctypes.POINTER(_PdoCache), ctypes.c_void_p, ctypes.c_void_p,
                                   ctypes.c_int]
        lib.pdo_max_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def max_threads() -> int:
    return int(_load().pdo_max_threads())


def _pack(cache: OracleCache):
    keep = []

    def ptr(a, dtype=None):
        if a is None:
            return None
        a = np.ascontiguousarray(a if dtype is None else a.astype(dtype, copy=False))
        keep.append(a)
        return a.ctypes.data

    c = _PdoCache(
        ptr(cache.k_cache), ptr(cache.v_cache), ptr(cache.k_scale), ptr(cache.v_scale),
        ptr(cache.block_table, np.int32), ptr(cache.seq_lens, np.int32),
        int(cache.block_table.shape[0]), cache.num_q_heads, cache.num_kv_heads, cache.head_dim,
        cache.block_size, int(cache.k_cache.shape[0]), int(cache.block_table.shape[1]),
        _KV[cache.kv_dtype])
    return c, keep


def decode(q: np.ndarray, cache: OracleCache, sm_scale: float | None = None,
           lo: np.ndarray | None = None, hi: np.ndarray | None = None,
           want_lse: bool = False, num_threads: int = 0):
    """fp32 decode attention on the host; optionally over [lo, hi) with the base-2 lse."""
    c, keep = _pack(cache)
    qf = np.ascontiguousarray(q.astype(np.float32))
    out = np.empty_like(qf)
    lse = np.empty(qf.shape[:2], dtype=np.float32) if want_lse else None
    lo_a = None if lo is None else np.ascontiguousarray(lo, dtype=np.int32)
    hi_a = None if hi is None else np.ascontiguousarray(hi, dtype=np.int32)
    scale = cache.softmax_scale if sm_scale is None else float(sm_scale)
    rc = _load().pdo_decode(ctypes.byref(c), qf.ctypes.data, scale,
                            None if lo_a is None else lo_a.ctypes.data,
                            None if hi_a is None else hi_a.ctypes.data,
                            out.ctypes.data, None if lse is None else lse.ctypes.data,
                            int(num_threads))
    if rc != 0:
        raise RuntimeError(f"pdo_decode failed with {rc}")
    del keep
    return (out, lse) if want_lse else out


def gather(cache: OracleCache, s_max: int | None = None):
    """Dense fp16 [B, Hkv, S_max, D] K and V with zeros past each request's length."""
    c, keep = _pack(cache)
    if s_max is None:
        s_max = int(cache.seq_lens.max())
    shape = (int(cache.block_table.shape[0]), cache.num_kv_heads, s_max, cache.head_dim)
    k = np.empty(shape, dtype=np.float16)
    v = np.empty(shape, dtype=np.float16)
    rc = _load().pdo_gather(ctypes.byref(c), k.ctypes.data, v.ctypes.data, int(s_max))
    if rc != 0:
        raise RuntimeError(f"pdo_gather failed with {rc}")
    del keep
    return k, v
