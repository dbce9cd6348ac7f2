"""CPU oracle for paged-KV grouped-query decode attention (numpy).

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU, the algorithm of the
reference's ground truth so that the CUDA path can be checked against it.  Only
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline leg of ``bench.py`` may
import it; the library itself never does.

Parity status: PINNED.  ``tests/golden/golden_v1.npz`` holds outputs of the unmodified
reference (``pagedattn.reference.reference_decode``, ``pagedattn.cache.gather_contiguous``,
``quantize_kv``/``dequantize_kv``, ``allocate`` and the split-merge arithmetic) produced by
``tests/golden/make_golden.py``; ``tests/test_oracle_golden.py`` checks every function here
against them (gathers bit for bit, attention to 1e-5 of the fp32 result, relative to its largest value).

Each function cites the reference lines it follows.  Arrays are numpy; 8-bit floating
point and bfloat16 have no numpy dtype, so caches of those kinds hold the raw bits
(``uint8`` for fp8_e5m2, ``uint16`` for bf16).
"""

from __future__ import annotations

import dataclasses

import numpy as np

LOG2E = 1.4426950408889634


@dataclasses.dataclass
class OracleCache:
    """Plain-array twin of the reference's PagedKVCache (pagedattn/cache.py:70-80)."""

    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    block_size: int
    kv_dtype: str  # "fp16" | "bf16" | "fp8_e5m2" | "int8"
    k_cache: np.ndarray  # [NB, PAGE, Hkv, D]: float16 | uint16 (bf16 bits) | uint8 (e5m2 bits) | int8
    v_cache: np.ndarray
    k_scale: np.ndarray | None  # [NB, PAGE, Hkv] float16
    v_scale: np.ndarray | None
    block_table: np.ndarray  # [B, max_blocks] int32
    seq_lens: np.ndarray  # [B] int32

    @property
    def softmax_scale(self) -> float:
        # pagedattn/config.py:51-53
        return float(self.head_dim) ** -0.5

    def bytes_read_per_decode_step(self) -> int:
        # pagedattn/cache.py:90-102, with scale bytes counted whenever scales exist
        n_tok = int(self.seq_lens.astype(np.int64).sum())
        total = 2 * n_tok * self.num_kv_heads * self.head_dim * self.k_cache.dtype.itemsize
        if self.k_scale is not None:
            total += 2 * n_tok * self.num_kv_heads * 2
        return total


def to_half(stored: np.ndarray, kv_dtype: str) -> np.ndarray:
    """Stored element -> fp16, no scale (pagedattn/cache.py:55-58, 61 ``q.to(float16)``)."""
    if kv_dtype == "fp16":
        return stored.astype(np.float16, copy=False)
    if kv_dtype == "bf16":
        as_f32 = (stored.astype(np.uint32) << 16).view(np.float32)
        return as_f32.astype(np.float16)
    if kv_dtype == "fp8_e5m2":
        # e5m2 is the high byte of an fp16 (pagedattn/cache.py:27-28)
        return (stored.astype(np.uint16) << 8).view(np.float16)
    if kv_dtype == "int8":
        return stored.astype(np.float16)
    raise ValueError(kv_dtype)


def dequantize_kv(stored: np.ndarray, scale: np.ndarray | None, kv_dtype: str) -> np.ndarray:
    """pagedattn/cache.py:51-62: fp16(stored) [* scale, rounded to fp16]."""
    half = to_half(stored, kv_dtype)
    if scale is None:
        if kv_dtype == "int8":
            raise AssertionError("int8 cache needs scales")
        return half
    # The fp32 product of two fp16 values is exact, so one rounding to fp16 happens here,
    # as in torch's half * half.
    return (half.astype(np.float32) * scale.astype(np.float32)[..., None]).astype(np.float16)


def quantize_int8(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """pagedattn/cache.py:43-47 for x [..., Hkv, D] fp16 -> (int8, fp16 scale [..., Hkv])."""
    amax = np.maximum(np.abs(x).max(axis=-1, keepdims=True).astype(np.float32), np.float32(1e-6))
    scale = (amax / np.float32(127.0)).astype(np.float16)
    # An all-zero row underflows its fp16 scale to 0; 0/0 then casts to 0 here as in torch.
    with np.errstate(invalid="ignore", divide="ignore"):
        q = np.rint(x.astype(np.float32) / scale.astype(np.float32))
        q = np.nan_to_num(np.clip(q, -127.0, 127.0), nan=0.0).astype(np.int8)
    return q, scale[..., 0]


def quantize_e5m2(x: np.ndarray) -> np.ndarray:
    """fp16 -> fp8_e5m2 bits, round to nearest even on the fp16 bits: what the reference's
    ``x.to(torch.float8_e5m2)`` does for finite inputs (pagedattn/cache.py:41-42)."""
    h = x.astype(np.float16).view(np.uint16).astype(np.uint32)
    return ((h + 0x7F + ((h >> 8) & 1)) >> 8).astype(np.uint8)


def cache_write(key: np.ndarray, value: np.ndarray, cache: OracleCache, slot_mapping: np.ndarray) -> None:
    """Store fp16 rows key/value [T, Hkv, D] at slot_mapping[t] = block * PAGE + offset, in place.

    The scatter the reference's backend delegates to the engine
    (integration/vllm_backend.py:117-122) combined with quantize_kv's rule per cache dtype
    (pagedattn/cache.py:33-48).  Negative slots are padding and are skipped.
    """
    for t, slot in enumerate(np.asarray(slot_mapping).tolist()):
        if slot < 0:
            continue
        blk, off = divmod(int(slot), cache.block_size)
        for store, scale, x in ((cache.k_cache, cache.k_scale, key[t]), (cache.v_cache, cache.v_scale, value[t])):
            if cache.kv_dtype == "fp16":
                store[blk, off] = x.astype(np.float16)
            elif cache.kv_dtype == "bf16":
                u = x.astype(np.float32).view(np.uint32)
                store[blk, off] = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
            elif cache.kv_dtype == "fp8_e5m2":
                store[blk, off] = quantize_e5m2(x)
                if scale is not None:
                    scale[blk, off] = np.float16(1.0)
            else:
                q, sc = quantize_int8(x)
                store[blk, off] = q
                scale[blk, off] = sc


def gather_contiguous(cache: OracleCache) -> tuple[np.ndarray, np.ndarray]:
    """Dense [B, Hkv, S_max, D] fp16 K and V (pagedattn/cache.py:187-215).

    Position s of request b lives in physical block ``block_table[b, s // PAGE]`` at
    token slot ``s % PAGE``.  Positions past a request's length read the page named by
    the (clamped) table entry, as the reference does; callers mask them.
    """
    s_max = int(cache.seq_lens.max()) if cache.seq_lens.size else 0
    pos = np.arange(s_max)
    blk = np.minimum(pos // cache.block_size, cache.block_table.shape[1] - 1)
    off = pos % cache.block_size
    phys = cache.block_table[:, blk].astype(np.int64)  # [B, S]
    out = []
    for store, scale in ((cache.k_cache, cache.k_scale), (cache.v_cache, cache.v_scale)):
        rows = store[phys, off[None, :]]  # [B, S, H, D]
        sc = scale[phys, off[None, :]] if scale is not None else None
        dense = dequantize_kv(rows, sc, cache.kv_dtype)
        out.append(np.ascontiguousarray(dense.transpose(0, 2, 1, 3)))
    return out[0], out[1]


def reference_decode(q: np.ndarray, cache: OracleCache, sm_scale: float | None = None) -> np.ndarray:
    """fp32 decode attention, [B, Hq, D] -> [B, Hq, D] float32 (pagedattn/reference.py:28-49).

    The reference rounds the fp32 result to q's dtype on return; passing it an fp32 q
    keeps the fp32 result, and that un-rounded value is what this returns.  ``sm_scale``
    defaults to head_dim ** -0.5 as in the reference.  Requests are handled one at a time
    to bound memory; a request of length 0 gives NaN in the reference and zeros here.
    """
    b, hq, d = q.shape
    hkv = cache.num_kv_heads
    group = hq // hkv
    scale = np.float32(cache.softmax_scale if sm_scale is None else sm_scale)
    out = np.zeros((b, hq, d), dtype=np.float32)
    qf = q.astype(np.float32)
    for i in range(b):
        n = int(cache.seq_lens[i])
        if n == 0:
            continue
        pos = np.arange(n)
        phys = cache.block_table[i, pos // cache.block_size].astype(np.int64)
        off = pos % cache.block_size
        k = dequantize_kv(cache.k_cache[phys, off],
                          None if cache.k_scale is None else cache.k_scale[phys, off],
                          cache.kv_dtype).astype(np.float32)  # [n, Hkv, D]
        v = dequantize_kv(cache.v_cache[phys, off],
                          None if cache.v_scale is None else cache.v_scale[phys, off],
                          cache.kv_dtype).astype(np.float32)
        for h in range(hq):
            kvh = h // group
            logits = (k[:, kvh, :] @ qf[i, h]) * scale  # [n]
            logits = logits - logits.max()
            p = np.exp(logits)
            p = p / p.sum(dtype=np.float32)
            out[i, h] = p.astype(np.float32) @ v[:, kvh, :]
    return out


def split_range(seq_len: int, split: int, num_splits: int, block_n: int = 64) -> tuple[int, int]:
    """Token range [lo, hi) of one split (pagedattn/triton_decode.py:78-82)."""
    tiles = -(-seq_len // block_n)
    chunk = -(-tiles // num_splits) * block_n
    lo = split * chunk
    return lo, min(lo + chunk, seq_len)


def partial_decode(q: np.ndarray, cache: OracleCache, lo: np.ndarray, hi: np.ndarray,
                   sm_scale: float | None = None) -> tuple[np.ndarray, np.ndarray]:
    """Attention over tokens [lo[b], hi[b]) only: normalised fp32 result and base-2 lse.

    Restates the split epilogue of pagedattn/triton_decode.py:169-188: an empty range
    gives a zero row with lse = -inf.
    """
    b, hq, d = q.shape
    group = hq // cache.num_kv_heads
    scale = np.float32(cache.softmax_scale if sm_scale is None else sm_scale)
    o = np.zeros((b, hq, d), dtype=np.float32)
    lse = np.full((b, hq), -np.inf, dtype=np.float32)
    qf = q.astype(np.float32)
    for i in range(b):
        a, z = int(lo[i]), int(min(hi[i], cache.seq_lens[i]))
        if a >= z:
            continue
        pos = np.arange(a, z)
        phys = cache.block_table[i, pos // cache.block_size].astype(np.int64)
        off = pos % cache.block_size
        k = dequantize_kv(cache.k_cache[phys, off],
                          None if cache.k_scale is None else cache.k_scale[phys, off],
                          cache.kv_dtype).astype(np.float32)
        v = dequantize_kv(cache.v_cache[phys, off],
                          None if cache.v_scale is None else cache.v_scale[phys, off],
                          cache.kv_dtype).astype(np.float32)
        for h in range(hq):
            s2 = (k[:, h // group, :] @ qf[i, h]) * np.float32(scale * LOG2E)
            m = s2.max()
            p = np.exp2(s2 - m)
            l = p.sum(dtype=np.float32)
            o[i, h] = (p / l) @ v[:, h // group, :]
            lse[i, h] = m + np.log2(l)
    return o, lse


def merge_partials(part_o: np.ndarray, part_lse: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """LSE-weighted merge over the leading axis (pagedattn/triton_decode.py:221-240).

    part_o [P, ..., D] normalised partials, part_lse [P, ...] base-2 log-sum-exp.
    Returns the merged result and its lse.  Rows whose partials are all empty give zeros
    and -inf (the reference divides 0 by 0 there).
    """
    m = part_lse.max(axis=0)
    safe_m = np.where(np.isfinite(m), m, 0.0).astype(np.float32)
    w = np.exp2(part_lse - safe_m[None])
    w = np.where(np.isfinite(part_lse), w, 0.0).astype(np.float32)
    denom = w.sum(axis=0, dtype=np.float32)
    num = (part_o * w[..., None]).sum(axis=0, dtype=np.float32)
    ok = denom > 0
    out = np.where(ok[..., None], num / np.where(ok, denom, 1.0)[..., None], 0.0).astype(np.float32)
    lse = np.where(ok, safe_m + np.log2(np.where(ok, denom, 1.0)), -np.inf).astype(np.float32)
    return out, lse


def reference_pick_num_splits(batch: int, num_kv_heads: int, max_seq_len: int,
                              sm_count: int, block_n: int) -> int:
    """The reference's own split heuristic (pagedattn/triton_decode.py:248-263).

    Kept to document what the library's re-derived policy replaces; results do not
    depend on the split count.
    """
    base = batch * num_kv_heads
    if base >= 2 * sm_count:
        return 1
    want = -(-2 * sm_count // base)
    useful = max(1, (max_seq_len // block_n) // 2)
    n = max(1, min(want, useful, 64))
    return 1 << (n.bit_length() - 1)
