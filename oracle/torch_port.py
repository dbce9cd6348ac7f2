"""Torch-on-CPU restatement of the reference's decode path, used for timing.

TEST INFRASTRUCTURE ONLY — see the header of paged_decode_oracle.py.  The reference's
ground truth is itself a chain of torch ops (pagedattn/reference.py:28-49 on top of
pagedattn/cache.py:187-215): index the pages into a dense fp16 [B, Hkv, S_max, D] pair,
widen to fp32, then for every query head a masked softmax between two einsums.  This
module performs the same chain on host tensors with torch's intra-op threads, so its
running time stands in for the reference's CPU path on a box where the reference tree
itself is not present.  Pinned against the golden file like the other oracles.
"""

from __future__ import annotations

import numpy as np
import torch

from .paged_decode_oracle import OracleCache


def _stored_as_half(store: np.ndarray, kv_dtype: str) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(store))
    if kv_dtype == "fp16":
        return t
    if kv_dtype == "bf16":
        return t.view(torch.bfloat16)
    if kv_dtype == "fp8_e5m2":
        return t.view(torch.float8_e5m2)
    return t


def dense_kv(cache: OracleCache) -> tuple[torch.Tensor, torch.Tensor]:
    """pagedattn/cache.py:196-214 with torch indexing."""
    lens = torch.from_numpy(cache.seq_lens.astype(np.int64))
    table = torch.from_numpy(cache.block_table.astype(np.int64))
    s_max = int(lens.max())
    pos = torch.arange(s_max)
    page = (pos // cache.block_size).clamp(max=table.shape[1] - 1)
    slot = (pos % cache.block_size).unsqueeze(0).expand(table.shape[0], -1)
    phys = table[:, page]
    dense = []
    for store, scale in ((cache.k_cache, cache.k_scale), (cache.v_cache, cache.v_scale)):
        rows = _stored_as_half(store, cache.kv_dtype)[phys, slot].to(torch.float16)
        if scale is not None:
            rows = (rows * torch.from_numpy(scale)[phys, slot].unsqueeze(-1)).to(torch.float16)
        dense.append(rows.permute(0, 2, 1, 3).contiguous())
    return dense[0], dense[1]


def decode(q: np.ndarray, cache: OracleCache, num_threads: int | None = None) -> np.ndarray:
    """pagedattn/reference.py:28-49 on the host; returns the fp32 result."""
    if num_threads:
        torch.set_num_threads(int(num_threads))
    k, v = dense_kv(cache)
    k, v = k.float(), v.float()
    qf = torch.from_numpy(q.astype(np.float32))
    b, hq, d = qf.shape
    group = hq // cache.num_kv_heads
    lens = torch.from_numpy(cache.seq_lens.astype(np.int64))
    dead = torch.arange(k.shape[2]).unsqueeze(0) >= lens.unsqueeze(1)
    out = torch.empty((b, hq, d), dtype=torch.float32)
    for h in range(hq):
        kv = h // group
        s = torch.einsum("bd,bsd->bs", qf[:, h], k[:, kv]) * cache.softmax_scale
        w = torch.softmax(s.masked_fill(dead, float("-inf")), dim=-1)
        out[:, h] = torch.einsum("bs,bsd->bd", w, v[:, kv])
    return out.numpy()
