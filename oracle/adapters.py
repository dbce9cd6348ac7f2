"""Conversions from the library's torch-side cache to the oracle's plain arrays.

TEST INFRASTRUCTURE ONLY — see the header of paged_decode_oracle.py.
"""

from __future__ import annotations

import numpy as np
import torch

from .paged_decode_oracle import OracleCache


def _store_to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy()
    if t.dtype == torch.float8_e5m2:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def from_torch_cache(cache) -> OracleCache:
    """OracleCache holding host copies of a PagedKVCache's tensors (strided views are densified)."""
    return OracleCache(
        num_q_heads=cache.shape.num_q_heads, num_kv_heads=cache.shape.num_kv_heads,
        head_dim=cache.shape.head_dim, block_size=cache.block_size, kv_dtype=cache.kv_dtype,
        k_cache=_store_to_numpy(cache.k_cache), v_cache=_store_to_numpy(cache.v_cache),
        k_scale=None if cache.k_scale is None else cache.k_scale.detach().contiguous().cpu().numpy(),
        v_scale=None if cache.v_scale is None else cache.v_scale.detach().contiguous().cpu().numpy(),
        block_table=cache.block_table.detach().cpu().numpy().astype(np.int32),
        seq_lens=cache.seq_lens.detach().cpu().numpy().astype(np.int32))


def q_to_f32(q: torch.Tensor) -> np.ndarray:
    return q.detach().float().cpu().numpy()
