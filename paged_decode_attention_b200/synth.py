"""Seeded synthetic decode workloads with the shapes of the five benchmark configurations.

The reference measures on synthetic caches as well (``allocate``, pagedattn/cache.py:105-184)
and on a real model this repository has no weights for; these tensors stand in for both.
Pages are drawn on the target device (a 1 GB pool takes milliseconds there), lengths and
block tables on the host from a seeded CPU generator, so a given (name, seed, device kind)
always yields the same batch.

  c1  Qwen2.5-0.5B shape   B 24,  14/2 heads, D 64,  page 16, fp16, len U[64,160], 256-block pool
  c2  Llama-3-8B shape     B 64,  32/8 heads, D 128, page 16, fp16, len U[2048,8192]
  c3  Llama-3-70B int8     B 128, 64/8 heads, D 128, page 16, int8 U[-127,127] + scales |N|/127+1e-4
  c4  long-context fp8     B 4,   32/8 heads, D 128, page 16, e5m2 N(0,1) + scales U[0.5,2], len 131072
  c5  Qwen2.5-7B ragged    B 256, 28/4 heads, D 128, page 32, fp16, len logN(ln 1024, 1.2) in [1,32768]
"""

from __future__ import annotations

import dataclasses
import math

import torch

from .cache import PagedKVCache
from .config import ModelShape, torch_dtype


@dataclasses.dataclass(frozen=True)
class Workload:
    name: str
    shape: ModelShape
    batch: int
    page: int
    kv_dtype: str
    scaled: bool
    description: str


WORKLOADS = {
    "c1": Workload("c1", ModelShape(14, 2, 64, "qwen2.5-0.5b"), 24, 16, "fp16", False,
                   "Qwen2.5-0.5B-shaped decode: B24, 14q/2kv, D64, page16, fp16, len U[64,160]"),
    "c2": Workload("c2", ModelShape(32, 8, 128, "llama3-8b"), 64, 16, "fp16", False,
                   "Llama-3-8B-shaped decode: B64, 32q/8kv, D128, page16, fp16, len U[2048,8192]"),
    "c3": Workload("c3", ModelShape(64, 8, 128, "llama3-70b"), 128, 16, "int8", True,
                   "Llama-3-70B-shaped int8-KV decode: B128, 64q/8kv, D128, page16, len 4096"),
    "c4": Workload("c4", ModelShape(32, 8, 128, "long-context"), 4, 16, "fp8_e5m2", True,
                   "long-context scaled fp8_e5m2 decode: B4, 32q/8kv, D128, page16, len 131072"),
    "c5": Workload("c5", ModelShape(28, 4, 128, "qwen2.5-7b"), 256, 32, "fp16", False,
                   "Qwen2.5-7B-shaped ragged batch: B256, 28q/4kv, D128, page32, fp16, len logN"),
}


def draw_lengths(name: str, gen: torch.Generator, batch: int | None = None,
                 seq_len: int | None = None) -> torch.Tensor:
    """int32 lengths of one batch of workload `name` from a CPU generator."""
    w = WORKLOADS[name]
    b = w.batch if batch is None else batch
    if seq_len is not None:
        return torch.full((b,), int(seq_len), dtype=torch.int32)
    if name == "c1":
        return torch.randint(64, 161, (b,), generator=gen, dtype=torch.int32)
    if name == "c2":
        return torch.randint(2048, 8193, (b,), generator=gen, dtype=torch.int32)
    if name == "c3":
        return torch.full((b,), 4096, dtype=torch.int32)
    if name == "c4":
        return torch.full((b,), 131072, dtype=torch.int32)
    z = torch.randn((b,), generator=gen, dtype=torch.float64)
    lens = torch.exp(math.log(1024.0) + 1.2 * z).round().clamp(1, 32768).to(torch.int32)
    ones = torch.randperm(b, generator=gen)[: max(1, b // 64)]
    lens[ones] = 1  # the configuration asks for length-1 requests; a draw rarely has one
    return lens


def make(name: str, device: str | torch.device = "cuda", seed: int = 0, batch: int | None = None,
         seq_len: int | None = None, pool_blocks: int | None = None,
         lengths: torch.Tensor | None = None) -> tuple[torch.Tensor, PagedKVCache]:
    """(q, cache) of workload `name` on `device`.

    ``batch``/``seq_len`` shrink or reshape the draw (for tests and sharding);
    ``pool_blocks`` enlarges the pool beyond the pages in use (c1 uses 256);
    ``lengths`` replaces the drawn lengths altogether (one rank's requests of a batch whose
    lengths were drawn once for all ranks).
    """
    w = WORKLOADS[name]
    dev = torch.device(device)
    host_gen = torch.Generator(device="cpu").manual_seed(seed)
    lens = (draw_lengths(name, host_gen, batch, seq_len) if lengths is None
            else lengths.to(torch.int32).cpu().reshape(-1))
    b = int(lens.numel())
    pages = (lens.to(torch.int64) + w.page - 1) // w.page
    used = int(pages.sum())
    pool = max(used, pool_blocks or (256 if name == "c1" else 0), 1)
    h, d = w.shape.num_kv_heads, w.shape.head_dim
    dev_gen = torch.Generator(device=dev).manual_seed(seed)

    def pages_tensor() -> torch.Tensor:
        if w.kv_dtype == "int8":
            return torch.randint(-127, 128, (pool, w.page, h, d), generator=dev_gen, device=dev,
                                 dtype=torch.int8)
        out = torch.empty((pool, w.page, h, d), dtype=torch_dtype(w.kv_dtype), device=dev)
        step = max(1, (256 << 20) // (w.page * h * d * 2))
        for lo in range(0, pool, step):
            hi = min(pool, lo + step)
            out[lo:hi] = torch.randn((hi - lo, w.page, h, d), generator=dev_gen, device=dev,
                                     dtype=torch.float16).to(out.dtype)
        return out

    def scales_tensor() -> torch.Tensor | None:
        if not w.scaled:
            return None
        if w.kv_dtype == "int8":
            s = torch.randn((pool, w.page, h), generator=dev_gen, device=dev).abs() / 127.0 + 1e-4
        else:
            s = torch.rand((pool, w.page, h), generator=dev_gen, device=dev) * 1.5 + 0.5
        return s.to(torch.float16)

    k_cache, k_scale = pages_tensor(), scales_tensor()
    v_cache, v_scale = pages_tensor(), scales_tensor()
    order = torch.randperm(pool, generator=host_gen)[:used].to(torch.int32)
    table = torch.zeros((b, max(1, int(pages.max()) if b else 1)), dtype=torch.int32)
    at = 0
    for row, n in enumerate(pages.tolist()):
        table[row, :n] = order[at:at + n]
        at += n
    q = torch.randn((b, w.shape.num_q_heads, d), generator=dev_gen, device=dev, dtype=torch.float16)
    cache = PagedKVCache(shape=w.shape, block_size=w.page, kv_dtype=w.kv_dtype, k_cache=k_cache,
                         v_cache=v_cache, k_scale=k_scale, v_scale=v_scale,
                         block_table=table.to(dev), seq_lens=lens.to(dev))
    return q, cache


def take_requests(cache: PagedKVCache, rows: list[int]) -> PagedKVCache:
    """A compact cache holding only the pages of the chosen requests (renumbered).

    Used to cut a bounded sample out of a large batch, e.g. for a CPU run.
    """
    lens = cache.seq_lens[rows].cpu()
    pages = ((lens.to(torch.int64) + cache.block_size - 1) // cache.block_size).tolist()
    table = cache.block_table[rows].cpu()
    ids = torch.cat([table[i, :n] for i, n in enumerate(pages)]) if rows else torch.zeros(0, dtype=torch.int32)
    ids_dev = ids.to(cache.k_cache.device, torch.int64)
    new_table = torch.zeros((len(rows), max(1, max(pages, default=1))), dtype=torch.int32)
    at = 0
    for i, n in enumerate(pages):
        new_table[i, :n] = torch.arange(at, at + n, dtype=torch.int32)
        at += n
    pick = lambda t: None if t is None else t.index_select(0, ids_dev).contiguous()
    return PagedKVCache(shape=cache.shape, block_size=cache.block_size, kv_dtype=cache.kv_dtype,
                        k_cache=pick(cache.k_cache), v_cache=pick(cache.v_cache),
                        k_scale=pick(cache.k_scale), v_scale=pick(cache.v_scale),
                        block_table=new_table.to(cache.k_cache.device),
                        seq_lens=lens.to(cache.k_cache.device))
