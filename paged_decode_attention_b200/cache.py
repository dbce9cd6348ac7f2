"""Paged KV cache: the argument bundle of the decode path and its fixtures.

The cache uses the "NHD" page layout of the reference
(``pagedattn/cache.py:3-8``): ``k_cache`` and ``v_cache`` are
``[num_blocks, block_size, num_kv_heads, head_dim]`` with ``head_dim``
contiguous, so the K (or V) of one (block, token, head) is one contiguous row.
Blocks, tokens and heads may have arbitrary element strides (a serving engine
may hand over strided views); the kernels take the strides, never assume them.

``PagedKVCache``, ``quantize_kv``, ``dequantize_kv``, ``allocate`` and
``gather_contiguous`` keep the reference's names, argument meaning and results
(``pagedattn/cache.py:33-215``).  Two documented extensions:

* fp8_e5m2 caches may carry per-(token, head) fp16 scales like int8 does (the
  reference has scales for int8 only); ``k_scale=None`` keeps the reference's
  unscaled fp8 behaviour.
* ``gather_contiguous`` runs the CUDA gather kernel (same address function as
  the decode kernel) and writes zeros at positions past a request's length,
  where the reference leaves whatever page the clamped block-table entry names.
"""

from __future__ import annotations

import dataclasses

import torch

from .config import KVDType, ModelShape, torch_dtype

FP8_E5M2_MAX = 57344.0
INT8_MAX = 127.0


def quantize_kv(x: torch.Tensor, kv_dtype: KVDType) -> tuple[torch.Tensor, torch.Tensor | None]:
    """Store ``x`` (``[..., num_kv_heads, head_dim]`` fp16) in the cache dtype.

    Returns ``(stored, scale)``.  int8 uses one fp16 scale per (token, head):
    ``scale = max|x| / 127`` (floored at 1e-6 before the division), values are
    rounded to nearest and clamped to ±127.  fp8_e5m2 is a plain cast with no
    scale; 16-bit dtypes are a cast.  Reference: ``pagedattn/cache.py:33-48``.
    """
    if kv_dtype in ("fp16", "bf16"):
        return x.to(torch_dtype(kv_dtype)), None
    if kv_dtype == "fp8_e5m2":
        return x.to(torch.float8_e5m2), None
    if kv_dtype != "int8":
        raise ValueError(f"unknown kv_dtype {kv_dtype}")
    peak = x.abs().amax(dim=-1, keepdim=True).float().clamp_min(1e-6)
    scale = (peak / INT8_MAX).to(torch.float16)
    stored = (x.float() / scale.float()).round().clamp(-INT8_MAX, INT8_MAX).to(torch.int8)
    return stored, scale.squeeze(-1)


def dequantize_kv(stored: torch.Tensor, scale: torch.Tensor | None, kv_dtype: KVDType) -> torch.Tensor:
    """fp16 values the decode path computes with (``pagedattn/cache.py:51-62``).

    With a scale the result is ``fp16(stored) * scale`` rounded to fp16 — the
    int8 rule of the reference, applied to fp8_e5m2 as well when a scale is
    given.
    """
    if kv_dtype not in ("fp16", "bf16", "fp8_e5m2", "int8"):
        raise ValueError(f"unknown kv_dtype {kv_dtype}")
    if kv_dtype == "int8" and scale is None:
        raise AssertionError("int8 cache needs scales")
    half = stored.to(torch.float16)
    if scale is None or kv_dtype in ("fp16", "bf16"):
        return half
    return (half * scale.unsqueeze(-1)).to(torch.float16)


@dataclasses.dataclass
class PagedKVCache:
    """Everything the decode kernel reads besides the query.

    Field names follow ``pagedattn/cache.py:70-80``.
    """

    shape: ModelShape
    block_size: int
    kv_dtype: KVDType
    k_cache: torch.Tensor  # [num_blocks, block_size, H_kv, D]
    v_cache: torch.Tensor
    k_scale: torch.Tensor | None  # [num_blocks, block_size, H_kv] fp16
    v_scale: torch.Tensor | None
    block_table: torch.Tensor  # [B, max_blocks] int32
    seq_lens: torch.Tensor  # [B] int32

    @property
    def batch(self) -> int:
        return int(self.block_table.shape[0])

    @property
    def num_blocks(self) -> int:
        return int(self.k_cache.shape[0])

    def bytes_read_per_decode_step(self) -> int:
        """KV bytes a perfect decode step must read from HBM.

        ``2 * sum(seq_lens) * H_kv * D * elem`` plus the fp16 scales when the
        cache has them; page-tail padding, q, out and the block table are not
        counted.  This is the numerator of every bandwidth figure
        (``pagedattn/cache.py:90-102``; the reference counts scales for int8,
        the only dtype it scales).
        """
        n_tok = int(self.seq_lens.sum().item())
        h, d = self.shape.num_kv_heads, self.shape.head_dim
        total = 2 * n_tok * h * d * self.k_cache.element_size()
        if self.k_scale is not None:
            total += 2 * n_tok * h * 2
        return total


def _as_len_tensor(seq_lens, batch: int) -> torch.Tensor:
    if isinstance(seq_lens, int):
        t = torch.full((batch,), seq_lens, dtype=torch.int32)
    elif isinstance(seq_lens, (list, tuple)):
        t = torch.tensor(list(seq_lens), dtype=torch.int32)
    else:
        t = seq_lens.to(torch.int32).cpu()
    if t.numel() != batch:
        raise AssertionError(f"{t.numel()} sequence lengths for batch {batch}")
    return t


def allocate(
    shape: ModelShape,
    batch: int,
    seq_lens,
    block_size: int = 16,
    kv_dtype: KVDType = "fp16",
    device: str = "cuda",
    shuffle: bool = True,
    seed: int = 0,
    slack_blocks: int = 0,
) -> PagedKVCache:
    """Build a paged cache filled with N(0,1) keys and values.

    Same arguments and, for a given torch build and device, the same tensors as
    the reference's generator (``pagedattn/cache.py:105-184``): the block
    permutation comes from a CPU generator seeded with ``seed``; K and V are
    drawn chunk by chunk (K then V within a chunk of at most 32 MiB of fp16)
    from a generator on ``device`` with the same seed and then quantized.  The
    pool holds ``sum(pages) + slack_blocks`` blocks; each request takes the
    next slice of the permutation (or ascending blocks when ``shuffle`` is
    false); unused block-table entries are zero.
    """
    lens = _as_len_tensor(seq_lens, batch)
    pages = ((lens + (block_size - 1)) // block_size).tolist()
    used = sum(pages)
    pool = used + slack_blocks
    h, d = shape.num_kv_heads, shape.head_dim

    store = torch_dtype(kv_dtype)
    k_cache = torch.empty((pool, block_size, h, d), dtype=store, device=device)
    v_cache = torch.empty_like(k_cache)
    scaled = kv_dtype == "int8"
    k_scale = torch.empty((pool, block_size, h), dtype=torch.float16, device=device) if scaled else None
    v_scale = torch.empty_like(k_scale) if scaled else None

    perm_gen = torch.Generator(device="cpu").manual_seed(seed)
    data_gen = torch.Generator(device=device).manual_seed(seed)
    per_chunk = max(1, min(pool, (32 << 20) // (block_size * h * d * 2)))
    for first in range(0, pool, per_chunk):
        last = min(first + per_chunk, pool)
        for dst, dst_scale in ((k_cache, k_scale), (v_cache, v_scale)):
            draw = torch.randn((last - first, block_size, h, d), dtype=torch.float16,
                               device=device, generator=data_gen)
            stored, scale = quantize_kv(draw, kv_dtype)
            dst[first:last] = stored
            if scale is not None:
                dst_scale[first:last] = scale

    if shuffle:
        order = torch.randperm(pool, generator=perm_gen)[:used]
    else:
        order = torch.arange(used)
    table = torch.zeros((batch, max(pages)), dtype=torch.int32)
    taken = 0
    for row, n in enumerate(pages):
        table[row, :n] = order[taken:taken + n].to(torch.int32)
        taken += n

    return PagedKVCache(shape=shape, block_size=block_size, kv_dtype=kv_dtype,
                        k_cache=k_cache, v_cache=v_cache, k_scale=k_scale, v_scale=v_scale,
                        block_table=table.to(device), seq_lens=lens.to(device))


def gather_contiguous(cache: PagedKVCache) -> tuple[torch.Tensor, torch.Tensor]:
    """Dense ``[B, H_kv, S_max, D]`` fp16 K and V, dequantized, via the GPU.

    Counterpart of ``pagedattn/cache.py:187-215``.  The copy is done by the
    library's gather kernel, which resolves pages exactly as the decode kernel
    does, so comparing its output bit for bit with a CPU gather checks the
    block-table indexing.  Positions at or beyond a request's length are zero.
    """
    from . import _cabi

    s_max = int(cache.seq_lens.max().item()) if cache.batch else 0
    h, d = cache.shape.num_kv_heads, cache.shape.head_dim
    dev = cache.k_cache.device
    k = torch.empty((cache.batch, h, s_max, d), dtype=torch.float16, device=dev)
    v = torch.empty_like(k)
    if cache.batch and s_max:
        _cabi.gather(cache, k, v, s_max)
    return k, v


def cache_write(key: torch.Tensor, value: torch.Tensor, cache: PagedKVCache, slot_mapping: torch.Tensor,
                status: torch.Tensor | None = None) -> None:
    """Store this step's keys and values (``[num_tokens, H_kv, D]``) into their cache slots.

    ``slot_mapping[t] = block * block_size + offset`` (int64, negative = padding, skipped).
    Quantises to the cache dtype on the way with ``quantize_kv``'s rules, bit for bit,
    including the per-(token, head) int8 scales.  It stands where the reference's backend
    calls the engine's ``reshape_and_cache_flash`` (``integration/vllm_backend.py:117-122``),
    and is the producer of exactly the layout the decode kernels read.
    """
    import ctypes

    from . import _cabi
    from .config import KV_CODE

    if not key.is_cuda:
        raise _cabi.NativeLibraryError("cache_write runs on CUDA tensors only")
    if key.shape != value.shape or key.dim() != 3 or key.stride() != value.stride() or key.stride(2) != 1:
        raise ValueError("key and value must be alike [num_tokens, H_kv, D] with head_dim contiguous")
    if slot_mapping.dtype != torch.int64 or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 tensor")
    if slot_mapping.numel() < key.shape[0]:
        raise ValueError("slot_mapping is shorter than the token count")
    k = cache.k_cache
    a = _cabi.PdCacheWriteArgs()
    a.key, a.value = key.data_ptr(), value.data_ptr()
    a.in_stride_token, a.in_stride_head = key.stride(0), key.stride(1)
    a.k_cache, a.v_cache = k.data_ptr(), cache.v_cache.data_ptr()
    a.kv_stride_block, a.kv_stride_token, a.kv_stride_head = k.stride(0), k.stride(1), k.stride(2)
    if cache.k_scale is not None:
        a.k_scale, a.v_scale = cache.k_scale.data_ptr(), cache.v_scale.data_ptr()
        a.scale_stride_block, a.scale_stride_token = cache.k_scale.stride(0), cache.k_scale.stride(1)
    a.slot_mapping = slot_mapping.data_ptr()
    a.num_tokens, a.num_kv_heads, a.head_dim = int(key.shape[0]), int(key.shape[1]), int(key.shape[2])
    a.block_size, a.num_blocks = int(k.shape[1]), int(k.shape[0])
    a.kv_dtype, a.io_dtype = KV_CODE[cache.kv_dtype], _cabi.IO_CODE[key.dtype]
    if status is not None:
        a.status = status.data_ptr()
    a.stream = torch.cuda.current_stream(key.device).cuda_stream
    with torch.cuda.device(key.device):
        _cabi.check(_cabi.load().pd_cache_write(ctypes.byref(a)), "pd_cache_write")
