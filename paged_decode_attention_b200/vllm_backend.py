"""vLLM V1 attention backend whose pure-decode steps run on the B200 decode library.

Counterpart of the reference's ``integration/vllm_backend.py:54-214``, re-targeted from the
vLLM 0.9 interface that file was written against to the one installed here (0.22):

* the KV cache is ``[num_blocks, 2, block_size, num_kv_heads, head_size]`` and
  ``kv_cache.unbind(1)`` yields *strided* K and V views — the C ABI takes their element
  strides, so no copy is made (the reference unbinds dim 0 of a ``[2, NB, ...]`` cache,
  ``:113``);
* ``forward`` has the extra ``output_block_scale`` argument and no longer writes this step's
  K/V into the cache (the engine does that before calling; the reference calls
  ``reshape_and_cache_flash`` itself, ``:117-122``);
* the backend is registered through the engine's registry as the CUSTOM backend instead of
  monkey-patching ``get_attn_backend_cls`` (``:180-205``).

What is kept: subclass the engine's Triton backend and override only ``forward``
(``:95-149``); a pure-decode batch (``max_query_len == 1``) of a plain decoder layer goes to
this library, everything else (prefill, mixed batches, quantized KV cache, ALiBi, soft cap,
sliding window, cascade, sinks, fused output quantization, profiling runs) is delegated to the
parent, never rejected (``_reason_to_delegate``, ``:67-90``); ``supports_shape`` gates head
geometry (``:54-60``); ``STATS`` counts decode and delegated calls so a run can prove the
kernel ran (``:64``); ``install()`` and ``maybe_install_from_env()`` keep their names and the
``PAGEDATTN_VLLM_BACKEND`` switch (``:208-214``).

Importing this module does not require vLLM; the backend classes exist only where it does.
"""

from __future__ import annotations

import os
from typing import Any

import torch

from .cache import PagedKVCache
from .config import ModelShape
from .decode import paged_decode

try:  # the classes below need the engine; the predicates do not
    from vllm.v1.attention.backends.triton_attn import TritonAttentionBackend, TritonAttentionImpl

    HAVE_VLLM = True
except Exception:  # pragma: no cover - depends on the environment
    TritonAttentionBackend = object  # type: ignore[assignment,misc]
    TritonAttentionImpl = object  # type: ignore[assignment,misc]
    HAVE_VLLM = False

QUALNAME = "paged_decode_attention_b200.vllm_backend.PagedDecodeB200Backend"

# Counters (same keys as the reference's): proof that decode was served here, not delegated.
STATS = {"decode_calls": 0, "decode_tokens": 0, "delegated_calls": 0}

_PLAIN_KV_DTYPES = ("auto", "float16", "bfloat16", "half")


def supports_shape(num_q_heads: int, num_kv_heads: int, head_dim: int) -> tuple[bool, str]:
    """Whether the decode library can serve this head geometry (reference ``:54-60``)."""
    if num_kv_heads <= 0 or num_q_heads % num_kv_heads != 0:
        return False, f"num_q_heads {num_q_heads} not divisible by num_kv_heads {num_kv_heads}"
    if head_dim not in (32, 64, 128, 256):
        return False, f"head_dim {head_dim} not in (32, 64, 128, 256)"
    return True, ""


def _reason_to_delegate(impl: Any, attn_metadata: Any, kv_cache: Any, output: Any,
                        output_scale: Any, output_block_scale: Any = None) -> str:
    """Why this call must go to the parent implementation; "" when it is ours.

    The reference's list (``:67-90``) plus the features the newer engine added to the same
    ``forward``: block-scaled output, attention sinks, non-decoder layers, multimodal prefix
    ranges, chunked look-back.
    """
    if attn_metadata is None:
        return "profiling run (no metadata)"
    if output is None:
        return "no output buffer"
    if output_scale is not None or output_block_scale is not None:
        return "fused output quantization"
    if kv_cache is None or kv_cache.numel() == 0:
        return "empty kv cache"
    if str(getattr(impl, "kv_cache_dtype", "auto")) not in _PLAIN_KV_DTYPES:
        return "quantized kv cache"
    if getattr(impl, "alibi_slopes", None) is not None:
        return "alibi slopes"
    if getattr(impl, "logits_soft_cap", 0):
        return "logits soft cap"
    if tuple(getattr(impl, "sliding_window", (-1, -1))) != (-1, -1):
        return "sliding window"
    if getattr(impl, "sinks", None) is not None:
        return "attention sinks"
    if getattr(impl, "chunk_lookback", -1) not in (-1, None):
        return "chunked look-back"
    attn_type = getattr(impl, "attn_type", "decoder")
    if str(getattr(attn_type, "value", attn_type)) != "decoder":
        return "not a decoder self-attention layer"
    if getattr(attn_metadata, "local_attn_metadata", None) is not None:
        return "local (iRoPE) attention"
    if getattr(attn_metadata, "use_cascade", False):
        return "cascade attention"
    if getattr(attn_metadata, "mm_prefix_range_tensor", None) is not None:
        return "multimodal prefix ranges"
    if getattr(attn_metadata, "max_query_len", 2) != 1:
        return "not a pure-decode batch"
    return ""


def _decode_step(impl: Any, query: torch.Tensor, kv_cache: torch.Tensor, attn_metadata: Any,
                 output: torch.Tensor) -> None:
    """The decode-only body of ``forward`` (reference ``:113-149``), engine-independent."""
    key_cache, value_cache = kv_cache.unbind(1)  # strided [NB, PAGE, H, D] views, no copy
    n = int(attn_metadata.num_actual_tokens)
    q = query[:n].view(n, impl.num_heads, impl.head_size)
    out = output[:n].view(n, impl.num_heads, impl.head_size)
    cache = PagedKVCache(
        shape=ModelShape(impl.num_heads, impl.num_kv_heads, impl.head_size, name="vllm"),
        block_size=int(key_cache.shape[1]),
        kv_dtype="bf16" if key_cache.dtype == torch.bfloat16 else "fp16",
        k_cache=key_cache, v_cache=value_cache, k_scale=None, v_scale=None,
        block_table=attn_metadata.block_table[:n], seq_lens=attn_metadata.seq_lens[:n])
    # max_seq_len is a host int, so passing it costs no device sync (reference :139-142)
    paged_decode(q, cache, out=out, sm_scale=impl.scale,
                 max_seq_len=int(getattr(attn_metadata, "max_seq_len", 0) or 0))
    STATS["decode_calls"] += 1
    STATS["decode_tokens"] += n


if HAVE_VLLM:

    class PagedDecodeB200Impl(TritonAttentionImpl):  # type: ignore[misc]
        """Pure decode goes to the B200 library, everything else to the parent."""

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None,
                    output_scale=None, output_block_scale=None):
            why = _reason_to_delegate(self, attn_metadata, kv_cache, output, output_scale,
                                      output_block_scale)
            if not why:
                ok, why = supports_shape(self.num_heads, self.num_kv_heads, self.head_size)
                if ok and kv_cache.dtype not in (torch.float16, torch.bfloat16):
                    why = f"kv cache dtype {kv_cache.dtype}"
                if ok and query.dtype != kv_cache.dtype:
                    why = "query and cache dtypes differ"
            if why:
                STATS["delegated_calls"] += 1
                return super().forward(layer, query, key, value, kv_cache, attn_metadata, output,
                                       output_scale, output_block_scale)
            _decode_step(self, query, kv_cache, attn_metadata, output)
            return output

    class PagedDecodeB200Backend(TritonAttentionBackend):  # type: ignore[misc]
        """Same metadata builder and KV-cache layout as the engine's Triton backend."""

        @staticmethod
        def get_name() -> str:
            return "CUSTOM"

        @staticmethod
        def get_impl_cls():
            return PagedDecodeB200Impl

else:  # pragma: no cover - import path without vLLM
    PagedDecodeB200Impl = None  # type: ignore[assignment]
    PagedDecodeB200Backend = None  # type: ignore[assignment]


def install() -> str:
    """Register this backend as the engine's CUSTOM attention backend; returns its qualname.

    Select it with ``attention_backend="CUSTOM"`` (or the engine's equivalent setting) when
    constructing the engine.  Idempotent.
    """
    if not HAVE_VLLM:
        raise RuntimeError("vLLM is not importable in this environment")
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    register_backend(AttentionBackendEnum.CUSTOM, QUALNAME)
    return QUALNAME


def maybe_install_from_env() -> bool:
    """Install when ``PAGEDATTN_VLLM_BACKEND`` is 1/true, for a ``vllm.general_plugins`` entry
    point that runs inside the worker process (reference ``:208-214``)."""
    if os.environ.get("PAGEDATTN_VLLM_BACKEND", "") not in ("1", "true", "True"):
        return False
    install()
    return True
