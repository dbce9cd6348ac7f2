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
import time
from typing import Any

import torch

from .cache import PagedKVCache
from .config import ModelShape
from .decode import DecodeStep

try:  # the classes below need the engine; the predicates do not
    from vllm.v1.attention.backends.triton_attn import TritonAttentionBackend, TritonAttentionImpl

    HAVE_VLLM = True
except Exception:  # pragma: no cover - depends on the environment
    TritonAttentionBackend = object  # type: ignore[assignment,misc]
    TritonAttentionImpl = object  # type: ignore[assignment,misc]
    HAVE_VLLM = False

try:  # optional second parent: the engine's FlashAttention backend
    from vllm.v1.attention.backends.flash_attn import FlashAttentionBackend, FlashAttentionImpl

    HAVE_FLASH = HAVE_VLLM
except Exception:  # pragma: no cover - depends on the environment
    FlashAttentionBackend = object  # type: ignore[assignment,misc]
    FlashAttentionImpl = object  # type: ignore[assignment,misc]
    HAVE_FLASH = False

QUALNAME = "paged_decode_attention_b200.vllm_backend.PagedDecodeB200Backend"
QUALNAME_FLASH = "paged_decode_attention_b200.vllm_backend.PagedDecodeB200FlashBackend"

# Optional measurements for the engine check: CUDA-event pairs around every delegated call (the
# prefill attention time under either parent) and the host time spent issuing decode calls.
TIMING: dict[str, Any] = {"enabled": False, "delegated_events": [], "decode_host_s": []}

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


# Prepared decode calls, one per (layer's cache tensor, decode batch size): the argument block
# is validated and filled once, with scratch of its own, and later steps only refresh addresses.
# An engine decodes with a bounded set of batch sizes (its capture sizes, or at most its
# maximum number of sequences), so the table stays small; the oldest entry leaves beyond the cap.
_PREPARED: dict[tuple, Any] = {}
_PREPARED_CAP = 512


def _engine_views(impl: Any, query: torch.Tensor, kv_cache: torch.Tensor, attn_metadata: Any,
                  output: torch.Tensor):
    """(q, cache, out) of one pure-decode step as zero-copy views of the engine's buffers."""
    # [NB, PAGE, H, D] views, no copy: strided halves of a [NB, 2, ...] cache (Triton parent) or
    # the two dense halves of a [2, NB, ...] cache (FlashAttention parent)
    key_cache, value_cache = kv_cache.unbind(int(getattr(impl, "kv_axis", 1)))
    n = int(attn_metadata.num_actual_tokens)
    q = query[:n].view(n, impl.num_heads, impl.head_size)
    out = output[:n].view(n, impl.num_heads, impl.head_size)
    cache = PagedKVCache(
        shape=ModelShape(impl.num_heads, impl.num_kv_heads, impl.head_size, name="vllm"),
        block_size=int(key_cache.shape[1]),
        kv_dtype="bf16" if key_cache.dtype == torch.bfloat16 else "fp16",
        k_cache=key_cache, v_cache=value_cache, k_scale=None, v_scale=None,
        block_table=attn_metadata.block_table[:n], seq_lens=attn_metadata.seq_lens[:n])
    return q, cache, out


def _prepare_call(q: torch.Tensor, cache: PagedKVCache, out: torch.Tensor, sm_scale: float):
    return DecodeStep(q, cache, out, sm_scale=sm_scale)


def _decode_step(impl: Any, query: torch.Tensor, kv_cache: torch.Tensor, attn_metadata: Any,
                 output: torch.Tensor) -> None:
    """The decode-only body of ``forward`` (reference ``:113-149``), engine-independent.

    The first call for a (cache tensor, batch size, layout) builds the views and a prepared
    call; every later one is five ``data_ptr()`` reads, one stream look-up and one crossing of
    the C ABI.  The layouts that the addresses are refreshed under are part of the key.
    """
    n = int(attn_metadata.num_actual_tokens)
    bt, sl = attn_metadata.block_table, attn_metadata.seq_lens
    key = (kv_cache.data_ptr(), n, kv_cache.dtype, query.dtype, query.stride(0), output.stride(0),
           bt.stride(0), bt.shape[1], tuple(kv_cache.shape), impl.num_heads, float(impl.scale),
           int(getattr(impl, "kv_axis", 1)))
    call = _PREPARED.get(key)
    if call is None:
        q, cache, out = _engine_views(impl, query, kv_cache, attn_metadata, output)
        call = _prepare_call(q, cache, out, float(impl.scale))
        if len(_PREPARED) >= _PREPARED_CAP:
            _PREPARED.pop(next(iter(_PREPARED)))
        _PREPARED[key] = call
    # max_seq_len is a host int, so passing it costs no device sync (reference :139-142)
    call.step_at(query.data_ptr(), output.data_ptr(), bt.data_ptr(), sl.data_ptr(),
                 torch.cuda.current_stream(query.device).cuda_stream,
                 int(getattr(attn_metadata, "max_seq_len", 0) or 0))
    STATS["decode_calls"] += 1
    STATS["decode_tokens"] += n


def _forward(self, parent_forward, layer, query, key, value, kv_cache, attn_metadata, output,
             output_scale, output_block_scale):
    """Shared body of both backends' ``forward``: pure decode here, everything else to the parent."""
    why = _reason_to_delegate(self, attn_metadata, kv_cache, output, output_scale, output_block_scale)
    if not why:
        ok, why = supports_shape(self.num_heads, self.num_kv_heads, self.head_size)
        if ok and kv_cache.dtype not in (torch.float16, torch.bfloat16):
            why = f"kv cache dtype {kv_cache.dtype}"
        if ok and query.dtype != kv_cache.dtype:
            why = "query and cache dtypes differ"
    if why:
        STATS["delegated_calls"] += 1
        if TIMING["enabled"] and attn_metadata is not None and not torch.cuda.is_current_stream_capturing():
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            res = parent_forward(layer, query, key, value, kv_cache, attn_metadata, output, output_scale,
                                 output_block_scale)
            e1.record()
            TIMING["delegated_events"].append((e0, e1, int(attn_metadata.num_actual_tokens)))
            return res
        return parent_forward(layer, query, key, value, kv_cache, attn_metadata, output, output_scale,
                              output_block_scale)
    if TIMING["enabled"]:
        t0 = time.perf_counter()
        _decode_step(self, query, kv_cache, attn_metadata, output)
        TIMING["decode_host_s"].append(time.perf_counter() - t0)
    else:
        _decode_step(self, query, kv_cache, attn_metadata, output)
    return output


if HAVE_VLLM:

    class PagedDecodeB200Impl(TritonAttentionImpl):  # type: ignore[misc]
        """Pure decode goes to the B200 library, everything else to the engine's Triton backend."""

        kv_axis = 1  # cache [num_blocks, 2, block_size, num_kv_heads, head_size]

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None,
                    output_scale=None, output_block_scale=None):
            return _forward(self, super().forward, layer, query, key, value, kv_cache, attn_metadata, output,
                            output_scale, output_block_scale)

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

if HAVE_FLASH:

    class PagedDecodeB200FlashImpl(FlashAttentionImpl):  # type: ignore[misc]
        """Pure decode goes to the B200 library; prefill and mixed batches go to the engine's
        FlashAttention backend — the change the reference names as its next one (README.md:211-214):
        the decode win is kept and prefill runs on the engine's fast prefill kernel instead of the
        Triton one."""

        kv_axis = 0  # cache [2, num_blocks, block_size, num_kv_heads, head_size]

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None,
                    output_scale=None, output_block_scale=None):
            return _forward(self, super().forward, layer, query, key, value, kv_cache, attn_metadata, output,
                            output_scale, output_block_scale)

    class PagedDecodeB200FlashBackend(FlashAttentionBackend):  # type: ignore[misc]
        """Same metadata builder and KV-cache layout as the engine's FlashAttention backend."""

        @staticmethod
        def get_name() -> str:
            return "CUSTOM"

        @staticmethod
        def get_impl_cls():
            return PagedDecodeB200FlashImpl

else:  # pragma: no cover - import path without the engine's FlashAttention backend
    PagedDecodeB200FlashImpl = None  # type: ignore[assignment]
    PagedDecodeB200FlashBackend = None  # type: ignore[assignment]


def install(parent: str | None = None) -> str:
    """Register this backend as the engine's CUSTOM attention backend; returns its qualname.

    ``parent`` names the engine backend that everything which is not a pure-decode batch is
    delegated to: ``"triton"`` (the reference's choice) or ``"flash"`` (the engine's
    FlashAttention backend); default: the ``PAGEDATTN_VLLM_PARENT`` environment variable, else
    ``"triton"``.  Select the backend with ``attention_backend="CUSTOM"`` (or the engine's
    equivalent setting) when constructing the engine.  Idempotent.
    """
    if not HAVE_VLLM:
        raise RuntimeError("vLLM is not importable in this environment")
    parent = parent or os.environ.get("PAGEDATTN_VLLM_PARENT", "triton")
    if parent not in ("triton", "flash"):
        raise ValueError("parent must be 'triton' or 'flash'")
    if parent == "flash" and not HAVE_FLASH:
        raise RuntimeError("the engine's FlashAttention backend is not importable here")
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    name = QUALNAME_FLASH if parent == "flash" else QUALNAME
    register_backend(AttentionBackendEnum.CUSTOM, name)
    return name


def maybe_install_from_env() -> bool:
    """Install when ``PAGEDATTN_VLLM_BACKEND`` is 1/true, for a ``vllm.general_plugins`` entry
    point that runs inside the worker process (reference ``:208-214``)."""
    if os.environ.get("PAGEDATTN_VLLM_BACKEND", "") not in ("1", "true", "True"):
        return False
    install()
    return True
