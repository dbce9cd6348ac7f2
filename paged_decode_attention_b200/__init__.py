"""B200-native paged-KV grouped-query decode attention.

Public names follow the reference package (pagedattn/__init__.py:3-13) for everything on
the decode path: the shape vocabulary, the paged cache and its helpers, and the decode
entry point (``paged_decode``, also exported under the reference's name
``paged_decode_triton``) with ``pick_num_splits``.  The compute lives in
``libpaged_decode_b200.so`` (hand-written sm_100a CUDA behind the C ABI of
include/paged_decode.h); nothing here falls back to PyTorch or the CPU.
"""

from . import synth
from .config import (KVDType, LLAMA3_8B, LLAMA3_70B, MHA_DEBUG, QWEN25_05B, QWEN25_7B, ModelShape,
                     kv_bytes_per_token, torch_dtype)
from .cache import (PagedKVCache, allocate, cache_write, dequantize_kv, gather_contiguous,
                    quantize_kv)
from .decode import (DecodeStep, HostDecoder, merge_partials, paged_decode, paged_decode_static,
                     paged_decode_triton, pick_num_splits)

__all__ = [
    "KVDType", "LLAMA3_8B", "LLAMA3_70B", "MHA_DEBUG", "QWEN25_05B", "QWEN25_7B", "ModelShape",
    "kv_bytes_per_token", "torch_dtype",
    "PagedKVCache", "allocate", "gather_contiguous", "quantize_kv", "dequantize_kv", "cache_write",
    "paged_decode", "paged_decode_triton", "paged_decode_static", "pick_num_splits", "merge_partials", "HostDecoder", "DecodeStep",
]
