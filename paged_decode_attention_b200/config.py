"""Attention shapes and KV-cache element types for paged decode attention.

Host-side vocabulary of the decode path.  The names and meanings follow the
reference's ``pagedattn/config.py:16-71`` (``KVDType``, ``ModelShape``,
``kv_bytes_per_token``, ``torch_dtype`` and the three shape presets) so a
caller of that module can switch imports without changing call sites.  The
4 GB-card VRAM planner and ``gpu_info`` of that file are not part of the decode
path and are not provided.
"""

from __future__ import annotations

import dataclasses
from typing import Literal

import torch

KVDType = Literal["fp16", "bf16", "fp8_e5m2", "int8"]

KV_DTYPES: tuple[str, ...] = ("fp16", "bf16", "fp8_e5m2", "int8")

# Storage width of one cached K or V element.
_ELEM_BYTES = {"fp16": 2, "bf16": 2, "fp8_e5m2": 1, "int8": 1}

_TORCH = {
    "fp16": torch.float16,
    "bf16": torch.bfloat16,
    "fp8_e5m2": torch.float8_e5m2,
    "int8": torch.int8,
}

# Integer codes shared with the C ABI (``PD_KV_*`` in include/paged_decode.h).
KV_CODE = {"fp16": 0, "bf16": 1, "fp8_e5m2": 2, "int8": 3}


@dataclasses.dataclass(frozen=True)
class ModelShape:
    """Grouped-query attention geometry of one layer.

    ``num_q_heads`` query heads share ``num_kv_heads`` K/V heads in equal
    groups; ``softmax_scale`` is ``head_dim ** -0.5`` (reference
    ``pagedattn/config.py:34-53``).
    """

    num_q_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    name: str = "llama3-8b"

    @property
    def gqa_group(self) -> int:
        if self.num_kv_heads <= 0 or self.num_q_heads % self.num_kv_heads:
            raise AssertionError(
                f"num_q_heads={self.num_q_heads} not divisible by "
                f"num_kv_heads={self.num_kv_heads}"
            )
        return self.num_q_heads // self.num_kv_heads

    @property
    def softmax_scale(self) -> float:
        return float(self.head_dim) ** -0.5


LLAMA3_8B = ModelShape(32, 8, 128, "llama3-8b")
LLAMA3_70B = ModelShape(64, 8, 128, "llama3-70b")
MHA_DEBUG = ModelShape(8, 8, 128, "mha-debug")
QWEN25_05B = ModelShape(14, 2, 64, "qwen2.5-0.5b")
QWEN25_7B = ModelShape(28, 4, 128, "qwen2.5-7b")


def elem_bytes(kv_dtype: str) -> int:
    return _ELEM_BYTES[kv_dtype]


def torch_dtype(kv_dtype: str) -> torch.dtype:
    return _TORCH[kv_dtype]


def kv_bytes_per_token(shape: ModelShape, kv_dtype: str, scaled: bool | None = None) -> float:
    """Bytes of K plus V cache one token occupies in one layer.

    int8 always carries a per-(token, head) fp16 scale for K and for V
    (reference ``pagedattn/config.py:61-67``).  ``scaled=True`` counts the same
    scale bytes for fp8_e5m2, which this library accepts as an extension.
    """
    per = 2.0 * shape.num_kv_heads * shape.head_dim * _ELEM_BYTES[kv_dtype]
    if scaled is None:
        scaled = kv_dtype == "int8"
    if scaled:
        per += 2 * shape.num_kv_heads * 2
    return per
