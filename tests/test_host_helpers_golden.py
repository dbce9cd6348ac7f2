"""The package's own host helpers against the golden vectors the reference produced.

``quantize_kv``, ``dequantize_kv`` and ``allocate`` (pagedattn/cache.py:33-62, 105-184) are
fixture-side functions of the reference that this package re-implements under the same
names.  The golden file holds their outputs from the unmodified reference on the CPU
(tests/golden/make_golden.py); the package's versions must reproduce them bit for bit.
"""

from __future__ import annotations

import hashlib

import numpy as np
import pytest
import torch

import paged_decode_attention_b200 as pda


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy() if t.element_size() == 1 else t.contiguous().view(torch.int16).numpy()


def test_quantize_kv_matches_reference_vectors(golden):
    x = torch.from_numpy(golden["quant/x"])
    q8, s8 = pda.quantize_kv(x, "int8")
    assert q8.dtype == torch.int8 and s8.dtype == torch.float16
    assert np.array_equal(q8.numpy(), golden["quant/int8"])
    assert np.array_equal(_bits(s8), golden["quant/int8_scale"].view(np.int16))
    f8, none = pda.quantize_kv(x, "fp8_e5m2")
    assert none is None and f8.dtype == torch.float8_e5m2
    assert np.array_equal(f8.view(torch.uint8).numpy(), golden["quant/e5m2_bits"])
    # 16-bit dtypes are plain casts with no scale
    h, none = pda.quantize_kv(x, "fp16")
    assert none is None and torch.equal(h, x)


def test_dequantize_kv_matches_reference_vectors(golden):
    q8 = torch.from_numpy(golden["quant/int8"])
    s8 = torch.from_numpy(golden["quant/int8_scale"])
    deq = pda.dequantize_kv(q8, s8, "int8")
    assert deq.dtype == torch.float16
    assert np.array_equal(_bits(deq), golden["quant/int8_dequant"].view(np.int16))
    f8 = torch.from_numpy(golden["quant/e5m2_bits"]).view(torch.float8_e5m2)
    deq8 = pda.dequantize_kv(f8, None, "fp8_e5m2")
    assert np.array_equal(_bits(deq8), golden["quant/e5m2_dequant"].view(np.int16))
    with pytest.raises(AssertionError):
        pda.dequantize_kv(q8, None, "int8")


@pytest.mark.parametrize("tag,kw", [("shuffled", dict(shuffle=True)), ("sequential", dict(shuffle=False)),
                                    ("slack_int8", dict(shuffle=True, kv_dtype="int8", slack_blocks=5))])
def test_allocate_reproduces_reference_cache(golden, tag, kw):
    """Same arguments as the generator used: block table, lengths, every page byte and the
    byte count of a decode step are the reference's."""
    c = pda.allocate(pda.ModelShape(8, 2, 64, "t"), 3, [5, 40, 17], block_size=16, device="cpu", seed=3, **kw)
    assert np.array_equal(c.block_table.numpy(), golden[f"allocate/{tag}/block_table"])
    assert np.array_equal(c.seq_lens.numpy(), golden[f"allocate/{tag}/seq_lens"])
    raw = c.k_cache.numpy().tobytes() + c.v_cache.numpy().tobytes()
    if c.k_scale is not None:
        raw += c.k_scale.numpy().tobytes() + c.v_scale.numpy().tobytes()
    assert hashlib.sha256(raw).hexdigest() == str(golden[f"allocate/{tag}/pages_sha"])
    assert c.bytes_read_per_decode_step() == int(golden[f"allocate/{tag}/bytes_read"])
    assert c.num_blocks == sum(-(-n // 16) for n in (5, 40, 17)) + kw.get("slack_blocks", 0)
