"""The allocation-free entry point, pd_decode_static, against pd_decode.

Some callers of this library cannot allocate device memory when a decode step runs: the
serving process gave every free byte of HBM to its KV pages, or the step runs on a thread
where the engine forbids allocator calls.  For them the library keeps the streaming
kernel's scratch in a fixed 8 MiB device array of its own.  These tests call that entry
point through the C ABI and require the same output as the ordinary entry point, on two
consecutive calls with different batches (the array is shared and keeps old contents), and
check that a request too big for the array is refused before anything is launched.

The file name sorts last so a stop-at-first-failure run has already covered everything else.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

import cases
import helpers
import paged_decode_attention_b200 as pda
from paged_decode_attention_b200 import _cabi, decode as pdec


def _both_ways(case, golden, num_splits=None):
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    want = pda.paged_decode(q, cache, kernel="stream", num_splits=num_splits)
    got = torch.full_like(q, float("nan"))
    args = pdec.build_args(q, cache, got, kernel="stream", num_splits=num_splits)
    assert args.workspace is None  # no scratch handed over
    rc = _cabi.load().pd_decode_static(ctypes.byref(args))
    torch.cuda.synchronize()
    assert rc == 0, _cabi.status_string(rc)
    # same kernel, same schedule: within the parity tolerance of each other and of the reference
    assert float((got.float() - want.float()).abs().max()) <= helpers.ABS_TOL
    helpers.assert_close(got, golden[f"{case.name}/out_f32"], what=f"static/{case.name}")


@pytest.mark.gpu
def test_static_scratch_entry_point_twice_in_a_row(golden):
    _both_ways(cases.BY_NAME["llama8b_ragged"], golden)           # fp16, partial slots in use
    _both_ways(cases.BY_NAME["c3_mini"], golden, num_splits=4)    # int8 + scales, explicit splits
    _both_ways(cases.BY_NAME["llama8b_ragged"], golden)           # again over the stale contents


@pytest.mark.gpu
def test_python_wrapper_needs_out_and_matches(golden):
    case = cases.BY_NAME["c1_qwen05b"]
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    with pytest.raises(ValueError):
        pda.paged_decode_static(q, cache, None)
    out = torch.empty_like(q)
    assert pda.paged_decode_static(q, cache, out).data_ptr() == out.data_ptr()
    helpers.assert_close(out, golden[f"{case.name}/out_f32"], what="static wrapper")


def test_request_beyond_the_fixed_scratch_is_refused():
    """Needs no GPU: the size check comes before anything touches a device."""
    shape = pda.ModelShape(32, 8, 128, "t")
    b = 600  # (148 workers + 600 requests) slots * 32 heads * 129 floats exceeds 8 MiB
    cache = pda.PagedKVCache(shape, 16, "fp16", torch.empty((b, 16, 8, 128), dtype=torch.float16),
                             torch.empty((b, 16, 8, 128), dtype=torch.float16), None, None,
                             torch.zeros((b, 1), dtype=torch.int32), torch.ones(b, dtype=torch.int32))
    q = torch.empty((b, 32, 128), dtype=torch.float16)
    args = pdec.build_args(q, cache, torch.empty_like(q), kernel="stream", sm_count=148)
    need = ctypes.c_uint64(0)
    assert _cabi.load().pd_workspace_bytes(ctypes.byref(args), ctypes.byref(need)) == 0
    assert need.value > _cabi.STATIC_SCRATCH_BYTES
    assert _cabi.load().pd_decode_static(ctypes.byref(args)) == _cabi.ERR_TOO_LARGE
    assert "scratch" in _cabi.status_string(_cabi.ERR_TOO_LARGE)
