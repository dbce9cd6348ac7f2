"""Glue between the seeded numpy cases, the oracle and the CUDA library (tests only)."""

from __future__ import annotations

import numpy as np
import torch

import cases
from oracle.paged_decode_oracle import OracleCache
from paged_decode_attention_b200 import ModelShape, PagedKVCache

# Tolerances of the parity contract: against the reference's fp32 result, the fp16 output
# must be within 2e-3 absolute, and within 1e-2 of the largest reference value
# (the reference's own metric, tests/test_correctness.py:28,48-51).  The 2e-3 holds as it
# stands wherever the largest reference value is below 4.  From 4 upwards rounding the result
# to fp16 alone costs up to 1.95e-3 (half a unit in the last place of [4, 8)), so no
# arithmetic could meet 2e-3 there; only in that range the bound grows in proportion:
# 2e-3 * max|ref| / 2 (4e-3 at 4: the rounding plus the same 2e-3 for the arithmetic).
ABS_TOL = 2e-3
ABS_TOL_SCALES_FROM = 4.0
REL_TOL = 1e-2
# bf16 has 8 significand bits: rounding the output alone costs up to 2^-9 of its value
# (7.8e-3 just below 4); 1.6e-2 is that plus the arithmetic, scaled the same way from 4 upwards.
ABS_TOL_BF16 = 1.6e-2


def abs_tolerance(ref_f32: np.ndarray, bf16: bool = False) -> float:
    """Absolute bound for a result whose fp32 truth is `ref_f32`."""
    peak = float(np.abs(ref_f32).max()) if ref_f32.size else 0.0
    base = ABS_TOL_BF16 if bf16 else ABS_TOL
    return base if peak < ABS_TOL_SCALES_FROM else base * peak / 2.0


def store_to_torch(a: np.ndarray, kv_dtype: str, device) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    if kv_dtype == "bf16":
        return t.view(torch.bfloat16)
    if kv_dtype == "fp8_e5m2":
        return t.view(torch.float8_e5m2)
    return t


def to_device_cache(oc: OracleCache, device="cuda") -> PagedKVCache:
    return PagedKVCache(
        shape=ModelShape(oc.num_q_heads, oc.num_kv_heads, oc.head_dim, "case"),
        block_size=oc.block_size, kv_dtype=oc.kv_dtype,
        k_cache=store_to_torch(oc.k_cache, oc.kv_dtype, device),
        v_cache=store_to_torch(oc.v_cache, oc.kv_dtype, device),
        k_scale=None if oc.k_scale is None else torch.from_numpy(oc.k_scale).to(device),
        v_scale=None if oc.v_scale is None else torch.from_numpy(oc.v_scale).to(device),
        block_table=torch.from_numpy(oc.block_table).to(device),
        seq_lens=torch.from_numpy(oc.seq_lens).to(device))


def q_to_device(case: cases.Case, q: np.ndarray, device="cuda") -> torch.Tensor:
    t = torch.from_numpy(q).to(device)
    return t.view(torch.bfloat16) if case.io_dtype == "bf16" else t


def errors(got: torch.Tensor, ref_f32: np.ndarray) -> tuple[float, float]:
    """(max abs error, max abs error / max |ref|) of a device result against fp32 truth."""
    g = got.detach().float().cpu().numpy()
    err = float(np.abs(g - ref_f32).max()) if g.size else 0.0
    return err, err / max(float(np.abs(ref_f32).max()) if g.size else 0.0, 1e-6)


def assert_close(got: torch.Tensor, ref_f32: np.ndarray, bf16: bool = False, what: str = "") -> None:
    assert not torch.isnan(got.float()).any(), f"{what}: NaN in output"
    err, rel = errors(got, ref_f32)
    tol = abs_tolerance(ref_f32, bf16)
    assert err <= tol, f"{what}: max-abs error {err:.3e} > {tol}"
    assert rel <= REL_TOL, f"{what}: relative error {rel:.3e} > {REL_TOL}"
