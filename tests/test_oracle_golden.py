"""Pins the CPU oracles against outputs of the unmodified reference (golden_v1.npz).

Mirrors the reference's own test list (tests/test_correctness.py) case by case: the
numpy, C and torch restatements must reproduce reference_decode's fp32 result and
gather_contiguous's bits on the same seeded inputs.
"""

from __future__ import annotations

import numpy as np
import pytest

import cases
from oracle import c_oracle, paged_decode_oracle as po, torch_port

# fp32 summation order differs between torch's einsum and these loops
ORACLE_REL = 1e-5
SMALL = [c for c in cases.CASES if sum(c.lens) * c.hq <= 3_000_000]


def _rel(got, ref):
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-6))


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.name)
def test_inputs_are_the_ones_the_reference_saw(case, golden):
    q, oc = cases.build(case)
    assert cases.sha256_inputs(q, oc) == str(golden[f"{case.name}/in_sha"])


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.name)
def test_c_oracle_matches_reference(case, golden):
    q, oc = cases.build(case)
    got = c_oracle.decode(cases.q_as_f32(case, q), oc)
    assert _rel(got, golden[f"{case.name}/out_f32"]) < ORACLE_REL


@pytest.mark.parametrize("case", SMALL, ids=lambda c: c.name)
def test_numpy_oracle_matches_reference(case, golden):
    q, oc = cases.build(case)
    got = po.reference_decode(cases.q_as_f32(case, q), oc)
    assert _rel(got, golden[f"{case.name}/out_f32"]) < ORACLE_REL


@pytest.mark.parametrize("case", [cases.BY_NAME[n] for n in (
    "llama8b_b2_s65", "llama8b_int8_s2048", "llama8b_e5m2_scaled_s700", "llama8b_bf16_s300",
    "c1_qwen05b", "c5_mini")], ids=lambda c: c.name)
def test_torch_port_matches_reference(case, golden):
    q, oc = cases.build(case)
    got = torch_port.decode(cases.q_as_f32(case, q), oc)
    assert _rel(got, golden[f"{case.name}/out_f32"]) < ORACLE_REL


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.name)
def test_gather_is_bit_exact(case, golden):
    """Block-table indexing and dequantisation, bit for bit (pagedattn/cache.py:187-215)."""
    q, oc = cases.build(case)
    k, v = c_oracle.gather(oc)
    assert cases.sha256_valid_rows(k, oc.seq_lens) == str(golden[f"{case.name}/k_sha"])
    assert cases.sha256_valid_rows(v, oc.seq_lens) == str(golden[f"{case.name}/v_sha"])
    if sum(case.lens) * case.hkv * case.d <= 4_000_000:
        k2, v2 = po.gather_contiguous(oc)
        assert cases.sha256_valid_rows(k2, oc.seq_lens) == str(golden[f"{case.name}/k_sha"])
        assert cases.sha256_valid_rows(v2, oc.seq_lens) == str(golden[f"{case.name}/v_sha"])


def test_quantize_dequantize_known_answers(golden):
    x = golden["quant/x"]
    q8, s8 = po.quantize_int8(x)
    assert np.array_equal(q8, golden["quant/int8"])
    assert np.array_equal(s8.view(np.uint16), golden["quant/int8_scale"].view(np.uint16))
    deq = po.dequantize_kv(q8, s8, "int8")
    assert np.array_equal(deq.view(np.uint16), golden["quant/int8_dequant"].view(np.uint16))
    bits = cases._f16_to_e5m2_bits(x)
    assert np.array_equal(bits, golden["quant/e5m2_bits"])
    assert np.array_equal(po.quantize_e5m2(x), golden["quant/e5m2_bits"])
    deq8 = po.dequantize_kv(bits, None, "fp8_e5m2")
    assert np.array_equal(deq8.view(np.uint16), golden["quant/e5m2_dequant"].view(np.uint16))


def test_reference_split_policy_table(golden):
    for (b, h, s, sm), want in zip(golden["splits/args"], golden["splits/value"]):
        assert po.reference_pick_num_splits(int(b), int(h), int(s), int(sm), 64) == int(want)


@pytest.mark.parametrize("name,splits", [("llama8b_ragged", 4), ("llama8b_b2_s4097", 8),
                                         ("c1_qwen05b", 3), ("c3_mini", 5)])
def test_split_then_merge_equals_whole(name, splits, golden):
    """The split rule (triton_decode.py:78-82), its epilogue (:169-188) and the merge
    (:221-240) together reproduce the unsplit result, including empty splits."""
    case = cases.BY_NAME[name]
    q, oc = cases.build(case)
    qf = cases.q_as_f32(case, q)
    parts, lses = [], []
    for s in range(splits):
        rng = [po.split_range(int(n), s, splits) for n in oc.seq_lens]
        lo = np.array([r[0] for r in rng], dtype=np.int32)
        hi = np.array([r[1] for r in rng], dtype=np.int32)
        o, l = c_oracle.decode(qf, oc, lo=lo, hi=hi, want_lse=True)
        parts.append(o)
        lses.append(l)
    merged, _ = po.merge_partials(np.stack(parts), np.stack(lses))
    assert _rel(merged, golden[f"{name}/out_f32"]) < ORACLE_REL
    if name == "llama8b_ragged":
        assert np.isneginf(np.stack(lses)[:, 1]).sum() == (splits - 1) * case.hq  # seq_len 1


def test_numpy_and_c_partials_agree():
    case = cases.BY_NAME["llama8b_e5m2_scaled_s700"]
    q, oc = cases.build(case)
    lo = np.array([64, 320], dtype=np.int32)
    hi = np.array([640, 9999], dtype=np.int32)
    o1, l1 = po.partial_decode(q.astype(np.float32), oc, lo, hi)
    o2, l2 = c_oracle.decode(q.astype(np.float32), oc, lo=lo, hi=hi, want_lse=True)
    assert _rel(o1, o2) < ORACLE_REL
    assert np.allclose(l1, l2, rtol=0, atol=2e-5)


def test_oracle_cache_write_reproduces_quantize_kv(golden):
    """Rows scattered by the oracle's cache write hold exactly the reference's quantize_kv output."""
    x = golden["quant/x"]  # [37, 4, 64] fp16
    slots = np.random.Generator(np.random.PCG64(5)).permutation(48)[:37].astype(np.int64)
    slots[5] = -1
    for kv_dtype, want, want_scale in (("int8", golden["quant/int8"], golden["quant/int8_scale"]),
                                       ("fp8_e5m2", golden["quant/e5m2_bits"], None)):
        store = np.int8 if kv_dtype == "int8" else np.uint8
        oc = po.OracleCache(8, 4, 64, 16, kv_dtype, np.zeros((3, 16, 4, 64), store), np.zeros((3, 16, 4, 64), store),
                            np.zeros((3, 16, 4), np.float16) if want_scale is not None else None,
                            np.zeros((3, 16, 4), np.float16) if want_scale is not None else None,
                            np.zeros((1, 3), np.int32), np.zeros(1, np.int32))
        po.cache_write(x, x[::-1].copy(), oc, slots)
        for t, slot in enumerate(slots):
            if slot < 0:
                continue
            blk, off = divmod(int(slot), 16)
            assert np.array_equal(oc.k_cache[blk, off], want[t])
            assert np.array_equal(oc.v_cache[blk, off], want[36 - t])
            if want_scale is not None:
                assert np.array_equal(oc.k_scale[blk, off].view(np.uint16), want_scale[t].view(np.uint16))
