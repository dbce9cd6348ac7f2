"""GPU parity of the CUDA decode path, called through the C ABI, against the golden
outputs of the reference and the CPU oracle.

Mirrors the reference's test list (tests/test_correctness.py): tile-edge lengths, split
counts, quantized caches, page sizes, a ragged batch with length 1 and empty splits,
group of one, shuffled vs ascending tables, other model shapes — for both CUDA kernels.
"""

from __future__ import annotations

import ctypes
import dataclasses

import numpy as np
import pytest
import torch

import cases
import helpers
from oracle import c_oracle, paged_decode_oracle as po
import paged_decode_attention_b200 as pda
from paged_decode_attention_b200 import _cabi, decode as pdec

pytestmark = pytest.mark.gpu

KERNELS = ("simple", "stream")


def _run(case, kernel, num_splits, **kw):
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    args = pdec.build_args(q, cache, torch.empty_like(q), kernel="auto" if kernel == "stream" else kernel)
    if kernel == "stream" and pdec.selected_kernel(args) != "stream":
        pytest.skip("streaming kernel does not serve this shape")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = pda.paged_decode(q, cache, num_splits=num_splits, kernel=kernel, status=status, **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out


@pytest.mark.parametrize("num_splits", [None, 1, 4])
@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.name)
def test_matches_reference_golden(case, kernel, num_splits, golden):
    out = _run(case, kernel, num_splits)
    helpers.assert_close(out, golden[f"{case.name}/out_f32"], bf16=case.io_dtype == "bf16",
                         what=f"{case.name}/{kernel}/splits={num_splits}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", ["llama8b_fp8_e5m2_s2048", "llama8b_int8_s2048", "llama8b_b2_s4097"])
def test_eight_splits(name, kernel, golden):
    """tests/test_correctness.py:64-70 runs the quantized caches with 8 splits."""
    out = _run(cases.BY_NAME[name], kernel, 8)
    helpers.assert_close(out, golden[f"{name}/out_f32"], what=name)


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.name)
def test_gather_bit_exact(case, golden):
    """Block-table indexing and dequantisation of the CUDA address function, bit for bit."""
    _, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    k, v = pda.gather_contiguous(cache)
    torch.cuda.synchronize()
    assert cases.sha256_valid_rows(k.cpu().numpy(), oc.seq_lens) == str(golden[f"{case.name}/k_sha"])
    assert cases.sha256_valid_rows(v.cpu().numpy(), oc.seq_lens) == str(golden[f"{case.name}/v_sha"])


@pytest.mark.parametrize("kernel", KERNELS)
def test_block_n_page_64(kernel, golden):
    """tests/test_correctness.py:73-78 passes block_n = max(64, page)."""
    case = cases.BY_NAME["llama8b_page64_s1000"]
    out = _run(case, kernel, 4, block_n=64)
    helpers.assert_close(out, golden[f"{case.name}/out_f32"], what="page64")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("kv_dtype,ceiling", [("int8", 0.02), ("fp8_e5m2", 0.15)])
def test_quantization_accuracy(kv_dtype, ceiling, kernel):
    """Quantized cache vs the fp16 cache of the same values (tests/test_correctness.py:125-145)."""
    rng = np.random.Generator(np.random.PCG64(11))
    shape = pda.LLAMA3_8B
    pages, page, b = 128, 16, 2
    raw = rng.standard_normal((2, b * pages, page, 8, 128), dtype=np.float32).astype(np.float16)
    table = rng.permutation(b * pages).astype(np.int32).reshape(b, pages)
    lens = np.full(b, pages * page, dtype=np.int32)
    q_np = rng.standard_normal((b, 32, 128), dtype=np.float32).astype(np.float16)
    oc16 = po.OracleCache(32, 8, 128, page, "fp16", raw[0], raw[1], None, None, table, lens)
    ref = c_oracle.decode(q_np, oc16)
    kq, ks = pda.quantize_kv(torch.from_numpy(raw[0]).cuda(), kv_dtype)
    vq, vs = pda.quantize_kv(torch.from_numpy(raw[1]).cuda(), kv_dtype)
    cache = pda.PagedKVCache(shape, page, kv_dtype, kq, vq, ks, vs,
                             torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda())
    out = pda.paged_decode(torch.from_numpy(q_np).cuda(), cache, kernel=kernel if kernel == "simple" else "auto")
    _, rel = helpers.errors(out, ref)
    assert rel < ceiling, f"{kv_dtype}: {rel:.4f}"


@pytest.mark.parametrize("kernel", KERNELS)
def test_sm_scale_override_and_out_argument(kernel):
    case = cases.BY_NAME["c2_mini"]
    q_np, oc = cases.build(case)
    ref = c_oracle.decode(q_np.astype(np.float32), oc, sm_scale=0.05)
    cache = helpers.to_device_cache(oc)
    q = torch.from_numpy(q_np).cuda()
    out = torch.full_like(q, 7.0)
    got = pda.paged_decode(q, cache, out=out, sm_scale=0.05, kernel=kernel if kernel == "simple" else "auto")
    assert got.data_ptr() == out.data_ptr()
    helpers.assert_close(out, ref, what="sm_scale")


@pytest.mark.parametrize("kernel", KERNELS)
def test_strided_q_out_and_interleaved_kv_layout(kernel, golden):
    """K and V as strided views of one [NB, 2, PAGE, H, D] allocation (the layout newer
    serving engines use), q and out as slices of padded buffers."""
    case = cases.BY_NAME["llama8b_b3_s300"]
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    both = torch.stack([cache.k_cache, cache.v_cache], dim=1).contiguous()
    cache.k_cache, cache.v_cache = both.unbind(1)
    assert not cache.k_cache.is_contiguous()
    qbuf = torch.zeros((5, 40, 128), dtype=torch.float16, device="cuda")
    obuf = torch.zeros_like(qbuf)
    qbuf[:3, 4:36] = torch.from_numpy(q_np).cuda()
    out = pda.paged_decode(qbuf[:3, 4:36], cache, out=obuf[:3, 4:36], kernel=kernel if kernel == "simple" else "auto")
    helpers.assert_close(out, golden[f"{case.name}/out_f32"], what="strided")
    assert float(obuf[3:].abs().max()) == 0.0 and float(obuf[:, :4].abs().max()) == 0.0


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("num_splits", [None, 3])
def test_zero_length_requests_give_zero_rows(kernel, num_splits):
    case = cases.Case("zeros", 32, 8, 128, 16, "fp16", (0, 33, 0, 1), seed=23)
    q_np, oc = cases.build(case)
    ref = c_oracle.decode(q_np.astype(np.float32), oc)
    out = _run(case, kernel, num_splits)
    assert float(out[0].abs().max()) == 0.0 and float(out[2].abs().max()) == 0.0
    helpers.assert_close(out, ref, what="zero-length")


@pytest.mark.parametrize("kernel", KERNELS)
def test_bad_block_id_sets_status_and_does_not_touch_memory(kernel):
    """An id outside the pool is reported through the status word and its page skipped."""
    case = cases.BY_NAME["llama8b_b2_s65"]
    q_np, oc = cases.build(case)
    oc.block_table[1, 2] = oc.k_cache.shape[0] + 5
    cache = helpers.to_device_cache(oc)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = pda.paged_decode(torch.from_numpy(q_np).cuda(), cache, status=status,
                           kernel=kernel if kernel == "simple" else "auto")
    torch.cuda.synchronize()
    assert int(status.item()) & _cabi.DEV_BAD_BLOCK
    assert not torch.isnan(out).any()


@pytest.mark.parametrize("kernel", KERNELS)
def test_length_beyond_the_block_table_row_is_cut_and_flagged(kernel):
    """A length larger than max_blocks * page cannot be served: every kernel (and the gather)
    cuts it at the end of the block-table row, raises PD_DEV_BAD_BLOCK, gives finite output,
    and leaves the other request's row exactly as without the bad length."""
    case = cases.BY_NAME["llama8b_b2_s65"]
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    q = torch.from_numpy(q_np).cuda()
    which = kernel if kernel == "simple" else "auto"
    clean = pda.paged_decode(q, cache, kernel=which).clone()
    cap = cache.block_table.shape[1] * cache.block_size
    lens = cache.seq_lens.clone()
    lens[1] = cap + 5 * cache.block_size + 3
    bad = dataclasses.replace(cache, seq_lens=lens)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = pda.paged_decode(q, bad, status=status, kernel=which)
    torch.cuda.synchronize()
    assert int(status.item()) & _cabi.DEV_BAD_BLOCK
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out[0], clean[0])
    # the row with the oversized length equals a decode of exactly the tokens its row can name
    lens_cap = cache.seq_lens.clone()
    lens_cap[1] = cap
    want = pda.paged_decode(q, dataclasses.replace(cache, seq_lens=lens_cap), kernel=which)
    assert torch.equal(out[1], want[1])
    # the gather applies the same cut: rows past it stay zero
    args = _cabi.PdDecodeArgs()
    _cabi.fill_cache_fields(args, bad)
    st2 = torch.zeros(1, dtype=torch.int32, device="cuda")
    args.status = st2.data_ptr()
    s_max = cap + 16
    kd = torch.full((2, cache.shape.num_kv_heads, s_max, cache.shape.head_dim), 7.0, dtype=torch.float16, device="cuda")
    vd = torch.full_like(kd, 7.0)
    g = _cabi.PdGatherArgs(ctypes.pointer(args), kd.data_ptr(), vd.data_ptr(), s_max)
    _cabi.check(_cabi.load().pd_gather(ctypes.byref(g)), "pd_gather")
    torch.cuda.synchronize()
    assert int(st2.item()) & _cabi.DEV_BAD_BLOCK
    assert float(kd[1, :, cap:].abs().max()) == 0.0 and float(vd[1, :, cap:].abs().max()) == 0.0


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", ["llama8b_ragged", "c4_mini", "c1_qwen05b"])
def test_fp32_result_and_lse(name, kernel):
    case = cases.BY_NAME[name]
    q_np, oc = cases.build(case)
    ref_o, ref_lse = c_oracle.decode(cases.q_as_f32(case, q_np), oc, want_lse=True)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    f32 = torch.empty(q.shape, dtype=torch.float32, device="cuda")
    lse = torch.empty(q.shape[:2], dtype=torch.float32, device="cuda")
    pda.paged_decode(q, cache, result_f32=f32, result_lse=lse, kernel=kernel if kernel == "simple" else "auto")
    helpers.assert_close(f32, ref_o, what="fp32 result")
    assert np.abs(lse.cpu().numpy() - ref_lse).max() < 5e-3


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("hq,hkv,d,kv_dtype", [(32, 2, 128, "fp16"), (24, 2, 128, "int8"), (12, 1, 64, "fp16"),
                                               (48, 4, 128, "fp8_e5m2")])
def test_wide_groups(hq, hkv, d, kv_dtype, kernel):
    """Groups of 9..16 query heads per kv head (two n-tiles in the streaming kernel)."""
    case = cases.Case("wide", hq, hkv, d, 16, kv_dtype, (333, 1, 1500), seed=31)
    q_np, oc = cases.build(case)
    ref = c_oracle.decode(q_np.astype(np.float32), oc)
    for splits in (None, 3):
        helpers.assert_close(_run(case, kernel, splits), ref, what=f"group {hq // hkv} {kv_dtype}")


@pytest.mark.parametrize("kv_dtype,lens", [("fp16", (40000,)), ("int8", (30000, 700)), ("fp16", (9000, 9000, 20))])
def test_deep_merges_of_long_requests(kv_dtype, lens):
    """One request cut over (nearly) every worker: its partials are merged in two levels."""
    case = cases.Case("deep", 32, 8, 128, 16, kv_dtype, lens, seed=41)
    q_np, oc = cases.build(case)
    ref, ref_lse = c_oracle.decode(q_np.astype(np.float32), oc, want_lse=True)
    cache = helpers.to_device_cache(oc)
    q = torch.from_numpy(q_np).cuda()
    f32 = torch.empty(q.shape, dtype=torch.float32, device="cuda")
    lse = torch.empty(q.shape[:2], dtype=torch.float32, device="cuda")
    for _ in range(2):  # twice: the counters must be left clean
        out = pda.paged_decode(q, cache, kernel="stream", result_f32=f32, result_lse=lse)
        helpers.assert_close(out, ref, what=f"deep {kv_dtype} {lens}")
        helpers.assert_close(f32, ref, what="deep fp32")
        assert np.abs(lse.cpu().numpy() - ref_lse).max() < 5e-3


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("hq,hkv,io", [(16, 4, "fp16"), (8, 1, "fp16"), (16, 2, "bf16"), (32, 8, "fp16")])
def test_head_dim_256(hq, hkv, io, kernel):
    case = cases.Case("d256", hq, hkv, 256, 16, io, (700, 33, 2100), seed=53, io_dtype=io)
    q_np, oc = cases.build(case)
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    for splits in (None, 2):
        helpers.assert_close(_run(case, kernel, splits), ref, bf16=io == "bf16", what=f"D256 {hq}/{hkv} {io}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("hq,hkv,kv,scaled", [(16, 4, "int8", True), (8, 1, "fp8_e5m2", False),
                                              (24, 2, "fp8_e5m2", True), (32, 8, "int8", True),
                                              (36, 3, "int8", True)])
def test_head_dim_256_on_8bit_pages(hq, hkv, kv, scaled, kernel):
    """Rows of two 128-byte pieces on 8-bit pages: both kernels, with and without scales,
    groups on one and on two n-tiles, a masked last tile, a one-token request."""
    case = cases.Case("d256q", hq, hkv, 256, 16, kv, (700, 33, 2100, 1), seed=59, scaled=scaled,
                      scale_kind="uniform" if kv == "fp8_e5m2" else "quant")
    q_np, oc = cases.build(case)
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    if kernel == "stream":
        cache = helpers.to_device_cache(oc)
        q = helpers.q_to_device(case, q_np)
        assert pdec.selected_kernel(pdec.build_args(q, cache, torch.empty_like(q))) == "stream"
    for splits in (None, 3):
        helpers.assert_close(_run(case, kernel, splits), ref, what=f"D256 {hq}/{hkv} {kv}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("hq,hkv,d,kv,scaled", [
    (14, 2, 64, "int8", True), (14, 2, 64, "fp8_e5m2", False), (16, 8, 64, "fp8_e5m2", True),
    (24, 2, 64, "int8", True), (4, 4, 64, "int8", True),
    (14, 2, 32, "fp16", None), (16, 8, 32, "bf16", None), (24, 2, 32, "fp16", None), (3, 1, 32, "fp16", None)])
def test_64_byte_rows(hq, hkv, d, kv, scaled, kernel):
    """Rows of 64 bytes (head_dim 64 on 8-bit pages, 32 on 16-bit pages) move with the 64-byte
    swizzle: both kernels, every head-block width, one and two n-tiles, ragged lengths."""
    io = "bf16" if kv == "bf16" else "fp16"
    case = cases.Case("row64", hq, hkv, d, 16, kv, (150, 17, 64, 1, 1300), seed=61, scaled=scaled,
                      scale_kind="uniform" if kv == "fp8_e5m2" else "quant", io_dtype=io)
    q_np, oc = cases.build(case)
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    if kernel == "stream":
        cache = helpers.to_device_cache(oc)
        q = helpers.q_to_device(case, q_np)
        assert pdec.selected_kernel(pdec.build_args(q, cache, torch.empty_like(q))) == "stream"
    for splits in (None, 3):
        helpers.assert_close(_run(case, kernel, splits), ref, bf16=io == "bf16", what=f"row64 {hq}/{hkv} D{d} {kv}")


@pytest.mark.parametrize("d,kv,scaled", [(64, "int8", True), (64, "fp8_e5m2", False), (128, "fp8_e5m2", True),
                                         (128, "int8", True)])
def test_many_requests_on_8bit_pages_with_eight_kv_heads(d, kv, scaled):
    """Many short ragged requests (some empty) on 8-bit pages with eight kv heads, at both row
    widths: segments of one, two and odd numbers of tiles through the paired-tile loop."""
    rng = np.random.Generator(np.random.PCG64(71))
    lens = tuple(int(n) for n in rng.integers(0, 400, size=72))
    case = cases.Case("w2", 32, 8, d, 16, kv, lens, seed=67, scaled=scaled,
                      scale_kind="uniform" if kv == "fp8_e5m2" else "quant")
    q_np, oc = cases.build(case)
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    for splits in (None, 2):
        helpers.assert_close(_run(case, "stream", splits), ref, what=f"many requests D{d} {kv}")


@pytest.mark.parametrize("batch,kv_dtype", [(4096, "fp16"), (4097, "fp16"), (4096, "int8")])
def test_batches_at_the_virtual_sequence_limit(batch, kv_dtype):
    """4096 short requests are the most the streaming kernel lays out; one more and the automatic
    choice is the general kernel.  Either way the oracle's result."""
    rng = np.random.Generator(np.random.PCG64(batch))
    lens = tuple(int(n) for n in rng.integers(0, 40, size=batch))
    case = cases.Case(f"limit{batch}", 32, 8, 128, 16, kv_dtype, lens, seed=91)
    q_np, oc = cases.build(case)
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    args = pdec.build_args(q, cache, torch.empty_like(q))
    assert pdec.selected_kernel(args) == ("stream" if batch <= 4096 else "simple")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):  # twice: 32 768 arrival counters must be left clean
        out = pda.paged_decode(q, cache, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        helpers.assert_close(out, ref, what=f"{batch} requests, {kv_dtype}")


@pytest.mark.parametrize("kv", ["int8", "fp8_e5m2"])
def test_8bit_pages_with_32_byte_rows_take_the_general_kernel(kv):
    """head_dim 32 on 8-bit pages is a 32-byte row, which the streaming kernel does not serve:
    `auto` must pick the general kernel and still match."""
    case = cases.Case("d32q", 14, 2, 32, 16, kv, (150, 17, 64), seed=61)
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    assert pdec.selected_kernel(pdec.build_args(q, cache, torch.empty_like(q))) == "simple"
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    helpers.assert_close(_run(case, "auto", None), ref, what=f"D32 {kv}")


def test_merge_partials_matches_oracle():
    rng = np.random.Generator(np.random.PCG64(77))
    po_ = rng.standard_normal((5, 3, 14, 64), dtype=np.float32)
    pl = (rng.standard_normal((5, 3, 14), dtype=np.float32) * 6).astype(np.float32)
    pl[2] = -np.inf            # an empty partial
    pl[:, 1, 3] = -np.inf      # a row with nothing at all
    want_o, want_l = po.merge_partials(po_, pl)
    out, f32, lse = pda.merge_partials(torch.from_numpy(po_).cuda(), torch.from_numpy(pl).cuda(), want_f32=True)
    assert np.abs(f32.cpu().numpy() - want_o).max() < 1e-5
    assert np.array_equal(np.isneginf(lse.cpu().numpy()), np.isneginf(want_l))
    fin = np.isfinite(want_l)
    assert np.abs(lse.cpu().numpy()[fin] - want_l[fin]).max() < 1e-4
    assert np.abs(out.float().cpu().numpy() - want_o).max() < 2e-3


def test_host_buffer_entry_point_equals_device_call(golden):
    case = cases.BY_NAME["c1_qwen05b"]
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    dec = pda.HostDecoder(cache)
    out_host = torch.empty((case.batch, case.hq, case.d), dtype=torch.float16).pin_memory()
    dec.step(torch.from_numpy(q_np).pin_memory(), torch.from_numpy(oc.block_table).pin_memory(),
             torch.from_numpy(oc.seq_lens).pin_memory(), out_host)
    helpers.assert_close(out_host, golden[f"{case.name}/out_f32"], what="host entry")


@pytest.mark.parametrize("name", ["c1_qwen05b", "llama8b_ragged", "llama8b_int8_s2048", "c4_mini"])
@pytest.mark.parametrize("direct", ["out", "bt", "q", "out+bt+q"])
def test_host_buffers_used_in_place_give_the_staged_result(name, direct):
    """PD_FLAG_HOST_DIRECT_OUT / _BT / _Q: the kernels write the result to, and read the block table
    and q from, the caller's pinned buffers themselves.  Same bits as the staged call; pageable buffers fall back to staging."""
    case = cases.BY_NAME[name]
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    q_t = torch.from_numpy(q_np) if case.io_dtype != "bf16" else torch.from_numpy(q_np).view(torch.bfloat16)
    bt, sl = torch.from_numpy(oc.block_table), torch.from_numpy(oc.seq_lens)

    def run(mode, pinned=True):
        dec = pda.HostDecoder(cache, io_dtype=q_t.dtype, direct=mode)
        out = torch.full(q_t.shape, 7.0, dtype=q_t.dtype)
        pin = (lambda t: t.pin_memory()) if pinned else (lambda t: t.clone())
        out = pin(out)
        dec.step(pin(q_t), pin(bt), pin(sl), out)
        return out

    staged = run("none")
    helpers.assert_close(staged, ref, bf16=case.io_dtype == "bf16", what=f"{name} staged")
    assert torch.equal(run(direct), staged), "in-place host buffers must give the staged bits"
    assert torch.equal(run(direct, pinned=False), staged), "pageable buffers are staged as before"


@pytest.mark.parametrize("seed", range(0, 36, 3))
def test_query_rows_staged_through_shared_memory_give_the_same_bits(seed):
    """PD_FLAG_STAGE_Q: the consumer warps copy their group's query rows into shared memory with
    16-byte loads and take the fragments from there.  The same values reach the same registers,
    so the result is bit for bit that of the plain call - over head counts, groups (one and two
    n-tiles), head_dim 64-256 and every page type; rows that are not one dense run ignore the flag."""
    case, splits = _random_case(seed)
    if sum(case.lens) == 0:
        pytest.skip("degenerate draw")
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    probe = pdec.build_args(q, cache, torch.empty_like(q), num_splits=splits)
    if pdec.selected_kernel(probe) != "stream":
        pytest.skip("streaming kernel does not serve this shape")
    plain = pda.DecodeStep(q, cache, num_splits=splits, kernel="stream").step().clone()
    staged = pda.DecodeStep(q, cache, num_splits=splits, kernel="stream")
    staged.args.flags |= _cabi.FLAG_STAGE_Q
    assert torch.equal(staged.step(), plain)
    wide = torch.zeros((q.shape[0], q.shape[1], q.shape[2] + 8), dtype=q.dtype, device="cuda")
    wide[..., :q.shape[2]] = q
    strided = pda.DecodeStep(wide[..., :q.shape[2]], cache, num_splits=splits, kernel="stream")
    strided.args.flags |= _cabi.FLAG_STAGE_Q
    assert torch.equal(strided.step(), plain)


def test_rejects_bad_arguments_without_launching():
    case = cases.BY_NAME["llama8b_b2_s64"]
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    q = torch.from_numpy(q_np).cuda()
    with pytest.raises(AssertionError):
        pda.paged_decode(q, cache, block_n=24)
    with pytest.raises(AssertionError):
        pda.paged_decode(q[:, :, :64], cache)
    args = pdec.build_args(q, cache, torch.empty_like(q), num_splits=4, kernel="simple")
    assert _cabi.load().pd_decode(ctypes.byref(args)) == -3  # split scratch not supplied


@pytest.mark.parametrize("kv_dtype", ["fp16", "bf16", "fp8_e5m2", "int8"])
@pytest.mark.parametrize("d", [64, 128])
def test_cache_write_is_bit_exact_and_feeds_decode(kv_dtype, d):
    """The cache-write kernel stores what the reference's quantize_kv would, bit for bit, and a
    decode over the pages it wrote equals the oracle's decode over the oracle's pages."""
    rng = np.random.Generator(np.random.PCG64(1234 + d))
    hq, hkv, page, nb = 16, 4, 16, 12
    lens = np.array([37, 90], dtype=np.int32)
    table = rng.permutation(nb).astype(np.int32).reshape(2, 6)
    store = {"fp16": np.float16, "bf16": np.uint16, "fp8_e5m2": np.uint8, "int8": np.int8}[kv_dtype]
    scaled = kv_dtype == "int8"
    oc = po.OracleCache(hq, hkv, d, page, kv_dtype, np.zeros((nb, page, hkv, d), store),
                        np.zeros((nb, page, hkv, d), store),
                        np.zeros((nb, page, hkv), np.float16) if scaled else None,
                        np.zeros((nb, page, hkv), np.float16) if scaled else None, table, lens)
    cache = helpers.to_device_cache(oc)
    tokens = int(lens.sum())
    key = (rng.standard_normal((tokens + 2, hkv, d), dtype=np.float32) * 1.5).astype(np.float16)
    val = rng.standard_normal((tokens + 2, hkv, d), dtype=np.float32).astype(np.float16)
    key[3, 1] = 0  # an all-zero row
    slots = np.concatenate([table[b, np.arange(n) // page].astype(np.int64) * page + np.arange(n) % page
                            for b, n in enumerate(lens)] + [np.array([-1, -1], dtype=np.int64)])
    po.cache_write(key, val, oc, slots)
    io = torch.bfloat16 if kv_dtype == "bf16" else torch.float16
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    pda.cache_write(torch.from_numpy(key).cuda().to(io), torch.from_numpy(val).cuda().to(io), cache,
                    torch.from_numpy(slots).cuda(), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = adapters_from(cache)
    if kv_dtype == "bf16":
        # the device input was rounded to bf16 first; compare against the same rounding
        oc2 = po.OracleCache(hq, hkv, d, page, kv_dtype, np.zeros_like(oc.k_cache), np.zeros_like(oc.v_cache),
                             None, None, table, lens)
        po.cache_write(key, val, oc2, slots)
        oc = oc2
    assert np.array_equal(got.k_cache.view(np.uint8), oc.k_cache.view(np.uint8))
    assert np.array_equal(got.v_cache.view(np.uint8), oc.v_cache.view(np.uint8))
    if scaled:
        assert np.array_equal(got.k_scale.view(np.uint16), oc.k_scale.view(np.uint16))
        assert np.array_equal(got.v_scale.view(np.uint16), oc.v_scale.view(np.uint16))
    q_np = rng.standard_normal((2, hq, d), dtype=np.float32).astype(np.float16)
    ref = c_oracle.decode(q_np.astype(np.float32), oc)
    out = pda.paged_decode(torch.from_numpy(q_np).cuda().to(io), cache)
    helpers.assert_close(out, ref, bf16=kv_dtype == "bf16", what=f"decode after write {kv_dtype}")


def adapters_from(cache):
    from oracle import adapters

    return adapters.from_torch_cache(cache)


def test_cache_write_flags_slots_outside_the_pool():
    oc = po.OracleCache(4, 2, 64, 16, "fp16", np.zeros((2, 16, 2, 64), np.float16), np.zeros((2, 16, 2, 64), np.float16),
                        None, None, np.zeros((1, 2), np.int32), np.zeros(1, np.int32))
    cache = helpers.to_device_cache(oc)
    kv = torch.ones((3, 2, 64), dtype=torch.float16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    pda.cache_write(kv, kv, cache, torch.tensor([5, 2 * 16 + 1, -1], device="cuda"), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & _cabi.DEV_BAD_BLOCK
    assert float(cache.k_cache[0, 5].min()) == 1.0 and float(cache.k_cache.sum()) == 2 * 64


def test_bounded_wait_gives_up_and_leaves_the_context_usable():
    """Failure detection without a fault: a wait nothing ends runs out after its limit, reports
    PD_DEV_TIMEOUT through the status word, and the next decode on the same context is correct."""
    import time

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    rc = _cabi.load().pd_selftest_bounded_wait(status.data_ptr(), 50_000_000,
                                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert int(status.item()) & _cabi.DEV_TIMEOUT
    assert 0.04 <= took < 1.0, took
    case = cases.BY_NAME["llama8b_b2_s65"]
    q_np, oc = cases.build(case)
    out = pda.paged_decode(torch.from_numpy(q_np).cuda(), helpers.to_device_cache(oc))
    helpers.assert_close(out, c_oracle.decode(q_np.astype(np.float32), oc), what="after timeout")


def _random_case(seed: int) -> tuple[cases.Case, int | None]:
    rng = np.random.Generator(np.random.PCG64(seed))
    kv_dtype = ["fp16", "fp16", "int8", "fp8_e5m2", "bf16"][seed % 5]
    d = 128 if kv_dtype in ("int8", "fp8_e5m2") else int(rng.choice([64, 128, 256]))
    hkv = int(rng.choice([1, 2, 3, 4, 8]))
    group = int(rng.choice([1, 2, 4, 5, 7, 8, 12]))
    page = int(rng.choice([16, 32, 64]))
    b = int(rng.integers(1, 40))
    kind = seed % 3
    if kind == 0:    # many short requests, some empty
        lens = rng.integers(0, 70, size=b)
    elif kind == 1:  # ragged with a long tail
        lens = np.clip(np.rint(np.exp(np.log(200) + 1.3 * rng.standard_normal(b))), 0, 6000)
    else:            # a few long requests
        lens = rng.integers(1000, 9000, size=min(b, 5))
    splits = [None, None, 1, 2, 5][int(rng.integers(0, 5))]
    scaled = True if kv_dtype == "int8" else bool(rng.integers(0, 2)) if kv_dtype == "fp8_e5m2" else None
    case = cases.Case(f"rand{seed}", hkv * group, hkv, d, page, kv_dtype, tuple(int(n) for n in lens), seed=1000 + seed,
                      scaled=scaled, scale_kind="uniform" if kv_dtype == "fp8_e5m2" else "quant",
                      io_dtype="bf16" if kv_dtype == "bf16" else "fp16", slack=int(rng.integers(0, 9)))
    return case, splits


@pytest.mark.parametrize("seed", range(36))
def test_random_batches_match_the_oracle(seed):
    """Seeded random geometry: head counts, groups, page sizes, dtypes, length distributions
    (empty requests, long tails, few long requests) and split counts, both kernels."""
    case, splits = _random_case(seed)
    if sum(case.lens) == 0:
        pytest.skip("degenerate draw")
    q_np, oc = cases.build(case)
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    for kernel in ("auto", "simple"):
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = pda.paged_decode(q, cache, num_splits=splits, kernel=kernel, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        helpers.assert_close(out, ref, bf16=case.io_dtype == "bf16", what=f"{case.name}/{kernel}/{splits}")


def test_repeated_one_shot_calls_reuse_their_argument_block_and_follow_the_tensors(monkeypatch):
    """paged_decode keeps the validated argument block of a call and reuses it when the next
    call names the same tensors; anything that changes (a new lengths tensor, another out)
    builds a new one, and data changed in place is simply read again by the kernel."""
    case = cases.BY_NAME["llama8b_ragged"]
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    built = []
    real = pdec.build_args
    monkeypatch.setattr(pdec, "build_args", lambda *a, **k: (built.append(1), real(*a, **k))[1])
    monkeypatch.setattr(pdec, "_args_cache", {})
    out = torch.empty_like(q)
    first = pda.paged_decode(q, cache, out=out).clone()
    again = pda.paged_decode(q, cache, out=out).clone()
    assert len(built) == 1 and torch.equal(first, again)
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    helpers.assert_close(again, ref, what="cached call")
    # lengths halved IN PLACE: same argument block, the kernel reads the new values
    cache.seq_lens.copy_(torch.clamp(cache.seq_lens // 2, min=1))
    oc2 = dataclasses.replace(oc, seq_lens=np.maximum(oc.seq_lens // 2, 1).astype(np.int32))
    half = pda.paged_decode(q, cache, out=out)
    assert len(built) == 1
    helpers.assert_close(half, c_oracle.decode(cases.q_as_f32(case, q_np), oc2), what="in-place lengths")
    # a NEW lengths tensor: another address, another block
    cache2 = dataclasses.replace(cache, seq_lens=torch.from_numpy(oc.seq_lens).cuda())
    full = pda.paged_decode(q, cache2, out=out)
    assert len(built) == 2
    helpers.assert_close(full, ref, what="new lengths tensor")
    pda.paged_decode(q, cache2)  # fresh out tensor each call: built again, still right
    assert len(built) == 3


@pytest.mark.parametrize("name", ["c2_mini", "c3_mini", "c5_mini", "c1_qwen05b"])
def test_prepared_step_keeps_its_counters_at_zero_and_follows_new_addresses(name):
    """DecodeStep vouches for its zero-filled scratch (PD_FLAG_COUNTERS_ZERO: no clear per call):
    after every call the merge counters must be zero again, whatever the lengths were, and
    step_at must serve fresh q / out / table / length buffers of the same layout."""
    case = cases.BY_NAME[name]
    q_np, oc = cases.build(case)
    cache = helpers.to_device_cache(oc)
    q = helpers.q_to_device(case, q_np)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    step = pda.DecodeStep(q, cache, status=status)
    assert step.args.flags & _cabi.FLAG_COUNTERS_ZERO
    n = ctypes.c_uint64(0)
    _cabi.check(_cabi.load().pd_counter_bytes(ctypes.byref(step.args), ctypes.byref(n)), "pd_counter_bytes")
    ref = c_oracle.decode(cases.q_as_f32(case, q_np), oc)
    for _ in range(3):
        out = step.step()
        torch.cuda.synchronize()
        helpers.assert_close(out, ref, bf16=case.io_dtype == "bf16", what="prepared step")
        if n.value:
            assert int(step._ws[: n.value].view(torch.int32).abs().sum()) == 0
    # shorter lengths in place: other segment counts, same scratch
    lens2 = np.maximum(oc.seq_lens // 3, 1).astype(np.int32)
    cache.seq_lens.copy_(torch.from_numpy(lens2))
    out = step.step()
    ref2 = c_oracle.decode(cases.q_as_f32(case, q_np), dataclasses.replace(oc, seq_lens=lens2))
    helpers.assert_close(out, ref2, bf16=case.io_dtype == "bf16", what="shorter lengths")
    if n.value:
        assert int(step._ws[: n.value].view(torch.int32).abs().sum()) == 0
    # new buffers, same layout
    q2, out2 = q.clone(), torch.empty_like(q)
    bt2, sl2 = cache.block_table.clone(), torch.from_numpy(oc.seq_lens).cuda()
    step.step_at(q2.data_ptr(), out2.data_ptr(), bt2.data_ptr(), sl2.data_ptr(),
                 torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    helpers.assert_close(out2, ref, bf16=case.io_dtype == "bf16", what="step_at")
    assert int(status.item()) == 0
