"""The five benchmark configurations at full size on the GPU.

Each is compared with the C oracle on the box's host cores (seconds) and checked through
properties that do not depend on size: results are invariant under the split count, bitwise
invariant under a physical permutation of the pages, a constant V gives that constant back,
and token-range shards merged by log-sum-exp equal the unsharded result (the arithmetic the
multi-GPU long-context path uses).
"""

from __future__ import annotations

import dataclasses

import pytest
import torch

import helpers
from oracle import adapters, c_oracle
import paged_decode_attention_b200 as pda
from paged_decode_attention_b200 import sharding, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["c2", "c3", "c4", "c5"])
def workload(request):
    q, cache = synth.make(request.param, device="cuda", seed=2)
    ref = c_oracle.decode(adapters.q_to_f32(q), adapters.from_torch_cache(cache))
    yield request.param, q, cache, ref
    del q, cache
    torch.cuda.empty_cache()


def test_matches_oracle_at_full_size(workload):
    name, q, cache, ref = workload
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = pda.paged_decode(q, cache, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    helpers.assert_close(out, ref, what=f"{name} full size")
    if name == "c5":
        assert int((cache.seq_lens == 1).sum()) >= 1  # the length-1 edge is in the batch


def test_split_count_does_not_change_the_result(workload):
    name, q, cache, ref = workload
    base = pda.paged_decode(q, cache, num_splits=1).float()
    for splits in (None, 3, 8):
        other = pda.paged_decode(q, cache, num_splits=splits).float()
        assert float((other - base).abs().max()) <= 1e-3, (name, splits)


def test_page_permutation_is_bitwise_invisible(workload):
    name, q, cache, _ = workload
    base = pda.paged_decode(q, cache).clone()
    perm = torch.randperm(cache.num_blocks, device="cuda", generator=torch.Generator("cuda").manual_seed(5))
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(cache.num_blocks, device="cuda")
    moved = dataclasses.replace(
        cache, k_cache=cache.k_cache[perm], v_cache=cache.v_cache[perm],
        k_scale=None if cache.k_scale is None else cache.k_scale[perm],
        v_scale=None if cache.v_scale is None else cache.v_scale[perm],
        block_table=inv[cache.block_table.long()].to(torch.int32))
    again = pda.paged_decode(q, moved)
    assert torch.equal(base, again), name


def test_constant_values_come_back(workload):
    name, q, cache, _ = workload
    if cache.kv_dtype == "int8":
        v = torch.full_like(cache.v_cache, 64)
        vs = torch.full_like(cache.v_scale, 1.0 / 64)
    elif cache.kv_dtype == "fp8_e5m2":
        v = torch.full(cache.v_cache.shape, 1.0, dtype=torch.float16, device="cuda").to(torch.float8_e5m2)
        vs = torch.ones_like(cache.v_scale)
    else:
        v, vs = torch.ones_like(cache.v_cache), None
    out = pda.paged_decode(q, dataclasses.replace(cache, v_cache=v, v_scale=vs))
    live = (cache.seq_lens > 0)
    assert float((out[live].float() - 1.0).abs().max()) <= 2e-3, name


def test_token_range_shards_merge_to_the_whole():
    """c4's multi-GPU scheme on one GPU: four token slices decoded apart, merged by lse."""
    name, world = "c4", 4
    q, cache = synth.make(name, device="cuda", seed=9, seq_len=16384)
    ref = c_oracle.decode(adapters.q_to_f32(q), adapters.from_torch_cache(cache))
    b, hq, d = q.shape
    parts = torch.empty((world, b, hq, d), dtype=torch.float32, device="cuda")
    lses = torch.empty((world, b, hq), dtype=torch.float32, device="cuda")
    for r, (lo, hi) in enumerate(sharding.token_ranges(16384, world, cache.block_size)):
        p0, p1 = lo // cache.block_size, -(-hi // cache.block_size)
        shard = dataclasses.replace(cache, block_table=cache.block_table[:, p0:p1].contiguous(),
                                    seq_lens=torch.full((b,), hi - lo, dtype=torch.int32, device="cuda"))
        pda.paged_decode(q, shard, result_f32=parts[r], result_lse=lses[r])
    out = pda.merge_partials(parts, lses)
    helpers.assert_close(out, ref, what="sharded c4")


def test_prepared_step_equals_direct_call():
    q, cache = synth.make("c5", device="cuda", seed=4, batch=32)
    step = pda.DecodeStep(q, cache)
    assert torch.equal(step.step(), pda.paged_decode(q, cache))
    assert torch.equal(step(), step.out)


def test_sharded_decoder_single_rank_with_and_without_graph():
    """The KV-range-sharded step degenerates to a plain decode on one rank; its CUDA-graph
    replay must give the same bits as issuing the three operations from the host."""
    q, cache = synth.make("c4", device="cuda", seed=6, seq_len=4096)
    want = pda.paged_decode(q, cache)
    dec = sharding.KVRangeShardedDecoder(q, cache)
    plain = dec.step().clone()
    assert float((plain.float() - want.float()).abs().max()) <= 1e-3
    dec.capture()
    dec.out.zero_()
    assert torch.equal(dec.step(), plain)
