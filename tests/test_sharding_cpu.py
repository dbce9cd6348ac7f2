"""Host-side tests of the multi-GPU partitioning, incl. world-size-2 gloo runs on the CPU.

The GPU kernels are replaced by the CPU oracle inside the KV-range-sharded step so the
plumbing (slice ownership, the flat partial buffer, the all-gather, the merge over ranks)
is exercised without a GPU.
"""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import paged_decode_attention_b200 as pda
from paged_decode_attention_b200 import sharding, synth
from oracle import adapters, c_oracle, paged_decode_oracle as po


def test_partition_requests_balances_tokens():
    rng = np.random.default_rng(0)
    lens = np.clip(np.rint(np.exp(np.log(1024) + 1.2 * rng.standard_normal(256))), 1, 32768).astype(int)
    for world in (1, 2, 4, 8):
        shards = sharding.partition_requests(lens, world)
        flat = sorted(i for s in shards for i in s)
        assert flat == list(range(256))                      # every request exactly once
        loads = [int(lens[s].sum()) for s in shards]
        assert max(loads) - min(loads) <= lens.max()         # greedy bound
        assert max(loads) <= 1.1 * lens.sum() / world + lens.max()
    assert sharding.partition_requests([5, 5], 4) == [[0], [1], [], []]
    with pytest.raises(ValueError):
        sharding.partition_requests([1], 0)


def test_token_ranges_are_page_aligned_and_cover():
    for seq_len, world, page in ((131072, 8, 16), (1000, 4, 16), (17, 4, 16), (0, 2, 32), (4097, 3, 64)):
        r = sharding.token_ranges(seq_len, world, page)
        assert len(r) == world and r[0][0] == 0 and r[-1][1] == seq_len
        for (lo, hi), (lo2, _) in zip(r, r[1:]):
            assert hi == lo2 and lo <= hi
        assert all(lo % page == 0 for lo, hi in r if hi > lo)  # empty trailing slices sit at the end


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_decode(q, cache, f32, lse, kernel):
    o, l = c_oracle.decode(adapters.q_to_f32(q), adapters.from_torch_cache(cache), want_lse=True)
    f32.copy_(torch.from_numpy(o))
    lse.copy_(torch.from_numpy(l))


def _oracle_merge(parts, lses, out):
    merged, _ = po.merge_partials(parts.numpy(), lses.numpy())
    out.copy_(torch.from_numpy(merged).to(out.dtype))


def _worker(rank: int, world: int, port: int, result_path: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, cache = sharding.make_kv_range_shard("c4", rank, world, "cpu", seed=3, batch=2, seq_len=1000)
        dec = sharding.KVRangeShardedDecoder(q, cache, decode_fn=_oracle_decode, merge_fn=_oracle_merge)
        out = dec.step()
        # every rank must hold the same merged result
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        assert all(torch.equal(gathered[0], g) for g in gathered)
        lens = [int(n) for n in cache.seq_lens.tolist()]
        if rank == 0:
            torch.save({"out": out, "q": q, "lens0": lens}, result_path)
        dec.close()
        dec.close()  # idempotent
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_kv_range_sharded_step_over_gloo(tmp_path):
    world = 2
    path = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(world, _free_port(), path), nprocs=world, join=True)
    got = torch.load(path)
    # rebuild the unsharded problem from the two shards and decode it whole
    shards = [sharding.make_kv_range_shard("c4", r, world, "cpu", seed=3, batch=2, seq_len=1000)
              for r in range(world)]
    assert [int(n) for n in shards[0][1].seq_lens] == got["lens0"] == [512, 512]
    assert [int(n) for n in shards[1][1].seq_lens] == [488, 488]
    assert torch.equal(shards[0][0], shards[1][0])            # q is shared
    parts, lses = [], []
    for q, cache in shards:
        o, l = c_oracle.decode(adapters.q_to_f32(q), adapters.from_torch_cache(cache), want_lse=True)
        parts.append(o)
        lses.append(l)
    # whole-sequence truth: concatenate both shards' pages into one cache per request
    q, c0 = shards[0]
    c1 = shards[1][1]
    nb0 = c0.k_cache.shape[0]
    whole = pda.PagedKVCache(
        shape=c0.shape, block_size=c0.block_size, kv_dtype=c0.kv_dtype,
        k_cache=torch.cat([c0.k_cache.view(torch.uint8), c1.k_cache.view(torch.uint8)]).view(c0.k_cache.dtype),
        v_cache=torch.cat([c0.v_cache.view(torch.uint8), c1.v_cache.view(torch.uint8)]).view(c0.v_cache.dtype),
        k_scale=torch.cat([c0.k_scale, c1.k_scale]), v_scale=torch.cat([c0.v_scale, c1.v_scale]),
        block_table=torch.cat([c0.block_table, c1.block_table + nb0], dim=1),
        seq_lens=c0.seq_lens + c1.seq_lens)
    truth = c_oracle.decode(adapters.q_to_f32(q), adapters.from_torch_cache(whole))
    err = np.abs(got["out"].float().numpy() - truth).max()
    assert err <= 2e-3, err


def test_request_sharding_needs_no_exchange():
    """Each rank's slice of a ragged batch decodes to exactly the rows of the whole batch."""
    q, cache = synth.make("c5", device="cpu", seed=1, batch=12)
    truth = c_oracle.decode(adapters.q_to_f32(q), adapters.from_torch_cache(cache))
    shards = sharding.partition_requests(cache.seq_lens.tolist(), 3)
    for rows in shards:
        sub = synth.take_requests(cache, rows)
        part = c_oracle.decode(adapters.q_to_f32(q[rows]), adapters.from_torch_cache(sub))
        assert np.array_equal(part, truth[rows])
