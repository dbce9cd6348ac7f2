"""Two-GPU run of the KV-range-sharded long-context step (skipped on boxes with one GPU).

All three exchange paths — NCCL all-gather + merge kernel, a push kernel's peer stores + merge
kernel, and the decode kernel storing its own units with the merge launched behind it — must
reproduce the single-GPU decode of the whole sequence, host-issued and replayed from a CUDA
graph, with a clean status word.  NVLS is switched off and the peer paths use plain stores
only.  Every decoder is closed (its captured graph released) on all ranks before the process
group is destroyed.
"""

from __future__ import annotations

import os
import socket
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_path: str):
    import datetime

    import torch.distributed as dist

    from paged_decode_attention_b200 import sharding

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=60))
    try:
        q, cache = sharding.make_kv_range_shard("c4", rank, world, dev, seed=3, batch=2, seq_len=8192)
        results = {}
        for exchange in ("nccl", "peer", "fused"):
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            dec = sharding.KVRangeShardedDecoder(q, cache, group=dist.group.WORLD, exchange=exchange,
                                                 status=status)
            for _ in range(3):
                host_issued = dec.step().clone()
            dec.capture()
            for _ in range(3):
                replayed = dec.step().clone()
            torch.cuda.synchronize()
            assert int(status.item()) == 0, f"{exchange}: status {int(status.item())}"
            assert torch.equal(host_issued, replayed), exchange
            results[exchange] = host_issued
            dec.close()
        assert float((results["nccl"].float() - results["peer"].float()).abs().max()) <= 1e-3
        assert float((results["fused"].float() - results["peer"].float()).abs().max()) <= 1e-3
        # every rank holds the same merged result
        both = [torch.empty_like(results["peer"]) for _ in range(world)]
        dist.all_gather(both, results["peer"])
        assert all(torch.equal(both[0], t) for t in both)
        if rank == 0:
            torch.save({"out": results["peer"].cpu(), "q": q.cpu()}, out_path)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_kv_range_sharding_on_two_gpus(tmp_path):
    import dataclasses

    import numpy as np
    import torch.multiprocessing as mp

    from oracle import adapters, c_oracle
    from paged_decode_attention_b200 import sharding

    world, path = 2, str(tmp_path / "r0.pt")
    ctx = mp.spawn(_worker, args=(world, _free_port(), path), nprocs=world, join=False)
    deadline = time.monotonic() + 240
    while not ctx.join(timeout=5):
        if time.monotonic() > deadline:
            for proc in ctx.processes:  # exactly the ranks started above
                proc.kill()
            pytest.fail("the ranks did not exit within four minutes")
    got = torch.load(path)
    # truth: both shards' pages in one cache, decoded whole by the CPU oracle
    shards = [sharding.make_kv_range_shard("c4", r, world, "cuda:0", seed=3, batch=2, seq_len=8192)[1]
              for r in range(world)]
    c0, c1 = shards
    whole = dataclasses.replace(
        c0, k_cache=torch.cat([c0.k_cache.view(torch.uint8), c1.k_cache.view(torch.uint8)]).view(c0.k_cache.dtype),
        v_cache=torch.cat([c0.v_cache.view(torch.uint8), c1.v_cache.view(torch.uint8)]).view(c0.v_cache.dtype),
        k_scale=torch.cat([c0.k_scale, c1.k_scale]), v_scale=torch.cat([c0.v_scale, c1.v_scale]),
        block_table=torch.cat([c0.block_table, c1.block_table + c0.num_blocks], dim=1),
        seq_lens=c0.seq_lens + c1.seq_lens)
    truth = c_oracle.decode(got["q"].float().numpy(), adapters.from_torch_cache(whole))
    assert np.abs(got["out"].float().numpy() - truth).max() <= 2e-3
