"""The cross-rank exchange on ONE GPU: several ranks played by one process, one stream.

Every rank's exchange buffer lives on the same device and every send is issued before any
merge, so no kernel ever waits for a later launch; the merges find their flags set.  Covers
the push kernel and the decode kernel's own push (pd_decode_exchange), odd-sized partials, and
the give-up path of the bounded wait.
"""

from __future__ import annotations

import ctypes
import dataclasses

import numpy as np
import pytest
import torch

import helpers
from oracle import adapters, c_oracle, paged_decode_oracle as po
import paged_decode_attention_b200 as pda
from paged_decode_attention_b200 import _cabi, sharding

pytestmark = pytest.mark.gpu


class _Ranks:
    """`world` exchange buffers on one device and one PdExchangeArgs per played rank."""

    def __init__(self, world, b, hq, d, status=None, wait_ns=0):
        lib = _cabi.load()
        nbytes = int(lib.pd_exchange_bytes(world, b * hq, d))
        assert nbytes > 0
        self.bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        self.ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in self.bufs])
        self.outs = [torch.full((b, hq, d), 9.0, dtype=torch.float16, device="cuda") for _ in range(world)]
        self.args = []
        for r in range(world):
            a = _cabi.PdExchangeArgs()
            a.peer_bufs = ctypes.cast(self.ptrs, ctypes.POINTER(ctypes.c_void_p))
            a.world, a.rank = world, r
            a.rows, a.head_dim, a.rows_per_batch = b * hq, d, hq
            a.out, a.out_stride_b, a.out_stride_h = self.outs[r].data_ptr(), hq * d, d
            a.io_dtype = 0
            a.wait_limit_ns = wait_ns
            if status is not None:
                a.status = status.data_ptr()
            a.stream = torch.cuda.current_stream().cuda_stream
            self.args.append(a)


@pytest.mark.parametrize("world,b,hq,d", [(2, 1, 14, 64), (3, 2, 6, 128), (8, 4, 32, 128), (2, 1, 1, 64)])
def test_push_and_merge_with_every_rank_on_one_gpu(world, b, hq, d):
    """Odd-sized partials (rows * (d + 1) = 910, 1548, .., 65 words): the two-word stores must
    stay aligned, the odd last word must arrive too, and the merge must equal the oracle's
    log-sum-exp merge."""
    lib = _cabi.load()
    gen = torch.Generator(device="cuda").manual_seed(world * 1000 + hq)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ranks = _Ranks(world, b, hq, d, status=status)
    for step in range(3):  # both parities, and the step counter moving on
        locs = []
        for r in range(world):
            o = torch.randn((b * hq, d), generator=gen, device="cuda")
            lse = torch.randn((b * hq,), generator=gen, device="cuda") * 3
            if r == 1:
                lse[0] = float("-inf")  # an empty partial for one row
            locs.append(torch.cat([o.reshape(-1), lse]).contiguous())
        for r in range(world):
            ranks.args[r].local = locs[r].data_ptr()
            ranks.args[r].phases = _cabi.EXCHANGE_SEND
            assert lib.pd_exchange_step(ctypes.byref(ranks.args[r])) == 0
        for r in range(world):
            ranks.args[r].phases = _cabi.EXCHANGE_MERGE
            assert lib.pd_exchange_step(ctypes.byref(ranks.args[r])) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        parts = np.stack([t[: b * hq * d].view(b, hq, d).cpu().numpy() for t in locs])
        lses = np.stack([t[b * hq * d:].view(b, hq).cpu().numpy() for t in locs])
        want, _ = po.merge_partials(parts, lses)
        for r in range(world):
            assert np.abs(ranks.outs[r].float().cpu().numpy() - want).max() <= 2e-3, (step, r)
        assert all(torch.equal(ranks.outs[0], o) for o in ranks.outs)


@pytest.mark.parametrize("name,batch,seq_len,world", [("c4", 2, 8192, 2), ("c4", 1, 20000, 4), ("c2", 3, 700, 2),
                                                      ("c3", 2, 1500, 3), ("c4", 3, 40, 4)])
def test_decode_kernel_pushes_its_own_units(name, batch, seq_len, world):
    """pd_decode_exchange: each rank's streaming decode stores its units into all buffers; the
    merged result equals the decode of the whole (concatenated) sequence.  The last case has
    ranks whose slice of the request is empty."""
    lib = _cabi.load()
    shards = [sharding.make_kv_range_shard(name, r, world, "cuda", seed=5, batch=batch, seq_len=seq_len)
              for r in range(world)]
    q = shards[0][0]
    b, hq, d = q.shape
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ranks = _Ranks(world, b, hq, d, status=status)
    steps = [pda.DecodeStep(q, cache, None, status=status, no_output=True) for _, cache in shards]
    for it in range(2):
        for r in range(world):
            steps[r].args.stream = ranks.args[r].stream
            ranks.args[r].phases = _cabi.EXCHANGE_SEND
            assert lib.pd_decode_exchange(ctypes.byref(steps[r].args), ctypes.byref(ranks.args[r])) == 0
        for r in range(world):
            ranks.args[r].phases = _cabi.EXCHANGE_MERGE
            assert lib.pd_decode_exchange(ctypes.byref(steps[r].args), ctypes.byref(ranks.args[r])) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
    caches = [c for _, c in shards]
    cat8 = lambda ts: torch.cat([t.view(torch.uint8) for t in ts]).view(ts[0].dtype)
    offsets = np.cumsum([0] + [c.num_blocks for c in caches[:-1]])
    c0 = caches[0]
    whole = dataclasses.replace(
        c0, k_cache=cat8([c.k_cache for c in caches]), v_cache=cat8([c.v_cache for c in caches]),
        k_scale=None if c0.k_scale is None else torch.cat([c.k_scale for c in caches]),
        v_scale=None if c0.v_scale is None else torch.cat([c.v_scale for c in caches]),
        block_table=torch.cat([c.block_table + int(o) for c, o in zip(caches, offsets)], dim=1),
        seq_lens=sum(c.seq_lens for c in caches))
    # a rank's slice ends on a page boundary, so the concatenated table is a valid table of the whole
    truth = c_oracle.decode(adapters.q_to_f32(q), adapters.from_torch_cache(whole))
    for r in range(world):
        helpers.assert_close(ranks.outs[r], truth, what=f"rank {r}")
    assert all(torch.equal(ranks.outs[0], o) for o in ranks.outs)


def test_merge_gives_up_when_a_rank_never_sends():
    """Rank 1 of 2 never sends: rank 0's merge waits its (shortened) limit, raises
    PD_DEV_TIMEOUT, leaves `out` alone and returns; the device keeps working."""
    lib = _cabi.load()
    b, hq, d = 2, 8, 64
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ranks = _Ranks(2, b, hq, d, status=status, wait_ns=50_000_000)
    local = torch.randn(b * hq * (d + 1), device="cuda")
    ranks.args[0].local = local.data_ptr()
    assert lib.pd_exchange_step(ctypes.byref(ranks.args[0])) == 0
    torch.cuda.synchronize()
    assert int(status.item()) & _cabi.DEV_TIMEOUT
    assert float((ranks.outs[0] - 9.0).abs().max()) == 0.0
    # a limit above one second is refused on the host
    ranks.args[0].wait_limit_ns = 2_000_000_000
    assert lib.pd_exchange_step(ctypes.byref(ranks.args[0])) == -1
    # the context is intact: an ordinary decode still matches the oracle
    q, cache = pda.synth.make("c2", device="cuda", seed=2, batch=2, seq_len=300)
    out = pda.paged_decode(q, cache)
    ref = c_oracle.decode(adapters.q_to_f32(q), adapters.from_torch_cache(cache))
    helpers.assert_close(out, ref, what="decode after a timeout")
