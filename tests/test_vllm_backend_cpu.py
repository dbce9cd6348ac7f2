"""Host-side tests of the vLLM override with fake engine objects (no GPU, no model).

The reference has no test of its backend (only a run-time guard that decode_calls > 0,
integration/bench_vllm.py:162-170); these cover the delegation predicate, the shape gate,
the zero-copy cache views, the counters and the registration.
"""

from __future__ import annotations

import types

import pytest
import torch

from paged_decode_attention_b200 import vllm_backend as vb


def _impl(**kw):
    base = dict(num_heads=32, num_kv_heads=8, head_size=128, scale=0.0883, kv_cache_dtype="auto",
                alibi_slopes=None, logits_soft_cap=None, sliding_window=(-1, -1), sinks=None,
                chunk_lookback=-1, attn_type="decoder", kv_sharing_target_layer_name=None)
    base.update(kw)
    return types.SimpleNamespace(**base)


def _meta(n=3, max_blocks=4, **kw):
    base = dict(num_actual_tokens=n, max_query_len=1, max_seq_len=40,
                seq_lens=torch.tensor([17, 40, 5, 9][: n + 1], dtype=torch.int32),
                block_table=torch.arange((n + 1) * max_blocks, dtype=torch.int32).view(n + 1, max_blocks),
                use_cascade=False, mm_prefix_range_tensor=None)
    base.update(kw)
    return types.SimpleNamespace(**base)


def _kv(nb=20, page=16, h=8, d=128, dtype=torch.float16):
    return torch.zeros((nb, 2, page, h, d), dtype=dtype)


def test_supports_shape():
    assert vb.supports_shape(32, 8, 128) == (True, "")
    assert vb.supports_shape(14, 2, 64)[0]
    assert not vb.supports_shape(30, 8, 128)[0]
    assert not vb.supports_shape(32, 8, 96)[0]
    assert not vb.supports_shape(32, 0, 128)[0]


@pytest.mark.parametrize("change,expect", [
    (dict(meta=None), "profiling"),
    (dict(output=None), "no output"),
    (dict(output_scale=torch.ones(1)), "output quant"),
    (dict(output_block_scale=torch.ones(1)), "output quant"),
    (dict(kv=torch.zeros(0)), "empty"),
    (dict(impl=dict(kv_cache_dtype="fp8_e4m3")), "quantized"),
    (dict(impl=dict(alibi_slopes=[0.5])), "alibi"),
    (dict(impl=dict(logits_soft_cap=30.0)), "soft cap"),
    (dict(impl=dict(sliding_window=(127, 0))), "sliding"),
    (dict(impl=dict(sinks=torch.zeros(32))), "sinks"),
    (dict(impl=dict(attn_type="encoder_only")), "decoder"),
    (dict(metakw=dict(use_cascade=True)), "cascade"),
    (dict(metakw=dict(local_attn_metadata=object())), "local"),
    (dict(metakw=dict(mm_prefix_range_tensor=torch.zeros(1))), "multimodal"),
    (dict(metakw=dict(max_query_len=7)), "pure-decode"),
])
def test_every_reason_to_delegate(change, expect):
    impl = _impl(**change.get("impl", {}))
    meta = change["meta"] if "meta" in change else _meta(**change.get("metakw", {}))
    kv = change.get("kv", _kv())
    out = change["output"] if "output" in change else torch.zeros(4, 32, 128)
    why = vb._reason_to_delegate(impl, meta, kv, out, change.get("output_scale"),
                                 change.get("output_block_scale"))
    assert expect in why


def test_pure_decode_is_ours():
    assert vb._reason_to_delegate(_impl(), _meta(), _kv(), torch.zeros(4, 32, 128), None, None) == ""


class _FakeCall:
    def __init__(self, log):
        self.log = log

    def step_at(self, q_ptr, out_ptr, bt_ptr, sl_ptr, stream, max_seq_len=0):
        self.log.append(dict(q=q_ptr, out=out_ptr, bt=bt_ptr, sl=sl_ptr, stream=stream, max_seq_len=max_seq_len))


def _patch_native(monkeypatch, seen, log):
    def fake_prepare(q, cache, out, sm_scale):
        seen.append(dict(q=q, cache=cache, out=out, sm_scale=sm_scale))
        return _FakeCall(log)

    monkeypatch.setattr(vb, "_prepare_call", fake_prepare)
    monkeypatch.setattr(vb, "_PREPARED", {})
    monkeypatch.setattr(vb.torch.cuda, "current_stream", lambda dev=None: types.SimpleNamespace(cuda_stream=77))


def test_decode_step_builds_zero_copy_views(monkeypatch):
    seen, log = [], []
    _patch_native(monkeypatch, seen, log)
    before = dict(vb.STATS)
    kv = _kv()
    query = torch.zeros(4, 32, 128, dtype=torch.float16)   # padded to 4 tokens, 3 are real
    output = torch.zeros(4, 32 * 128, dtype=torch.float16)
    meta = _meta(n=3)
    vb._decode_step(_impl(), query, kv, meta, output)
    c = seen[0]["cache"]
    assert c.k_cache.data_ptr() == kv.data_ptr()                      # views, not copies
    assert c.v_cache.data_ptr() == kv[:, 1].data_ptr()
    assert c.k_cache.shape == (20, 16, 8, 128) and c.k_cache.stride(0) == 2 * 16 * 8 * 128
    assert c.block_size == 16 and c.kv_dtype == "fp16" and c.k_scale is None
    assert c.block_table.shape[0] == 3 and c.seq_lens.shape[0] == 3
    assert seen[0]["q"].shape == (3, 32, 128) and seen[0]["q"].data_ptr() == query.data_ptr()
    assert seen[0]["out"].shape == (3, 32, 128) and seen[0]["out"].data_ptr() == output.data_ptr()
    assert seen[0]["sm_scale"] == pytest.approx(0.0883)
    assert log[0] == dict(q=query.data_ptr(), out=output.data_ptr(), bt=meta.block_table.data_ptr(),
                          sl=meta.seq_lens.data_ptr(), stream=77, max_seq_len=40)
    assert vb.STATS["decode_calls"] == before["decode_calls"] + 1
    assert vb.STATS["decode_tokens"] == before["decode_tokens"] + 3


def test_prepared_call_is_reused_and_only_addresses_move(monkeypatch):
    """Same layer cache and batch size: prepared once; a new query buffer only changes the
    address handed over.  Another batch size or another layer's cache prepares anew."""
    seen, log = [], []
    _patch_native(monkeypatch, seen, log)
    kv, meta, impl = _kv(), _meta(n=3), _impl()
    q1 = torch.zeros(4, 32, 128, dtype=torch.float16)
    q2 = torch.zeros(4, 32, 128, dtype=torch.float16)
    out = torch.zeros(4, 32, 128, dtype=torch.float16)
    vb._decode_step(impl, q1, kv, meta, out)
    vb._decode_step(impl, q2, kv, meta, out)
    assert len(seen) == 1 and len(log) == 2
    assert log[0]["q"] == q1.data_ptr() and log[1]["q"] == q2.data_ptr()
    vb._decode_step(impl, q1, kv, _meta(n=2), out)            # other batch size
    vb._decode_step(impl, q1, _kv(), meta, out)               # other layer's cache
    assert len(seen) == 3 and len(log) == 4
    # the table is bounded
    monkeypatch.setattr(vb, "_PREPARED_CAP", 2)
    vb._decode_step(impl, q1, _kv(), meta, out)
    assert len(vb._PREPARED) <= 3


def test_bf16_cache_is_labelled(monkeypatch):
    seen, log = [], []
    _patch_native(monkeypatch, seen, log)
    vb._decode_step(_impl(), torch.zeros(4, 32, 128, dtype=torch.bfloat16), _kv(dtype=torch.bfloat16),
                    _meta(), torch.zeros(4, 32, 128, dtype=torch.bfloat16))
    assert seen[0]["cache"].kv_dtype == "bf16"


def test_env_switch_off_by_default(monkeypatch):
    monkeypatch.delenv("PAGEDATTN_VLLM_BACKEND", raising=False)
    assert vb.maybe_install_from_env() is False


@pytest.mark.skipif(not vb.HAVE_VLLM, reason="vLLM not importable")
@pytest.mark.parametrize("parent", ["triton", "flash"])
def test_forward_delegates_or_serves(monkeypatch, parent):
    if parent == "flash" and not vb.HAVE_FLASH:
        pytest.skip("the engine's FlashAttention backend is not importable")
    impl_cls = vb.PagedDecodeB200FlashImpl if parent == "flash" else vb.PagedDecodeB200Impl
    parent_cls = vb.FlashAttentionImpl if parent == "flash" else vb.TritonAttentionImpl
    backend_cls = vb.PagedDecodeB200FlashBackend if parent == "flash" else vb.PagedDecodeB200Backend
    calls = {"parent": 0, "ours": 0}

    def parent_forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None,
                       output_scale=None, output_block_scale=None):
        calls["parent"] += 1
        return output

    monkeypatch.setattr(parent_cls, "forward", parent_forward)
    monkeypatch.setattr(vb, "_decode_step", lambda *a, **k: calls.__setitem__("ours", calls["ours"] + 1))
    impl = object.__new__(impl_cls)
    for k, v in vars(_impl()).items():
        setattr(impl, k, v)
    q = torch.zeros(4, 32, 128, dtype=torch.float16)
    out = torch.zeros(4, 32, 128, dtype=torch.float16)
    delegated0 = vb.STATS["delegated_calls"]
    assert impl.forward(None, q, None, None, _kv(), _meta(), out) is out
    assert calls == {"parent": 0, "ours": 1}
    impl.forward(None, q, None, None, _kv(), _meta(max_query_len=5), out)          # prefill
    impl.forward(None, q, None, None, _kv(), None, out)                            # profiling
    impl.forward(None, q.to(torch.bfloat16), None, None, _kv(), _meta(), out)      # dtype mismatch
    impl.head_size = 96
    impl.forward(None, q, None, None, _kv(d=96), _meta(), out)                     # shape gate
    assert calls == {"parent": 4, "ours": 1}
    assert vb.STATS["delegated_calls"] == delegated0 + 4
    assert backend_cls.get_impl_cls() is impl_cls and backend_cls.get_name() == "CUSTOM"
    assert impl_cls.kv_axis == (0 if parent == "flash" else 1)


def test_flash_parent_cache_views_are_the_two_dense_halves(monkeypatch):
    """[2, NB, PAGE, H, D] (the FlashAttention backend's layout): K and V are the halves along axis 0."""
    seen, log = [], []
    _patch_native(monkeypatch, seen, log)
    kv = torch.zeros((2, 20, 16, 8, 128), dtype=torch.float16)
    impl = _impl(kv_axis=0)
    q = torch.zeros(4, 32, 128, dtype=torch.float16)
    vb._decode_step(impl, q, kv, _meta(), torch.zeros(4, 32, 128, dtype=torch.float16))
    c = seen[0]["cache"]
    assert c.k_cache.data_ptr() == kv[0].data_ptr() and c.v_cache.data_ptr() == kv[1].data_ptr()
    assert c.k_cache.shape == (20, 16, 8, 128) and c.k_cache.is_contiguous()


@pytest.mark.skipif(not vb.HAVE_VLLM, reason="vLLM not importable")
def test_install_registers_custom_backend(monkeypatch):
    from vllm.v1.attention.backends.registry import AttentionBackendEnum

    monkeypatch.setenv("PAGEDATTN_VLLM_BACKEND", "1")
    assert vb.maybe_install_from_env() is True
    assert vb.install() == vb.QUALNAME
    assert AttentionBackendEnum.CUSTOM.get_path() == vb.QUALNAME
    if vb.HAVE_FLASH:
        assert vb.install(parent="flash") == vb.QUALNAME_FLASH
        assert AttentionBackendEnum.CUSTOM.get_path() == vb.QUALNAME_FLASH
        monkeypatch.setenv("PAGEDATTN_VLLM_PARENT", "flash")
        assert vb.install() == vb.QUALNAME_FLASH
        monkeypatch.delenv("PAGEDATTN_VLLM_PARENT")
    with pytest.raises(ValueError):
        vb.install(parent="other")
    assert vb.install() == vb.QUALNAME
