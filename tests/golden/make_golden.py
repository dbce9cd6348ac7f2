"""Produce tests/golden/golden_v1.npz by running the UNMODIFIED reference on the CPU.

Usage:  python tests/golden/make_golden.py --ref /path/to/paged-decode-attention

The reference tree is imported, never copied.  For every case of cases.CASES the file
stores what the reference computes on the seeded inputs of cases.build():

  <name>/out_f32     reference_decode(q.float(), cache)   fp32 result before rounding
  <name>/k_sha,v_sha digests of gather_contiguous(cache) with positions >= length zeroed
  <name>/in_sha      digest of the inputs (guards the seeded stream)

plus known-answer vectors of the helpers on the path: quantize_kv / dequantize_kv,
allocate's block tables and a digest of its pages, and a table of pick_num_splits.
The test suite only reads the .npz; this script needs the reference and is run by hand.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402


def _to_torch_store(a: np.ndarray, kv_dtype: str) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    if kv_dtype == "bf16":
        return t.view(torch.bfloat16)
    if kv_dtype == "fp8_e5m2":
        return t.view(torch.float8_e5m2)
    return t


def _ref_cache(ref, case: cases.Case, oc):
    """Reference PagedKVCache over the case's arrays.

    Scaled fp8 does not exist in the reference (its fp8 path ignores scales,
    pagedattn/cache.py:57-58), so such a cache is handed over as the fp16 cache holding
    fp16(fp8) * scale rounded to fp16 — the reference's int8 dequantisation rule
    (pagedattn/cache.py:59-61) applied to fp8.
    """
    shape = ref.ModelShape(case.hq, case.hkv, case.d, case.name)
    k = _to_torch_store(oc.k_cache, case.kv_dtype)
    v = _to_torch_store(oc.v_cache, case.kv_dtype)
    ks = None if oc.k_scale is None else torch.from_numpy(oc.k_scale)
    vs = None if oc.v_scale is None else torch.from_numpy(oc.v_scale)
    kv_dtype = case.kv_dtype
    if case.kv_dtype == "fp8_e5m2" and ks is not None:
        k = (k.to(torch.float16) * ks.unsqueeze(-1)).to(torch.float16)
        v = (v.to(torch.float16) * vs.unsqueeze(-1)).to(torch.float16)
        ks = vs = None
        kv_dtype = "fp16"
    return ref.PagedKVCache(shape=shape, block_size=case.page, kv_dtype=kv_dtype, k_cache=k,
                            v_cache=v, k_scale=ks, v_scale=vs,
                            block_table=torch.from_numpy(oc.block_table),
                            seq_lens=torch.from_numpy(oc.seq_lens))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("PAGEDATTN_REF"),
                    help="checkout of the reference project (or set PAGEDATTN_REF)")
    ap.add_argument("--out", default=str(HERE / "golden_v1.npz"))
    args = ap.parse_args()
    if not args.ref:
        ap.error("give --ref or set PAGEDATTN_REF to the reference checkout")
    sys.path.insert(0, args.ref)
    import pagedattn as ref  # the reference package, unmodified
    from pagedattn.cache import dequantize_kv, quantize_kv

    torch.set_num_threads(8)
    store: dict[str, np.ndarray] = {}

    for case in cases.CASES:
        q_np, oc = cases.build(case)
        rc = _ref_cache(ref, case, oc)
        q_t = torch.from_numpy(q_np)
        if case.io_dtype == "bf16":
            q_t = q_t.view(torch.bfloat16)
        out_f32 = ref.reference_decode(q_t.float(), rc)
        # what the reference returns for a 16-bit q is this fp32 result rounded to q's dtype
        assert torch.equal(ref.reference_decode(q_t, rc), out_f32.to(q_t.dtype))
        kd, vd = ref.gather_contiguous(rc)
        store[f"{case.name}/out_f32"] = out_f32.numpy()
        store[f"{case.name}/k_sha"] = np.array(cases.sha256_valid_rows(kd.numpy(), oc.seq_lens))
        store[f"{case.name}/v_sha"] = np.array(cases.sha256_valid_rows(vd.numpy(), oc.seq_lens))
        store[f"{case.name}/in_sha"] = np.array(cases.sha256_inputs(q_np, oc))
        print(f"{case.name:34s} |out| max {out_f32.abs().max():.4f}")

    # quantize_kv / dequantize_kv known answers (pagedattn/cache.py:33-62)
    rng = np.random.Generator(np.random.PCG64(9001))
    x = (rng.standard_normal((37, 4, 64), dtype=np.float32) * 1.7).astype(np.float16)
    x[3, 1] = 0  # all-zero row exercises the 1e-6 floor
    xt = torch.from_numpy(x)
    q8, s8 = quantize_kv(xt, "int8")
    f8, _ = quantize_kv(xt, "fp8_e5m2")
    store["quant/x"] = x
    store["quant/int8"] = q8.numpy()
    store["quant/int8_scale"] = s8.numpy()
    store["quant/int8_dequant"] = dequantize_kv(q8, s8, "int8").numpy()
    store["quant/e5m2_bits"] = f8.view(torch.uint8).numpy()
    store["quant/e5m2_dequant"] = dequantize_kv(f8, None, "fp8_e5m2").numpy()

    # allocate() on the CPU (pagedattn/cache.py:105-184): tables and a digest of the pages
    for tag, kw in (("shuffled", dict(shuffle=True)), ("sequential", dict(shuffle=False)),
                    ("slack_int8", dict(shuffle=True, kv_dtype="int8", slack_blocks=5))):
        c = ref.allocate(ref.ModelShape(8, 2, 64, "t"), 3, [5, 40, 17], block_size=16,
                         device="cpu", seed=3, **kw)
        store[f"allocate/{tag}/block_table"] = c.block_table.numpy()
        store[f"allocate/{tag}/seq_lens"] = c.seq_lens.numpy()
        raw = c.k_cache.numpy().tobytes() + c.v_cache.numpy().tobytes()
        if c.k_scale is not None:
            raw += c.k_scale.numpy().tobytes() + c.v_scale.numpy().tobytes()
        store[f"allocate/{tag}/pages_sha"] = np.array(hashlib.sha256(raw).hexdigest())
        store[f"allocate/{tag}/bytes_read"] = np.array(c.bytes_read_per_decode_step())

    # pick_num_splits table (pagedattn/triton_decode.py:248-263)
    grid = [(b, h, s, sm) for b in (1, 4, 24, 64, 256) for h in (2, 8)
            for s in (64, 1000, 8192, 131072) for sm in (16, 148)]
    store["splits/args"] = np.array(grid, dtype=np.int64)
    store["splits/value"] = np.array([ref.pick_num_splits(b, h, s, sm, 64) for b, h, s, sm in grid],
                                     dtype=np.int64)

    np.savez_compressed(args.out, **store)
    print("wrote", args.out, pathlib.Path(args.out).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
