"""Seeded synthetic inputs shared by the golden-file generator and the parity tests.

Every case is built with numpy's PCG64 stream from its own seed, so the generator that
ran the reference (make_golden.py) and the tests that run the CUDA path and the oracle see
bit-identical q, pages, scales, block tables and lengths.  ``sha256_inputs`` guards
against drift of that stream: its digest is stored beside each golden output.

The case list mirrors the shapes the reference's own tests use
(tests/test_correctness.py:30-36, 64-110, 162-174) and adds scaled fp8, bf16, and small
versions of the five benchmark configurations.
"""

from __future__ import annotations

import dataclasses
import hashlib
import pathlib
import sys

import numpy as np

_ROOT = pathlib.Path(__file__).resolve().parents[2]
if str(_ROOT) not in sys.path:
    sys.path.insert(0, str(_ROOT))

from oracle.paged_decode_oracle import OracleCache, quantize_int8  # noqa: E402


@dataclasses.dataclass(frozen=True)
class Case:
    name: str
    hq: int
    hkv: int
    d: int
    page: int
    kv_dtype: str
    lens: tuple
    seed: int = 0
    scaled: bool | None = None  # None: int8 yes, others no
    fill: str = "normal"        # "normal": N(0,1) then stored/quantized; "uniform_int8": c3 style
    scale_kind: str = "quant"   # "quant" | "absnormal" (c3) | "uniform" (c4)
    shuffle: bool = True
    slack: int = 0
    io_dtype: str = "fp16"

    @property
    def batch(self) -> int:
        return len(self.lens)


def _f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = x.astype(np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def _f16_to_e5m2_bits(x: np.ndarray) -> np.ndarray:
    h = x.astype(np.float16).view(np.uint16).astype(np.uint32)
    return ((h + 0x7F + ((h >> 8) & 1)) >> 8).astype(np.uint8)


def lognormal_lens(rng: np.random.Generator, n: int, mu: float, sigma: float, lo: int, hi: int,
                   ones: int) -> tuple:
    z = rng.standard_normal(n)
    lens = np.clip(np.rint(np.exp(mu + sigma * z)), lo, hi).astype(np.int64)
    lens[rng.choice(n, size=ones, replace=False)] = 1
    return tuple(int(v) for v in lens)


def build(case: Case) -> tuple[np.ndarray, OracleCache]:
    """q (fp16, or bf16 bits when io_dtype is bf16) and the paged cache of a case."""
    rng = np.random.Generator(np.random.PCG64(case.seed))
    lens = np.asarray(case.lens, dtype=np.int32)
    pages = (lens.astype(np.int64) + case.page - 1) // case.page
    used = int(pages.sum())
    pool = used + case.slack
    shape = (pool, case.page, case.hkv, case.d)
    scaled = case.kv_dtype == "int8" if case.scaled is None else case.scaled

    def draw_store():
        if case.fill == "uniform_int8":
            return rng.integers(-127, 128, size=shape, dtype=np.int8), None
        raw = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
        if case.kv_dtype == "fp16":
            return raw, None
        if case.kv_dtype == "bf16":
            return _f32_to_bf16_bits(raw.astype(np.float32)), None
        if case.kv_dtype == "fp8_e5m2":
            return _f16_to_e5m2_bits(raw), None
        return quantize_int8(raw)

    def draw_scale(from_quant):
        if not scaled:
            return None
        if case.scale_kind == "quant" and from_quant is not None:
            return from_quant
        if case.scale_kind == "absnormal":
            s = np.abs(rng.standard_normal(shape[:3], dtype=np.float32)) / 127.0 + 1e-4
        else:
            s = rng.uniform(0.5, 2.0, size=shape[:3]).astype(np.float32)
        return s.astype(np.float16)

    k_cache, kq = draw_store()
    k_scale = draw_scale(kq)
    v_cache, vq = draw_store()
    v_scale = draw_scale(vq)

    order = rng.permutation(pool)[:used] if case.shuffle else np.arange(used)
    table = np.zeros((case.batch, max(1, int(pages.max()))), dtype=np.int32)
    at = 0
    for row, n in enumerate(pages):
        table[row, :n] = order[at:at + n]
        at += int(n)

    q = rng.standard_normal((case.batch, case.hq, case.d), dtype=np.float32).astype(np.float16)
    if case.io_dtype == "bf16":
        q = _f32_to_bf16_bits(q.astype(np.float32))

    cache = OracleCache(num_q_heads=case.hq, num_kv_heads=case.hkv, head_dim=case.d,
                        block_size=case.page, kv_dtype=case.kv_dtype, k_cache=k_cache,
                        v_cache=v_cache, k_scale=k_scale, v_scale=v_scale,
                        block_table=table, seq_lens=lens)
    return q, cache


def q_as_f32(case: Case, q: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(q) if case.io_dtype == "bf16" else q.astype(np.float32)


def sha256_inputs(q: np.ndarray, cache: OracleCache) -> str:
    h = hashlib.sha256()
    for a in (q, cache.k_cache, cache.v_cache, cache.k_scale, cache.v_scale,
              cache.block_table, cache.seq_lens):
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def sha256_valid_rows(dense: np.ndarray, lens: np.ndarray) -> str:
    """Digest of a dense [B, Hkv, S, D] gather with positions >= length zeroed."""
    d = np.array(dense, copy=True)
    for b, n in enumerate(lens):
        d[b, :, int(n):, :] = 0
    return hashlib.sha256(np.ascontiguousarray(d).view(np.uint16).tobytes()).hexdigest()


def _mini_c5_lens() -> tuple:
    rng = np.random.Generator(np.random.PCG64(505))
    return lognormal_lens(rng, 16, np.log(256.0), 1.2, 1, 4096, ones=2)


def _c1_lens() -> tuple:
    rng = np.random.Generator(np.random.PCG64(101))
    return tuple(int(v) for v in rng.integers(64, 161, size=24))


_L8B = dict(hq=32, hkv=8, d=128)

CASES: tuple[Case, ...] = tuple(
    # tests/test_correctness.py:36 (B, S) list on the Llama-3-8B shape
    [Case(f"llama8b_b{b}_s{s}", page=16, kv_dtype="fp16", lens=(s,) * b, seed=0, **_L8B)
     for b, s in ((2, 64), (2, 65), (3, 300), (1, 1024), (4, 1023), (2, 4097))]
    # tests/test_correctness.py:64-70 quantized caches
    + [Case(f"llama8b_{kd}_s2048", page=16, kv_dtype=kd, lens=(2048, 2048), seed=0, **_L8B)
       for kd in ("fp8_e5m2", "int8")]
    # tests/test_correctness.py:73-78 page sizes
    + [Case(f"llama8b_page{p}_s1000", page=p, kv_dtype="fp16", lens=(1000,) * 3, seed=0, **_L8B)
       for p in (16, 32, 64)]
    + [
        # tests/test_correctness.py:81-90 ragged batch incl. length 1 and empty splits
        Case("llama8b_ragged", page=16, kv_dtype="fp16",
             lens=(7, 1, 4096, 513, 16, 2047, 64, 129), seed=3, **_L8B),
        # tests/test_correctness.py:93-97 group of one
        Case("mha_group1_s512", hq=8, hkv=8, d=128, page=16, kv_dtype="fp16", lens=(512, 512), seed=0),
        # tests/test_correctness.py:100-110 ascending block table
        Case("llama8b_sequential_s1024", page=16, kv_dtype="fp16", lens=(1024, 1024), seed=5,
             shuffle=False, **_L8B),
    ]
    # tests/test_correctness.py:162-174 other model shapes
    + [Case(f"shape_{hq}x{hkv}x{d}_s777", hq=hq, hkv=hkv, d=d, page=16, kv_dtype="fp16",
            lens=(777,) * 3, seed=7)
       for hq, hkv, d in ((64, 8, 128), (32, 8, 64), (14, 2, 64), (16, 2, 64))]
    + [
        # extensions beyond the reference's tests
        Case("llama8b_e5m2_scaled_s700", page=16, kv_dtype="fp8_e5m2", lens=(700, 333), seed=13,
             scaled=True, scale_kind="uniform", **_L8B),
        Case("llama8b_bf16_s300", page=16, kv_dtype="bf16", lens=(300, 41), seed=17, io_dtype="bf16",
             **_L8B),
        Case("int8_d64_s500", hq=16, hkv=2, d=64, page=16, kv_dtype="int8", lens=(500, 77), seed=19),
        # the five benchmark configurations: c1 in full, c2-c5 scaled down
        Case("c1_qwen05b", hq=14, hkv=2, d=64, page=16, kv_dtype="fp16", lens=_c1_lens(), seed=101,
             slack=256 - sum((n + 15) // 16 for n in _c1_lens())),
        Case("c2_mini", page=16, kv_dtype="fp16", lens=(2048, 3111, 1500, 2600), seed=202, **_L8B),
        Case("c3_mini", hq=64, hkv=8, d=128, page=16, kv_dtype="int8", lens=(1024,) * 4, seed=303,
             fill="uniform_int8", scale_kind="absnormal"),
        Case("c4_mini", page=16, kv_dtype="fp8_e5m2", lens=(16384,), seed=404, scaled=True,
             scale_kind="uniform", **_L8B),
        Case("c5_mini", hq=28, hkv=4, d=128, page=32, kv_dtype="fp16", lens=_mini_c5_lens(), seed=505),
    ]
)

BY_NAME = {c.name: c for c in CASES}
