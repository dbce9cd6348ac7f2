"""CPU-side checks of the native boundary: the library loads, exports what the header
declares, validates arguments without a device, and the host policies behave."""

from __future__ import annotations

import ctypes
import pathlib
import re

import pytest
import torch

import paged_decode_attention_b200 as pda
from paged_decode_attention_b200 import _cabi, decode as pdec

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "paged_decode.h").read_text()
    declared = set(re.findall(r"PD_API\s+[\w\s\*]+?\b(pd_\w+)\s*\(", header))
    assert declared, "no declarations found"
    lib = _cabi.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(_cabi.EXPORTS)
    assert lib.pd_abi_version() == _cabi.ABI_VERSION


def test_struct_layout_matches_header_field_order():
    header = (ROOT / "include" / "paged_decode.h").read_text()
    body = header.split("typedef struct PdDecodeArgs {")[1].split("} PdDecodeArgs;")[0]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for stmt in body.split(";"):
        stmt = stmt.strip()
        if not stmt:
            continue
        for part in stmt.split(","):
            names.append(re.findall(r"(\w+)\s*$", part.strip())[0])
    assert names == [f[0] for f in _cabi.PdDecodeArgs._fields_]


def test_flag_and_size_constants_match_the_header():
    """The Python side's copies of the header's #defines."""
    import re
    text = (ROOT / "include" / "paged_decode.h").read_text()
    defines = {m.group(1): m.group(2) for m in re.finditer(r"#define\s+(PD_\w+)\s+\(?([-\w<> ]+?)\)?\s*(?:/\*|$)", text, re.M)}

    def value(name):
        return eval(defines[name].replace("u", ""))  # noqa: S307 - literals of the header

    assert value("PD_ABI_VERSION") == _cabi.ABI_VERSION
    for name in ("COUNTERS_ZERO", "EQUAL_TILE_SHARES", "HOST_DIRECT_OUT", "HOST_DIRECT_Q", "HOST_DIRECT_BT", "STAGE_Q"):
        assert value(f"PD_FLAG_{name}") == getattr(_cabi, f"FLAG_{name}"), name
    flags = [value(f"PD_FLAG_{n}") for n in ("COUNTERS_ZERO", "EQUAL_TILE_SHARES", "HOST_DIRECT_OUT", "HOST_DIRECT_Q",
                                             "HOST_DIRECT_BT", "STAGE_Q")]
    assert sorted(flags) == [1, 2, 4, 8, 16, 32]
    assert value("PD_STATIC_SCRATCH_BYTES") == _cabi.STATIC_SCRATCH_BYTES
    assert (value("PD_EXCHANGE_SEND"), value("PD_EXCHANGE_MERGE")) == (_cabi.EXCHANGE_SEND, _cabi.EXCHANGE_MERGE)
    assert (value("PD_DEV_BAD_BLOCK"), value("PD_DEV_TIMEOUT")) == (_cabi.DEV_BAD_BLOCK, _cabi.DEV_TIMEOUT)


def test_status_strings():
    assert _cabi.status_string(0) == "ok"
    for rc in (-1, -2, -3, -4):
        assert _cabi.status_string(rc) not in ("ok", "unknown status")


def _cpu_case(hq=32, hkv=8, d=128, page=16, kv_dtype="fp16", b=2, s=100):
    cache = pda.allocate(pda.ModelShape(hq, hkv, d, "t"), b, s, block_size=page, kv_dtype=kv_dtype,
                         device="cpu", seed=1)
    q = torch.zeros((b, hq, d), dtype=torch.float16)
    return q, cache


def test_validation_without_a_device():
    lib = _cabi.load()
    q, cache = _cpu_case()
    args = pdec.build_args(q, cache, torch.empty_like(q), sm_count=148)
    assert lib.pd_select_kernel(ctypes.byref(args)) in (1, 2)
    n = ctypes.c_uint64(123)
    assert lib.pd_workspace_bytes(ctypes.byref(args), ctypes.byref(n)) == 0

    bad = pdec.build_args(q, cache, torch.empty_like(q), sm_count=148)
    bad.num_q_heads = 30  # not a multiple of the kv heads
    assert lib.pd_select_kernel(ctypes.byref(bad)) == -1
    bad = pdec.build_args(q, cache, torch.empty_like(q), sm_count=148)
    bad.head_dim = 96
    assert lib.pd_select_kernel(ctypes.byref(bad)) == -2
    bad = pdec.build_args(q, cache, torch.empty_like(q), sm_count=148)
    bad.kv_dtype = 3  # int8 without scales
    assert lib.pd_select_kernel(ctypes.byref(bad)) == -1
    bad = pdec.build_args(q, cache, torch.empty_like(q), sm_count=148)
    bad.block_n = 24
    assert lib.pd_select_kernel(ctypes.byref(bad)) == -1
    assert lib.pd_select_kernel(None) == -1
    assert lib.pd_decode(None) == -1 and lib.pd_merge(None) == -1 and lib.pd_gather(None) == -1


@pytest.mark.parametrize("kv_dtype,d,expect", [("fp16", 32, 2), ("fp16", 64, 2), ("fp16", 128, 2), ("fp16", 256, 2),
                                               ("bf16", 32, 2), ("int8", 64, 2), ("int8", 128, 2), ("int8", 256, 2),
                                               ("fp8_e5m2", 64, 2), ("fp8_e5m2", 256, 2),
                                               ("int8", 32, 1), ("fp8_e5m2", 32, 1)])
def test_kernel_selection_by_row_width(kv_dtype, d, expect):
    """The streaming kernel (2) takes rows of 64 bytes and of one, two or four 128-byte pieces;
    32-byte rows go to the general kernel (1)."""
    q, cache = _cpu_case(hq=16, hkv=4, d=d, kv_dtype=kv_dtype)
    if kv_dtype == "bf16":
        q = q.to(torch.bfloat16)
    args = pdec.build_args(q, cache, torch.empty_like(q), sm_count=148)
    assert _cabi.load().pd_select_kernel(ctypes.byref(args)) == expect


def test_kernel_selection_at_the_virtual_sequence_limit():
    """The streaming kernel lays out at most 4096 virtual sequences (requests x head blocks x
    explicit splits); one more and the request goes to the general kernel, or is refused when the
    streaming kernel was asked for by name."""
    lib = _cabi.load()
    q, cache = _cpu_case(hq=32, hkv=8, d=128, b=2, s=40)
    args = pdec.build_args(q, cache, torch.empty_like(q), sm_count=148)
    for batch, splits, expect in ((4096, 1, 2), (4097, 1, 1), (512, 8, 2), (513, 8, 1), (1, 1024, 2)):
        args.batch, args.num_splits, args.kernel = batch, splits, 0
        assert lib.pd_select_kernel(ctypes.byref(args)) == expect, (batch, splits)
    args.batch, args.num_splits, args.kernel = 4097, 1, 2
    assert lib.pd_select_kernel(ctypes.byref(args)) == -2
    # 16 kv heads are two head blocks of eight: half as many requests fit
    q, cache = _cpu_case(hq=32, hkv=16, d=128, b=2, s=40)
    args = pdec.build_args(q, cache, torch.empty_like(q), sm_count=148)
    for batch, expect in ((2048, 2), (2049, 1)):
        args.batch = batch
        assert lib.pd_select_kernel(ctypes.byref(args)) == expect, batch


def test_simple_kernel_workspace_grows_with_splits():
    lib = _cabi.load()
    q, cache = _cpu_case(b=2, s=4096)
    sizes = []
    for splits in (1, 2, 8):
        args = pdec.build_args(q, cache, torch.empty_like(q), num_splits=splits, kernel="simple",
                               sm_count=148)
        n = ctypes.c_uint64(0)
        assert lib.pd_workspace_bytes(ctypes.byref(args), ctypes.byref(n)) == 0
        sizes.append(n.value)
    assert sizes[0] == 0 and sizes[1] >= 2 * 2 * 32 * 129 * 4 and sizes[2] >= 4 * sizes[1] - 4096


def test_python_entry_refuses_cpu_tensors():
    q, cache = _cpu_case()
    with pytest.raises(_cabi.NativeLibraryError):
        pda.paged_decode(q, cache)
    with pytest.raises(_cabi.NativeLibraryError):
        pda.gather_contiguous(cache)


def test_entry_point_asserts_like_the_reference():
    q, cache = _cpu_case()
    with pytest.raises(AssertionError):
        pdec.build_args(q[:, :, :64], cache, None)
    with pytest.raises(AssertionError):
        pdec.build_args(q, cache, None, block_n=40)


def test_pick_num_splits_policy():
    f = pda.pick_num_splits
    assert f(64, 8, 8192, 148, 64) >= 1
    assert f(256, 8, 8192, 148, 64) == 1          # enough CTAs already
    assert f(4, 8, 131072, 148, 64) > 8           # long context, few requests: split deep
    assert f(1, 8, 128, 148, 64) == 1             # too short to split
    assert f(1, 1, 10**6, 148, 64) <= 128
    for b in (1, 3, 24, 100):
        prev = None
        for s in (64, 512, 4096, 32768, 262144):
            n = f(b, 2, s, 148, 64)
            assert n >= 1 and (prev is None or n >= prev)  # never fewer splits for longer context
            assert n == 1 or s // n >= 4 * 64              # at least four tiles per split
            prev = n
    assert f(0, 8, 100, 148, 64) == 1 and f(4, 8, 100, 0, 64) == 1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.load()


def test_header_is_plain_c():
    """The boundary is a C ABI: the header must compile as C99 with no C++ or CUDA in sight."""
    import shutil
    import subprocess

    gcc = "/usr/bin/gcc" if pathlib.Path("/usr/bin/gcc").exists() else shutil.which("gcc")
    if not gcc:
        pytest.skip("no C compiler")
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-x", "c",
                        str(ROOT / "include" / "paged_decode.h")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def _header_fields(struct: str) -> list[str]:
    header = (ROOT / "include" / "paged_decode.h").read_text()
    body = header.split(f"typedef struct {struct} {{")[1].split(f"}} {struct};")[0]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for stmt in body.split(";"):
        stmt = stmt.strip()
        if not stmt:
            continue
        for part in stmt.split(","):
            names.append(re.findall(r"(\w+)\s*$", part.strip())[0])
    return names


@pytest.mark.parametrize("struct", ["PdExchangeArgs", "PdMergeArgs", "PdCacheWriteArgs", "PdHostIO"])
def test_other_struct_layouts_match_header_field_order(struct):
    assert _header_fields(struct) == [f[0] for f in getattr(_cabi, struct)._fields_]


@pytest.mark.parametrize("rows,d", [(1, 64), (6, 128), (14, 64), (128, 128), (910, 2), (3, 32)])
@pytest.mark.parametrize("world", [1, 2, 3, 8, 16])
def test_exchange_slots_are_aligned_and_disjoint(world, rows, d):
    """A partial is rows * (d + 1) words of 8 bytes, an odd count for odd row counts; every
    (parity, rank) slot must still start on a 16-byte boundary (two words are stored at a time),
    must not overlap its neighbour and must end inside the buffer."""
    lib = _cabi.load()
    total = int(lib.pd_exchange_bytes(world, rows, d))
    assert total > 0 and total % 256 == 0
    n_bytes = rows * (d + 1) * 8
    offs = []
    for parity in (0, 1):
        for r in range(world):
            off = int(lib.pd_exchange_part_offset(world, rows, d, parity, r))
            assert off % 256 == 0 and off >= 256
            offs.append(off)
    assert offs == sorted(offs)
    for a, b in zip(offs, offs[1:]):
        assert b - a >= n_bytes
    assert offs[-1] + n_bytes <= total


def test_exchange_sizes_reject_bad_arguments():
    lib = _cabi.load()
    assert lib.pd_exchange_bytes(17, 8, 64) == 0       # more than 16 ranks
    assert lib.pd_exchange_bytes(2, 8, 0) == 0
    assert lib.pd_exchange_part_offset(2, 8, 64, 2, 0) == 0
    assert lib.pd_exchange_part_offset(2, 8, 64, 0, 2) == 0
    x = _cabi.PdExchangeArgs()
    assert lib.pd_exchange_step(ctypes.byref(x)) == -1
    assert lib.pd_decode_exchange(None, ctypes.byref(x)) == -1


def test_workspace_handed_out_during_capture_is_never_dropped(monkeypatch):
    """A graph captured with a cached workspace keeps its raw address; when a larger request
    replaces the cache entry, the old buffer must stay referenced."""
    made = []

    def fake_empty(n, dtype=None, device=None):
        t = torch.zeros(int(n), dtype=dtype)
        made.append(t)
        return t

    monkeypatch.setattr(pdec.torch, "empty", fake_empty)
    monkeypatch.setattr(pdec.torch.cuda, "is_current_stream_capturing", lambda: True)
    monkeypatch.setattr(pdec, "_ws_cache", {})
    monkeypatch.setattr(pdec, "_ws_captured", [])
    dev = torch.device("cuda", 0)
    small = pdec._workspace(dev, 1000, stream=5)
    again = pdec._workspace(dev, 2000, stream=5)
    assert again is small and len(pdec._ws_captured) == 1
    big = pdec._workspace(dev, 8 << 20, stream=5)
    assert big is not small
    assert any(t is small for t in pdec._ws_captured) and any(t is big for t in pdec._ws_captured)
    monkeypatch.setattr(pdec.torch.cuda, "is_current_stream_capturing", lambda: False)
    other = pdec._workspace(dev, 100, stream=6)
    assert not any(t is other for t in pdec._ws_captured)
