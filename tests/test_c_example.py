"""The plain-C caller in examples/ — the C ABI used with no Python or torch in the process."""

from __future__ import annotations

import pathlib
import re
import subprocess

import numpy as np
import pytest

from oracle import c_oracle, paged_decode_oracle as po

ROOT = pathlib.Path(__file__).resolve().parents[1]
CUDA = pathlib.Path("/usr/local/cuda")


def _build(tmp_path) -> pathlib.Path:
    if not (CUDA / "include" / "cuda_runtime_api.h").exists() or not pathlib.Path("/usr/bin/gcc").exists():
        pytest.skip("needs gcc and the CUDA runtime headers")
    exe = tmp_path / "c_abi_decode"
    lib_dir = ROOT / "paged_decode_attention_b200"
    cmd = ["/usr/bin/gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-I", str(ROOT / "include"),
           "-I", str(CUDA / "include"), str(ROOT / "examples" / "c_abi_decode.c"),
           "-L", str(lib_dir), "-l:libpaged_decode_b200.so", "-L", str(CUDA / "lib64"), "-lcudart",
           f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{CUDA / 'lib64'}", "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_c_example_builds_and_links(tmp_path):
    _build(tmp_path)


@pytest.mark.gpu
def test_c_example_runs_and_matches_the_oracle(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr + r.stdout
    bits = [int(x, 16) for x in re.search(r"bits: (\w+) (\w+) (\w+) (\w+)", r.stdout).groups()]
    got = np.array(bits, dtype=np.uint16).view(np.float16).astype(np.float32)
    # the same inputs the C program builds
    b, hq, hkv, d, page, nb, maxb = 2, 8, 2, 64, 16, 8, 4
    i = np.arange(nb * page * hkv * d, dtype=np.int64)
    kv = (((i * 7) % 17) / 8.0 - 1.0).astype(np.float16).reshape(nb, page, hkv, d)
    j = np.arange(b * hq * d, dtype=np.int64)
    q = (((j * 5) % 13) / 8.0 - 0.75).astype(np.float16).reshape(b, hq, d)
    oc = po.OracleCache(hq, hkv, d, page, "fp16", kv, kv, None, None,
                        np.array([[5, 1, 6, 0], [3, 7, 0, 0]], dtype=np.int32), np.array([40, 17], dtype=np.int32))
    ref = c_oracle.decode(q.astype(np.float32), oc, sm_scale=0.125)
    assert np.abs(got - ref[0, 0, :4]).max() <= 2e-3
