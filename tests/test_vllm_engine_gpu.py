"""A real vLLM engine (random weights, Qwen2.5-0.5B attention shape) served by the B200 backend.

Runs ``examples/vllm_engine_check.py`` in its own process: the engine generates from the same
seeded prompts with its stock Triton attention backend and with this library registered as the
CUSTOM backend; the script compares log-probabilities step by step and reads the call counters
(the check the reference's serving bench prints, ``integration/bench_vllm.py:162-170``).
"""

from __future__ import annotations

import importlib.util
import json
import pathlib
import subprocess
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _run_check(*flags):
    if importlib.util.find_spec("vllm") is None:
        pytest.skip("vLLM is not installed")
    run = subprocess.run([sys.executable, str(ROOT / "examples" / "vllm_engine_check.py"), *flags],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    lines = [ln for ln in run.stdout.splitlines() if ln.startswith('{"check"')]
    assert lines, run.stdout[-2000:] + run.stderr[-4000:]
    res = json.loads(lines[-1])
    assert run.returncode == 0 and res["ok"], res
    assert res["steps_compared"] >= 48 and res["max_abs_logprob_delta"] <= res["tol"]
    return res


@pytest.mark.gpu
def test_engine_decode_steps_are_served_here_and_match_the_stock_backend():
    res = _run_check()
    # every pure-decode step of every layer ran here; only prefill and profiling were delegated
    assert res["stats"]["decode_calls"] == res["expected_decode_calls"]
    assert res["stats"]["decode_tokens"] == res["expected_decode_calls"] * 24
    assert 0 < res["stats"]["delegated_calls"] < res["stats"]["decode_calls"]


@pytest.mark.gpu
def test_engine_captures_the_decode_path_into_its_cuda_graphs():
    """The engine records whole decode batches into CUDA graphs and replays them: the decode
    call must be capturable as the engine issues it (no synchronisation, lengths read on the
    device at replay) and the replays must give the stock backend's results."""
    res = _run_check("--cudagraph")
    assert res["cudagraph"] and res["stats"]["decode_calls"] > 0


@pytest.mark.gpu
def test_engine_with_the_flash_attention_parent():
    """The variant that delegates prefill and mixed batches to the engine's FlashAttention
    backend (cache laid out [2, NB, PAGE, H, D]): every pure-decode call still runs here and the
    tokens match the stock FlashAttention backend's."""
    if importlib.util.find_spec("vllm") is None or importlib.util.find_spec(
            "vllm.v1.attention.backends.flash_attn") is None:
        pytest.skip("the engine's FlashAttention backend is not installed")
    res = _run_check("--parent", "flash")
    assert res["timing"]["parent"] == "flash"
    assert res["stats"]["decode_calls"] == res["expected_decode_calls"]
    assert res["timing"]["delegated_attention_calls"] > 0
