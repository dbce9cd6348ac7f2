"""Serve decode steps of a real vLLM engine with this library and compare with the stock backend.

The reference's claim for its backend is that it serves every pure-decode step of a vLLM
engine while the rest is delegated (its ``integration/bench_vllm.py:162-170`` prints the call
counters to prove it).  This script makes the same check for the B200 backend without model
weights on disk: it writes a small Qwen2-style ``config.json`` with the attention shape of
Qwen2.5-0.5B (14 query heads, 2 KV heads, head_dim 64), lets the engine build the model with
random weights (re-drawn here from a seeded generator so that attention is not degenerate),
and generates greedily from seeded token prompts twice — once with the engine's own attention
backend, once with ``attention_backend="CUSTOM"`` after ``install()``.  ``--parent`` picks the
engine backend that the non-decode calls are delegated to (and that the stock run uses):
``triton`` as in the reference, or ``flash`` — the reference's own next step
(README.md:211-214), which keeps the decode path here and runs prefill on the engine's
FlashAttention kernel.

It checks that (1) the decode counter shows layers x decode-steps calls served here and only
prefill/profiling calls delegated, and (2) at every generation step where both runs are still on
the same token prefix, the log-probabilities of the tokens both report agree within ``--tol``.

Needs a GPU and vLLM; prints one JSON line and exits non-zero when a check fails.
Run: ``python examples/vllm_engine_check.py``
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import pathlib
import statistics
import sys
import tempfile

os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")  # engine in this process: counters visible
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parents[1]))

LAYERS = 4
CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 896, "num_attention_heads": 14, "num_key_value_heads": 2,
    "num_hidden_layers": LAYERS, "intermediate_size": 2048, "vocab_size": 2048,
    "max_position_embeddings": 2048, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "hidden_act": "silu", "tie_word_embeddings": True, "torch_dtype": "float16",
    "bos_token_id": 1, "eos_token_id": 2, "use_sliding_window": False,
}


def _redraw_weights(model):
    """Seeded N(0, 0.05) matrices, unit norm gains, zero biases: the same model for both runs."""
    import torch

    gen = torch.Generator(device="cpu").manual_seed(1234)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            if p.dim() >= 2:
                p.copy_((torch.randn(p.shape, generator=gen) * 0.05).to(p.dtype))
            elif "norm" in name:
                p.fill_(1.0)
            else:
                p.zero_()
    return True


def _prompts(batch: int, lo: int, hi: int, vocab: int):
    import numpy as np

    rng = np.random.Generator(np.random.PCG64(0))
    lens = rng.integers(lo, hi + 1, size=batch)
    return [rng.integers(3, vocab, size=int(n)).tolist() for n in lens]


def _generate(model_dir: str, backend: str, prompts, steps: int, cudagraph: bool):
    import torch
    from vllm import LLM, SamplingParams
    from vllm.inputs import TokensPrompt

    # eager, or pure-decode batches captured whole into CUDA graphs (no compiler pass)
    mode = ({"enforce_eager": False,
             "compilation_config": {"mode": 0, "cudagraph_mode": "FULL_DECODE_ONLY",
                                    "cudagraph_capture_sizes": [8, 16, 24, 32]}}
            if cudagraph else {"enforce_eager": True})
    llm = LLM(model=model_dir, skip_tokenizer_init=True, load_format="dummy", dtype="float16",
              attention_backend=backend, max_model_len=1024,
              kv_cache_memory_bytes=2 << 30, max_num_seqs=32, seed=0,
              enable_prefix_caching=False, **mode)
    llm.apply_model(_redraw_weights)
    params = SamplingParams(temperature=0.0, max_tokens=steps, logprobs=5, ignore_eos=True,
                            detokenize=False)
    outs = llm.generate([TokensPrompt(prompt_token_ids=p) for p in prompts], params, use_tqdm=False)
    result = []
    for o in outs:
        c = o.outputs[0]
        result.append((list(c.token_ids),
                       [{int(t): float(lp.logprob) for t, lp in step.items()} for step in c.logprobs]))
    del llm
    gc.collect()
    torch.cuda.empty_cache()
    return result


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=24)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--tol", type=float, default=3e-2, help="max |delta log-prob| on shared tokens")
    ap.add_argument("--parent", choices=("triton", "flash"), default="triton",
                    help="engine backend the non-decode calls are delegated to")
    ap.add_argument("--cudagraph", action="store_true",
                    help="let the engine capture decode batches into CUDA graphs: the counters then "
                         "count captures and warm-ups, not replays")
    args = ap.parse_args()

    from paged_decode_attention_b200 import vllm_backend

    prompts = _prompts(args.batch, 64, 160, CONFIG["vocab_size"])
    with tempfile.TemporaryDirectory() as d:
        (pathlib.Path(d) / "config.json").write_text(json.dumps(CONFIG))
        stock = _generate(d, "FLASH_ATTN" if args.parent == "flash" else "TRITON_ATTN", prompts, args.steps,
                          args.cudagraph)
        vllm_backend.install(parent=args.parent)
        for k in vllm_backend.STATS:
            vllm_backend.STATS[k] = 0
        vllm_backend.TIMING.update(enabled=True, delegated_events=[], decode_host_s=[])
        ours = _generate(d, "CUSTOM", prompts, args.steps, args.cudagraph)
    stats = dict(vllm_backend.STATS)
    import torch

    torch.cuda.synchronize()
    # delegated calls that carried tokens are the prefill attention of each layer
    prefill = [(e0.elapsed_time(e1), n) for e0, e1, n in vllm_backend.TIMING["delegated_events"] if n > 0]
    timing = {"parent": args.parent,
              "delegated_attention_ms_total": sum(ms for ms, _ in prefill),
              "delegated_attention_calls": len(prefill),
              "delegated_attention_tokens": sum(n for _, n in prefill),
              "decode_host_us_median": 1e6 * statistics.median(vllm_backend.TIMING["decode_host_s"] or [0.0]),
              "decode_host_us_first_calls_max": 1e6 * max(vllm_backend.TIMING["decode_host_s"] or [0.0]),
              "note": "device time of the parent's forward on prefill and mixed batches (CUDA events); host "
                      "wall time of one decode call of this library as the engine issues it (no device wait): "
                      "the median is the steady state, the maximum is a first call that prepares the "
                      "argument block and its scratch"}

    compared = same_tokens = total = 0
    worst = 0.0
    for (tok_a, lp_a), (tok_b, lp_b) in zip(stock, ours):
        for i in range(min(len(tok_a), len(tok_b))):
            total += 1
            if tok_a[:i] != tok_b[:i]:
                break  # the runs have left the common prefix: later steps see different inputs
            shared = set(lp_a[i]) & set(lp_b[i])
            for t in shared:
                worst = max(worst, abs(lp_a[i][t] - lp_b[i][t]))
            compared += 1
            same_tokens += tok_a[i] == tok_b[i]

    # every step after the first is a pure-decode batch; the first (prefill) is delegated
    expect_decode = LAYERS * (args.steps - 1)
    if args.cudagraph:  # a replayed graph does not pass through Python: only captures are counted
        served = stats["decode_calls"] >= LAYERS
    else:
        served = (stats["decode_calls"] >= expect_decode
                  and stats["decode_tokens"] >= expect_decode * args.batch)
    ok = served and compared >= args.batch * 2 and worst <= args.tol
    print(json.dumps({"check": "vllm_engine", "ok": bool(ok), "cudagraph": args.cudagraph, "stats": stats,
                      "expected_decode_calls": expect_decode, "steps_compared": compared,
                      "steps_total": total, "same_greedy_token": same_tokens,
                      "max_abs_logprob_delta": worst, "tol": args.tol, "timing": timing,
                      "model": "Qwen2-style random weights, 14/2 heads, head_dim 64, 4 layers"}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
