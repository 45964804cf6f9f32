"""Prompt and single-token throughput of the Mosurax design beside the Llama decoder at equal layer sizes
(random bfloat16 weights, synthetic tokens): ``python bench.py --designs`` or
``python -m rustyllm_b200.bench_designs [--size NAME] [--steps K] [--warmup W]``.

For every size three models of the same width, heads, head size, feed-forward width (the experts that a token
uses together with the shared one are as wide as the dense feed-forward), vocabulary and depth:
  llama          grouped-query attention with rotary encoding, dense SwiGLU feed-forward
  mosurax-dense  learned positions, attention with a sink term and an output gate (one more projection of
                 heads x head size rows), dense feed-forward, soft-capped logits
  mosurax-moe    the same with every second layer's feed-forward a mixture of experts with a shared expert
Measured with CUDA events after warm-up: one prompt of ``prompt`` tokens as one step; then single-token steps of
``batch`` sequences that hold ``context`` tokens each (the captured step, as generation runs it).  One JSON line
a model and a summary line a size.  Weights of a size exceed the L2 cache; the prompt's activations do too.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List

SIZES = {
    # width 2,048: 16 heads over 4 KV heads of 128, feed-forward 8,192, 8 layers
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, layers=8, vocab=32768,
                  experts=16, top=3, expert_ff=2048, shared_ff=2048),
    # width 4,096: the layer of an 8B model (32 heads over 8 KV heads of 128, feed-forward 14,336), 4 layers
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, layers=4, vocab=32768,
                  experts=16, top=3, expert_ff=3584, shared_ff=3584),
}
MAX_POSITIONS = 4096


def llama_config(s: dict) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": s["vocab"], "hidden_size": s["width"],
            "intermediate_size": s["ff"], "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"],
            "num_key_value_heads": s["kv_heads"], "head_dim": s["dim"], "max_position_embeddings": MAX_POSITIONS,
            "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": False}


def mosurax_config(s: dict, experts: bool, window=None) -> dict:
    mixer = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5}
    if window:
        mixer["mask"] = {"size": window}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"]},
           "shared": {"ff": s["shared_ff"]}}
    layers = [{"type": "attention", "mixer": dict(mixer), "mlp": moe if (experts and i % 2) else dense} for i in range(s["layers"])]
    return {"architecture": "Mosurax", "vocab": s["vocab"], "width": s["width"], "max_positions": MAX_POSITIONS,
            "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": layers}


def measure(config: dict, prompt: int, batches: List[int], context: int, steps: int, warmup: int) -> Dict[str, float]:
    import numpy as np
    import torch
    from . import Runner
    max_b = max(batches)
    runner = Runner.from_config(config, seed=0, dtype="bfloat16", device="cuda:0",
                                max_cache_tokens=max(max_b * (context + 64 + steps + warmup), prompt + 64), max_batch=max_b,
                                max_context=MAX_POSITIONS)
    eng = runner.engine
    rng = np.random.default_rng(0)
    V = runner.model.spec.vocab_size
    out: Dict[str, float] = {"parameter_gb": round(runner.model.parameter_bytes() / 1e9, 3)}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # ---- one prompt as one step ----
    times = []
    for i in range(3 + 3):
        s = eng.alloc_slot()
        toks = rng.integers(0, V, size=prompt).tolist()
        e0.record()
        eng.step([s], [toks], "last")
        e1.record()
        torch.cuda.synchronize()
        eng.free_slot(s)
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    out["prefill_ms"] = round(min(times), 3)
    out["prefill_tok_s"] = round(prompt * 1000.0 / min(times), 1)
    # ---- single-token steps ----
    for B in batches:
        slots = [eng.alloc_slot() for _ in range(B)]
        for s in slots:
            eng.step([s], [rng.integers(0, V, size=context).tolist()], None)
        toks = [[int(t)] for t in rng.integers(0, V, size=B)]
        for _ in range(max(warmup, 3)):
            eng.step(slots, toks, "last")
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            eng.step(slots, toks, "last")
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out[f"decode_b{B}_ms"] = round(ms, 4)
        out[f"decode_b{B}_tok_s"] = round(B * 1000.0 / ms, 1)
        for s in slots:
            eng.free_slot(s)
    from . import kernels
    kernels.check_device_errors()
    del runner, eng
    torch.cuda.empty_cache()
    return out


def run(sizes: List[str], prompt: int = 2048, batches=(8, 64), context: int = 1024, steps: int = 32, warmup: int = 8,
        window: int = 0, models=("llama", "mosurax-dense", "mosurax-moe")) -> List[dict]:
    lines = []
    for name in sizes:
        s = SIZES[name]
        got = {}
        for model in models:
            cfg = llama_config(s) if model == "llama" else mosurax_config(s, model == "mosurax-moe", window or None)
            got[model] = measure(cfg, prompt, list(batches), context, steps, warmup)
            line = {"size": name, "model": model, "prompt_tokens": prompt, "context": context, "window": window or None,
                    "dtype": "bf16", "data": "synthetic", **got[model]}
            print(json.dumps(line), flush=True)
            lines.append(line)
        if "llama" in got:
            for model in models:
                if model == "llama":
                    continue
                ratio = {k: round(got[model][k] / got["llama"][k], 3) for k in got[model] if k.endswith("tok_s")}
                line = {"size": name, "model": model, "throughput_over_llama": ratio}
                print(json.dumps(line), flush=True)
                lines.append(line)
    return lines


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--size", action="append", choices=sorted(SIZES), help="default: all")
    ap.add_argument("--model", action="append", choices=["llama", "mosurax-dense", "mosurax-moe"], help="default: all three")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--batch", type=int, action="append", help="default: 8 and 64")
    ap.add_argument("--window", type=int, default=0, help="sliding window of the Mosurax layers (0: none, as Llama)")
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=8)
    a = ap.parse_args(argv)
    run(a.size or sorted(SIZES), a.prompt, tuple(a.batch or (8, 64)), a.context, a.steps, a.warmup, a.window,
        tuple(a.model or ("llama", "mosurax-dense", "mosurax-moe")))
    return 0


if __name__ == "__main__":
    sys.exit(main())
