"""Prompt and single-token throughput of the Mosurax and Mogutar designs beside the Llama decoder at equal layer sizes
(random bfloat16 weights, synthetic tokens): ``python bench.py --designs`` or
``python -m rustyllm_b200.bench_designs [--size NAME] [--steps K] [--warmup W]``.

For every size three models of the same width, heads, head size, feed-forward width (the experts that a token
uses together with the shared one are as wide as the dense feed-forward), vocabulary and depth:
  llama          grouped-query attention with rotary encoding, dense SwiGLU feed-forward
  mosurax-dense  learned positions, attention with a sink term and an output gate (one more projection of
                 heads x head size rows), dense feed-forward, soft-capped logits
  mosurax-moe    the same with every second layer's feed-forward a mixture of experts with a shared expert
  mogutar        post-norm layers, two in four with attention (convolved, normed, rotated q and k; soft-capped scores; a
                 window of 1,024 with 8 kept tokens) beside a selective state-space mixer of the model's width, two in
                 four with linear attention with decay; every feed-forward 16 experts in 4 groups (2 kept), 4 a token,
                 each a quarter of the dense width; a per-layer token input of 256 columns
``--kernels`` times the Mogutar design's own kernels alone at the sizes of a layer (a JSON line a kernel, with the
bytes it must move and their share of the measured copy bandwidth).
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


def mogutar_config(s: dict, window: int = 1024) -> dict:
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5, "conv": 4,
            "softcap": 30.0, "mask": {"size": window, "keep_first": 8},
            "rot": {"base": 1.0e6, "dims": s["dim"] // 2, "scaling": {"factor": 8.0, "original": 8192, "fast": 16.0, "slow": 2.0}}}
    right = {"heads": s["width"] // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8}
    mlp = {"kind": "moe", "router": {"experts": s["experts"], "top": 4, "groups": {"count": 4, "keep": 2}}, "expert": {"ff": s["expert_ff"]}}
    layers = []
    for i in range(s["layers"]):
        if i % 4 < 2:
            layers.append({"type": "parallel", "mixer": {"left": dict(left), "right": dict(right), "left_scale": 1.0, "right_scale": 1.0},
                           "mlp": dict(mlp)})
        else:
            layers.append({"type": "lightning", "mixer": {"heads": s["heads"], "dim": s["dim"], "vdim": s["dim"],
                                                           "decay": [1.0 - 2.0 ** -(5 + 4 * h / s["heads"]) for h in range(s["heads"])]},
                           "mlp": dict(mlp)})
    return {"architecture": "Mogutar", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5}, "token_side": {"dim": 256},
            "layers": layers}


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
        window: int = 0, models=("llama", "mosurax-dense", "mosurax-moe", "mogutar")) -> List[dict]:
    lines = []
    for name in sizes:
        s = SIZES[name]
        got = {}
        for model in models:
            cfg = llama_config(s) if model == "llama" else mogutar_config(s, window or 1024) if model == "mogutar" \
                else mosurax_config(s, model == "mosurax-moe", window or None)
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


def kernel_times(sizes: List[str], prompt: int = 2048, batch: int = 64, runs: int = 20) -> List[dict]:
    """The recurrent and fused kernels of the Mogutar design alone, bfloat16, at a layer's sizes: ``prompt`` tokens of
    one sequence, and one token of each of ``batch`` sequences.  Bytes: what the kernel must read and write once."""
    import json as _json
    import os
    import torch
    from . import kernels as K
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peaks = _json.load(f)
    except OSError:
        pass
    gbs = float(peaks.get("hbm_gbs", 6650.0))
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(runs):
            flush.zero_()                      # a buffer larger than L2 between runs
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2] * 1e3   # us

    lines = []

    def report(size, kernel, shape, us, nbytes):
        line = {"size": size, "kernel": kernel, "shape": shape, "us": round(us, 2), "gb": round(nbytes / 1e9, 4),
                "tb_s": round(nbytes / us / 1e6, 3), "of_copy_bandwidth": round(nbytes / us / 1e3 / gbs, 3)}
        print(_json.dumps(line), flush=True)
        lines.append(line)

    for name in sizes:
        s = SIZES[name]
        d, H, hd = s["width"], s["heads"], s["dim"]
        for what, M, B in (("prompt", prompt, 1), ("single tokens", batch, batch)):
            i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
            per = M // B
            cu, slots = i32([per * b for b in range(B + 1)]), i32(list(range(B)))
            slot_of_token = i32([b for b in range(B) for _ in range(per)])
            # linear attention with decay: heads of (hd, hd)
            state = torch.zeros((B, 4 * H * hd * hd), dtype=torch.uint8, device=dev)
            qkv = torch.randn((M, 3 * H * hd), dtype=torch.float32, device=dev).to(bf)
            o = torch.empty((M, H * hd), dtype=torch.float32, device=dev)
            decay = torch.full((H,), 0.99, dtype=torch.float32, device=dev)
            us = timed(lambda: K.linear_scan(qkv[:, :H * hd], qkv[:, H * hd:2 * H * hd], qkv[:, 2 * H * hd:], o, state, cu, slots, H, 1, hd, hd,
                                             decay, silu=True))
            report(name, "linear_scan (decay)", f"{what}: {M} tokens, {B} seq, {H} heads of {hd} x {hd}", us,
                   qkv.numel() * 2 + o.numel() * 4 + 2 * state.numel())
            # selective state space: width / 64 heads of (128, 64), 8 groups
            Hs, P, N, G = d // 64, 64, 128, 8
            state = torch.zeros((B, 4 * Hs * N * P), dtype=torch.uint8, device=dev)
            xbc = torch.randn((M, Hs * P + 2 * G * N), dtype=torch.float32, device=dev).to(bf)
            dt = torch.randn((M, Hs), dtype=torch.float32, device=dev).to(bf)
            y = torch.empty((M, Hs * P), dtype=torch.float32, device=dev)
            z32 = torch.zeros(Hs, dtype=torch.float32, device=dev)
            us = timed(lambda: K.linear_scan(xbc[:, Hs * P + G * N:], xbc[:, Hs * P:Hs * P + G * N], xbc[:, :Hs * P], y, state, cu, slots, Hs,
                                             Hs // G, N, P, z32, dt_raw=dt, dt_bias=z32, skip=z32))
            report(name, "linear_scan (selective)", f"{what}: {M} tokens, {B} seq, {Hs} heads of {N} x {P}", us,
                   xbc.numel() * 2 + dt.numel() * 2 + y.numel() * 4 + 2 * state.numel())
            # the convolution of x, B, C with its state
            C = Hs * P + 2 * G * N
            cstate = torch.zeros((B, 4 * 3 * C), dtype=torch.uint8, device=dev)
            w = torch.randn((C, 4), dtype=torch.float32, device=dev)
            out = torch.empty((M, C), dtype=bf, device=dev)
            us = timed(lambda: (K.short_conv(xbc, w, None, True, slot_of_token, cstate, out), K.short_conv_state(xbc, 4, cu, slots, cstate)))
            report(name, "short_conv + state", f"{what}: {M} tokens, {C} channels, 4 taps", us, 2 * xbc.numel() * 2 + 2 * cstate.numel())
            # the attention's preparation: convolution, head norms, rotation, cache write (keys and values to pages)
            G = s["kv_heads"]
            Cq = (H + 2 * G) * hd
            pstate = torch.zeros((B, 4 * 3 * Cq), dtype=torch.uint8, device=dev)
            u = torch.randn((M, Cq), dtype=torch.float32, device=dev).to(bf)
            qo = torch.empty((M, H * hd), dtype=bf, device=dev)
            pages = -(-per // K.PAGE_SIZE)
            k_pool = torch.zeros((B * pages, G, K.PAGE_SIZE, hd), dtype=bf, device=dev)
            v_pool = torch.zeros_like(k_pool)
            table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages)
            positions = i32([t for b in range(B) for t in range(per)])
            wq = torch.randn((Cq, 4), dtype=torch.float32, device=dev)
            nw = torch.ones(hd, dtype=torch.float32, device=dev)
            inv = torch.rand(hd // 4, dtype=torch.float32, device=dev)
            us = timed(lambda: (K.qkv_prepare(u, qo, wq, pstate, nw, nw, 1e-5, positions, slot_of_token, table, inv, hd // 2, 1.1, H, G, hd, hd,
                                              k_pool, v_pool), K.short_conv_state(u, 4, cu, slots, pstate)))
            report(name, "qkv_prepare + state", f"{what}: {M} tokens, {H} + 2 x {G} heads of {hd}, 4 taps", us, 2 * u.numel() * 2 + 2 * pstate.numel())
            # gate, norm in groups
            yn = torch.empty((M, Hs * P), dtype=bf, device=dev)
            gate = torch.randn((M, Hs * P), dtype=torch.float32, device=dev).to(bf)
            wn = torch.ones(Hs * P, dtype=torch.float32, device=dev)
            us = timed(lambda: K.gated_norm(y, gate, wn, 1e-5, yn, groups=8))
            report(name, "gated_norm", f"{what}: {M} x {Hs * P}", us, y.numel() * 4 + 2 * gate.numel() * 2)
            # x += norm(y0 + y1) * w, with the bfloat16 copy
            x = torch.randn((M, d), dtype=torch.float32, device=dev)
            y0, y1 = torch.randn_like(x), torch.randn_like(x)
            xb = torch.empty((M, d), dtype=bf, device=dev)
            wd = torch.ones(d, dtype=torch.float32, device=dev)
            us = timed(lambda: K.norm_add(x, y0, 1.0, y1, 1.0, wd, 1e-5, xb))
            report(name, "norm_add (two terms)", f"{what}: {M} x {d}", us, 4 * x.numel() * 4 + xb.numel() * 2)
    K.check_device_errors()
    return lines


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--size", action="append", choices=sorted(SIZES), help="default: all")
    ap.add_argument("--model", action="append", choices=["llama", "mosurax-dense", "mosurax-moe", "mogutar"], help="default: all four")
    ap.add_argument("--kernels", action="store_true", help="time the Mogutar design's own kernels alone instead")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--batch", type=int, action="append", help="default: 8 and 64")
    ap.add_argument("--window", type=int, default=0, help="sliding window of the Mosurax layers (0: none, as Llama)")
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=8)
    a = ap.parse_args(argv)
    if a.kernels:
        kernel_times(a.size or sorted(SIZES), a.prompt, max(a.batch or (64,)))
        return 0
    run(a.size or sorted(SIZES), a.prompt, tuple(a.batch or (8, 64)), a.context, a.steps, a.warmup, a.window,
        tuple(a.model or ("llama", "mosurax-dense", "mosurax-moe", "mogutar")))
    return 0


if __name__ == "__main__":
    sys.exit(main())
