"""A plain, slow implementation of the Mosurax decoder: whole sequences, no cache, one function
for each mechanism, float64 on the CPU, loops where a loop says it most plainly.

It shares no code with the package under test: it reads config.json and model.safetensors
itself and states every mechanism from its definition:

  embedding      x_t = E[token_t] + P[t]
  norm           y = x / sqrt(mean(x^2) + eps) * w
  attention      q, k, v = Wq h, Wk h, Wv h; query head a reads key/value head a // (H / G);
                 s_ij = (q_i . k_j) * scale for 0 <= i - j < window (all j <= i without a window);
                 p_ij = exp(s_ij) / (1 + sum_j exp(s_ij));  o_i = sum_j p_ij v_j;
                 out = Wo (concat(o) * sigmoid(Wg h))
  dense ff       Wdown (silu(Wgate h) * (Wup h))
  experts        z = Wr h + b; the `top` largest z chosen; weights = softmax over the chosen z;
                 sum of the chosen experts' outputs by weight, plus the shared expert's
  layer          x += attention(norm1(x)); x += ff(norm2(x))   (no second half without a feed-forward)
  loop           layers start .. stop - 1 run `times` times; before pass t > 0: x += embedding output;
                 before every pass: x += step[t]
  output         head (norm(x)), then cap * tanh(logits / cap)
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    dt = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
          "I32": torch.int32, "I64": torch.int64}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[b:e]), dtype=dt[info["dtype"]]).reshape(info["shape"]).clone()
    return out


def load_model_dir(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: v.to(F64) for k, v in w.items()}


# --------------------------------------------------------------------------- mechanisms
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def embed(tokens: Sequence[int], table: torch.Tensor, positions: torch.Tensor, first_position: int = 0) -> torch.Tensor:
    return torch.stack([table[t] + positions[first_position + i] for i, t in enumerate(tokens)])


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def gated_ff(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def sink_softmax(scores: Sequence[float]) -> List[float]:
    """p_j = exp(s_j) / (1 + sum exp(s_j)): the sum of the p_j is below 1."""
    m = max(0.0, max(scores))
    e = [math.exp(s - m) for s in scores]
    denom = math.exp(-m) + sum(e)
    return [v / denom for v in e]


def windowed_sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                            window: Optional[int], sink: bool = True) -> torch.Tensor:
    """q [n, H, hd], k [n, G, hd], v [n, G, vd] of one sequence from its first token -> [n, H, vd]."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for i in range(n):
        lo = 0 if window is None else max(0, i - window + 1)
        for a in range(H):
            g = a // (H // G)
            s = (k[lo:i + 1, g] @ q[i, a]) * scale               # the scores of keys lo .. i
            m = max(0.0, float(s.max())) if sink else float(s.max())
            e = torch.exp(s - m)
            denom = e.sum() + (math.exp(-m) if sink else 0.0)    # the sink: one more term, exp(0 - m)
            out[i, a] = (e / denom) @ v[lo:i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, m: dict) -> torch.Tensor:
    n = h.shape[0]
    H, G, hd, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + ".q"].T).view(n, H, hd)
    k = (h @ w[prefix + ".k"].T).view(n, G, hd)
    v = (h @ w[prefix + ".v"].T).view(n, G, vd)
    window = m["mask"]["size"] if m.get("mask") else None
    o = windowed_sink_attention(q, k, v, m["scale"], window).reshape(n, H * vd)
    gate = 1.0 / (1.0 + torch.exp(-(h @ w[prefix + ".g"].T)))
    return (o * gate) @ w[prefix + ".o"].T


def route(z: torch.Tensor, top: int):
    """One token's logits -> (chosen experts by falling logit, their weights)."""
    order = sorted(range(z.numel()), key=lambda e: (-float(z[e]), e))[:top]
    m = float(z[order[0]])
    e = [math.exp(float(z[i]) - m) for i in order]
    return order, [x / sum(e) for x in e]


def experts_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, mlp: dict) -> torch.Tensor:
    out = torch.zeros(h.shape[0], w[prefix + ".e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        z = w[prefix + ".router"] @ h[t] + w[prefix + ".router.b"]
        chosen, weights = route(z, mlp["router"]["top"])
        for e, we in zip(chosen, weights):
            p = f"{prefix}.e{e}"
            out[t] += we * gated_ff(h[t:t + 1], w[p + ".gate"], w[p + ".up"], w[p + ".down"])[0]
    if mlp.get("shared"):
        p = prefix + ".shared"
        out += gated_ff(h, w[p + ".gate"], w[p + ".up"], w[p + ".down"])
    return out


def layer(x: torch.Tensor, cfg: dict, w: Dict[str, torch.Tensor], i: int) -> torch.Tensor:
    l, eps = cfg["layers"][i], cfg["norm"]["eps"]
    x = x + attention_mixer(rms_norm(x, w[f"l{i}.norm1"], eps), w, f"l{i}.mix", l["mixer"])
    mlp = l.get("mlp")
    if mlp is not None:
        h = rms_norm(x, w[f"l{i}.norm2"], eps)
        if mlp["kind"] == "dense":
            x = x + gated_ff(h, w[f"l{i}.mlp.gate"], w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"])
        else:
            x = x + experts_ff(h, w, f"l{i}.mlp", mlp)
    return x


def soft_cap(logits: torch.Tensor, cap: Optional[float]) -> torch.Tensor:
    return logits if cap is None else cap * torch.tanh(logits / cap)


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], residuals: Optional[list] = None) -> torch.Tensor:
    """float64 logits [len(tokens), vocab]; ``residuals`` collects the stream after every layer run."""
    x = embed(tokens, w["embed"], w["pos"])
    x0 = x.clone()
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    runs: List[object] = list(range(n))
    if loop:
        runs = list(range(loop["start"]))
        for t in range(loop["times"]):
            runs.append(("pass", t))
            runs += list(range(loop["start"], loop["stop"]))
        runs += list(range(loop["stop"], n))
    for r in runs:
        if isinstance(r, tuple):
            if r[1] > 0:
                x = x + x0
            x = x + w["loop.step"][r[1]]
        else:
            x = layer(x, cfg, w, r)
            if residuals is not None:
                residuals.append(x.clone())
    logits = rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T
    return soft_cap(logits, cfg.get("logit_softcap"))


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], new_tokens: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(new_tokens):
        t = int(forward(cfg, w, toks)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out
