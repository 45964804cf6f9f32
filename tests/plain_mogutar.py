"""A plain, slow implementation of the Mogutar decoder: whole sequences, no cache, one function
for each mechanism, float64 on the CPU, loops over time where a recurrence says it most plainly.

It shares no code with the package under test: it reads config.json and model.safetensors
itself and states every mechanism from its definition (t: time, h: the sublayer's input).

  norm           n(y) = y / sqrt(mean(y^2) + eps) * w
  layer          x += n1(mixer(x));  x += n2(ff(x));  x += n_s(P_s (gelu_tanh(G_s x) * e_token[layer]))
  short conv     y_t = sum_j w[:, j] u_{t - taps + 1 + j}   (u = 0 before the sequence starts)
  attention      q, k, v = conv(W h + b); per head q, k <- n(q), n(k); partial rotary with stretched
                 frequencies; s_ij = cap * tanh((q_i . k_j) * scale / cap) for j <= i and
                 (i - j < window or j < keep_first); softmax; Wo
  state space    [z | x | B | C | dt] = W h; (x, B, C) <- silu(conv + bias); dt <- softplus(dt + dt_bias);
                 S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T;  y_t = S_t^T C_t + D x_t;
                 out = Wo (group_norm(y * silu(z)) * w)
  parallel       a * attention(h) + b * state_space(h)
  lightning      q, k, v = silu(W h); S_t = decay S_{t-1} + k_t v_t^T; o_t = S_t^T q_t;
                 out = Wo (n(concat o) * sigmoid(Wg h))
  experts        s = sigmoid(Wr h); choice = s + correction, limited to the best groups (a group's
                 score: its two largest choice scores); weights = s of the chosen, as they are
  output         head (n(x))
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


# --------------------------------------------------------------------------- small functions
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def short_conv(u: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u [T, C], w [C, taps]: the last column of w meets the current token."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y if bias is None else y + bias


# --------------------------------------------------------------------------- rotary positions
def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """Per pair i < dims/2 its angular frequency, and the factor on cos and sin."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: Sequence[int], dims: int, freqs: Sequence[float], mult: float) -> torch.Tensor:
    """x [T, heads, dim]: dimension i pairs with i + dims/2 among the first ``dims``; the rest pass."""
    out = x.clone()
    half = dims // 2
    for t, p in enumerate(positions):
        for i in range(half):
            a = p * freqs[i]
            c, s = math.cos(a) * mult, math.sin(a) * mult
            u, v = x[t, :, i], x[t, :, i + half]
            out[t, :, i] = u * c - v * s
            out[t, :, i + half] = v * c + u * s
    return out


# --------------------------------------------------------------------------- mixers
def visible(i: int, j: int, window: Optional[int], keep_first: int) -> bool:
    return j <= i and (window is None or i - j < window or j < keep_first)


def attend(q_i: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, i: int, window: Optional[int], keep_first: int,
           scale: float, cap: Optional[float]) -> torch.Tensor:
    """One query at position i over the keys [T, dim] and values [T, vdim] of its key/value head."""
    js = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
    s = (keys[js] @ q_i) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    return torch.softmax(s, dim=0) @ values[js]


def windowed_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, hd, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    if m.get("conv"):
        q, k, v = short_conv(q, w[p + "q.conv"]), short_conv(k, w[p + "k.conv"]), short_conv(v, w[p + "v.conv"])
    q = rms_norm(q.view(T, H, hd), w[p + "q.norm"], eps)
    k = rms_norm(k.view(T, G, hd), w[p + "k.norm"], eps)
    v = v.view(T, G, vd)
    rot = m.get("rot")
    if rot:
        freqs, mult = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q = rotate(q, range(T), rot["dims"], freqs, mult)
        k = rotate(k, range(T), rot["dims"], freqs, mult)
    mask = m.get("mask") or {}
    window, keep = mask.get("size"), mask.get("keep_first") or 0
    cap = m.get("softcap")
    out = torch.zeros(T, H, vd, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        for i in range(T):
            out[i, a] = attend(q[i, a], k[:, g], v[:, g], i, window, keep, m["scale"], cap)
    return out.reshape(T, H * vd) @ w[p + "o"].T


def state_space(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    Hn, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hn * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, Hn, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    rate = torch.exp(w[p + "A_log"])
    y = torch.zeros(T, Hn, P, dtype=F64)
    for a in range(Hn):
        g = a // (Hn // G)
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = torch.exp(-rate[a] * dt[t, a]) * S + dt[t, a] * torch.outer(B[t, g], x[t, a])
            y[t, a] = S.T @ C[t, g] + w[p + "D"][a] * x[t, a]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.view(T, parts, inner // parts), None, eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return m["left_scale"] * windowed_attention(h, w, p + "left.", m["left"], eps) \
        + m["right_scale"] * state_space(h, w, p + "right.", m["right"], eps)


def lightning_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, dk)
    k = silu(h @ w[p + "k"].T).view(T, H, dk)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = m["decay"][a] * S + torch.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    y = rms_norm(o.reshape(T, H * dv), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


# --------------------------------------------------------------------------- feed-forward
def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int, groups: Optional[dict]):
    """For one token: the chosen experts and their weights."""
    s = sigmoid(router @ h)
    choice = s + correction
    E = s.shape[0]
    allowed = [True] * E
    if groups and groups["count"] > 1 and groups["keep"] < groups["count"]:
        n, size = groups["count"], E // groups["count"]
        score = []
        for g in range(n):
            vals = sorted((float(choice[e]) for e in range(g * size, (g + 1) * size)), reverse=True)
            score.append(sum(vals[:2]))
        best = sorted(range(n), key=lambda g: (-score[g], g))[:groups["keep"]]
        allowed = [(e // size) in best for e in range(E)]
    order = sorted((e for e in range(E) if allowed[e]), key=lambda e: (-float(choice[e]), e))[:top]
    return order, [s[e] for e in order]


def experts_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        ids, ws = route(h[t], w[p + "router"], w[p + "correction"], r["top"], r.get("groups"))
        for e, we in zip(ids, ws):
            q = p + f"e{e}."
            out[t] += we * ((silu(w[q + "gate"] @ h[t]) * (w[q + "up"] @ h[t])) @ w[q + "down"].T)
    return out


def token_side(x: torch.Tensor, tokens: Sequence[int], w: Dict[str, torch.Tensor], layer: int, dim: int, eps: float) -> torch.Tensor:
    p = f"l{layer}.side."
    e = w["side.embed"][list(tokens)][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms_norm(y, w[p + "norm"], eps)


# --------------------------------------------------------------------------- the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], layer_outputs: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][list(tokens)]
    side = cfg.get("token_side")
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "parallel":
            y = parallel_mixer(x, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "lightning":
            y = lightning_mixer(x, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(experts_ff(x, w, p + "mlp.", layer["mlp"]), w[p + "norm2"], eps)
        if side:
            x = x + token_side(x, tokens, w, i, side["dim"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], new_tokens: int) -> List[int]:
    seq = list(prompt)
    out = []
    for _ in range(new_tokens):
        t = int(torch.argmax(forward(cfg, w, seq)[-1]))
        out.append(t)
        seq.append(t)
    return out
