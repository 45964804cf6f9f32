"""Small Mosurax configurations for tests, and a writer of random weights for them.

The configurations differ from one another in every size and option: heads and groups (one KV
head, as many KV heads as heads), key heads narrower and wider than value heads, windows of 1, of
less than a page, across page borders and none, dense / expert / absent feed-forwards, experts with
top = 1 and top = all, with and without a shared expert, loops over the first, the middle and all
layers with 1 to 3 passes and no loop, with and without a soft cap.

Weights are drawn so that faults show: queries and keys large enough that attention is far from
uniform (scores of standard deviation 1.5), router logits of standard deviation 1 with a bias,
logits of standard deviation 3 under the soft cap.  They are stored in bfloat16, so a 32-bit run
and a bfloat16 run compute on the same numbers.
"""
import json
import math
import os

import torch

from rustyllm_b200.weights.safetensors_io import write_safetensors


def attn(heads, kv_heads, dim, vdim, scale, window):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


CONFIGS = {
    # value heads wider than key heads, a window shorter than a page, every kind of feed-forward,
    # the two middle layers three times
    "P": {"architecture": "Mosurax", "vocab": 97, "width": 64, "max_positions": 320, "norm": {"eps": 1e-5},
          "logit_softcap": 7.0, "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [layer(attn(4, 2, 16, 24, 0.3, 9), dense(40)),
                     layer(attn(4, 2, 16, 24, 0.3, 9), moe(5, 2, 24, shared=32)),
                     layer(attn(4, 2, 16, 24, 0.3, 9), None),
                     layer(attn(4, 2, 16, 24, 0.3, 9), moe(3, 3, 16))]},
    # head size 64 for keys and values (the tensor-core attention's shape), one KV head, windows that
    # differ by layer: across a page border, none, across two; no loop, no soft cap, top = 1
    "Q": {"architecture": "Mosurax", "vocab": 211, "width": 128, "max_positions": 448, "norm": {"eps": 1e-6},
          "layers": [layer(attn(4, 1, 64, 64, 0.11, 70), dense(96)),
                     layer(attn(4, 1, 64, 64, 0.11, None), moe(4, 1, 48, shared=64)),
                     layer(attn(4, 1, 64, 64, 0.11, 130), dense(96))]},
    # head size 128, as many KV heads as heads, all layers looped once (one pass: only the pass's vector)
    "R": {"architecture": "Mosurax", "vocab": 130, "width": 256, "max_positions": 400, "norm": {"eps": 1e-5},
          "logit_softcap": 30.0, "loop": {"start": 0, "stop": 2, "times": 1},
          "layers": [layer(attn(2, 2, 128, 128, 0.07, 200), moe(6, 2, 64, shared=32)),
                     layer(attn(2, 2, 128, 128, 0.07, 65), dense(128))]},
    # a width that is no multiple of 64, value heads narrower than key heads, windows of 1 and 2,
    # the first layer twice, an odd vocabulary
    "S": {"architecture": "Mosurax", "vocab": 53, "width": 48, "max_positions": 200, "norm": {"eps": 1e-6},
          "logit_softcap": 4.0, "loop": {"start": 0, "stop": 1, "times": 2},
          "layers": [layer(attn(6, 3, 32, 8, 0.2, 1), dense(72)),
                     layer(attn(6, 3, 32, 8, 0.2, 2), moe(7, 3, 8, shared=8)),
                     layer(attn(3, 3, 16, 16, 0.25, 64), None)]},
}


def tensor_shapes(cfg):
    d = cfg["width"]
    out = {"embed": (cfg["vocab"], d), "pos": (cfg["max_positions"], d), "final.norm": (d,), "head": (cfg["vocab"], d)}
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], d)
    for i, l in enumerate(cfg["layers"]):
        m, p = l["mixer"], f"l{i}."
        out[p + "norm1"] = (d,)
        out[p + "mix.q"] = (m["heads"] * m["dim"], d)
        out[p + "mix.k"] = (m["kv_heads"] * m["dim"], d)
        out[p + "mix.v"] = (m["kv_heads"] * m["vdim"], d)
        out[p + "mix.g"] = (m["heads"] * m["vdim"], d)
        out[p + "mix.o"] = (d, m["heads"] * m["vdim"])
        mlp = l["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = (d,)

        def ff(prefix, f):
            out[prefix + "gate"], out[prefix + "up"], out[prefix + "down"] = (f, d), (f, d), (d, f)
        if mlp["kind"] == "dense":
            ff(p + "mlp.", mlp["ff"])
        else:
            E = mlp["router"]["experts"]
            out[p + "mlp.router"], out[p + "mlp.router.b"] = (E, d), (E,)
            for e in range(E):
                ff(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
            if mlp.get("shared"):
                ff(p + "mlp.shared.", mlp["shared"]["ff"])
    return out


def draw_weights(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        z = torch.randn(shape, generator=g, dtype=torch.float32)
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.1 * z
        elif name == "embed":
            t = z
        elif name in ("pos", "loop.step"):
            t = 0.5 * z
        elif name == "head":
            t = 3.0 * z / math.sqrt(d)
        elif leaf in ("q", "k"):
            m = cfg["layers"][int(name.split(".")[0][1:])]["mixer"]
            a = math.sqrt(1.5 / (m["scale"] * math.sqrt(m["dim"])))     # scores of standard deviation 1.5
            t = a * z / math.sqrt(d)
        elif leaf == "b":
            t = 0.5 * z
        elif leaf in ("o", "down"):
            t = 0.5 * z / math.sqrt(shape[1])
        else:
            t = z / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16)
    return out


def random_config(seed):
    """A configuration with every size drawn at random: widths that are no multiple of 8 or 64, 1 to 8 heads
    over any divisor of KV heads, key and value heads of 8 to 128 (equal or not), any window, 1 to 4 layers of
    any feed-forward, any loop."""
    import random
    rng = random.Random(seed)
    width = rng.choice([24, 40, 56, 72, 100, 136, 192, 204])
    n = rng.randrange(1, 5)
    layers = []
    for _ in range(n):
        heads = rng.choice([1, 2, 3, 4, 6, 8])
        kv = rng.choice([g for g in range(1, heads + 1) if heads % g == 0])
        dim = rng.choice([8, 16, 18, 24, 32, 48, 64, 64, 128, 128])
        vdim = dim if rng.random() < 0.6 else rng.choice([8, 16, 20, 32, 64, 128])
        window = rng.choice([None, 1, 2, 5, 33, 63, 64, 65, 100, 129, 1000])
        kind = rng.choice(["dense", "moe", "moe", None])
        if kind == "dense":
            mlp = dense(rng.choice([8, 20, 64, 100, 136]))
        elif kind == "moe":
            E = rng.randrange(1, 10)
            mlp = moe(E, rng.randrange(1, E + 1), rng.choice([8, 12, 16, 40, 64]), shared=rng.choice([None, 8, 24, 64]))
        else:
            mlp = None
        layers.append(layer(attn(heads, kv, dim, vdim, rng.choice([0.05, 0.125, 0.3, 1.0 / math.sqrt(dim)]), window), mlp))
    cfg = {"architecture": "Mosurax", "vocab": rng.choice([17, 64, 101, 300]), "width": width, "max_positions": 260,
           "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "layers": layers}
    if rng.random() < 0.7:
        cfg["logit_softcap"] = rng.choice([2.0, 10.0, 50.0])
    if rng.random() < 0.7:
        a = rng.randrange(0, n)
        cfg["loop"] = {"start": a, "stop": rng.randrange(a + 1, n + 1), "times": rng.randrange(1, 4)}
    return cfg


def write_model(name, path, seed=None, cfg=None):
    cfg = cfg or CONFIGS[name]
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), draw_weights(cfg, seed if seed is not None else sum(map(ord, name))))
    return path
