"""Small Mogutar configurations for tests, and a writer of random weights for them.

The configurations differ from one another in every size and option: heads over one, some and as many key/value
heads; key heads narrower than, wider than and equal to value heads; convolutions of 1 to 4 taps and none;
rotation of a part of a head, of all of it and none, with and without stretched frequencies; windows shorter than
a page, across page borders and none, with 0 to 5 kept first tokens; soft caps small enough to bend the scores and
none; state-space layers with one group and several, norm groups of 1 and more; lightning layers whose decays reach
from 0.5 to 0.999; experts in groups (keep some, keep all, no groups), top = 1 and top = all, layers without a
feed-forward; with and without the per-layer token input.

Weights are drawn so that faults show: query and key norm weights large enough that attention is far from uniform,
router logits of standard deviation 1.5 with corrections that change the choice, step sizes and decay rates that
make the state forget within tens of tokens in some heads and within thousands in others.  They are stored in
bfloat16, so a 32-bit run and a bfloat16 run compute on the same numbers.

``calm_router=True`` draws the routers so that no choice hinges on rounding: logits of standard deviation 0.05 to 0.2 and
corrections 0.4 apart (the groups' scores too), so the same experts are chosen for every token (their weights still differ from
token to token).  The bfloat16 runs of the engine tests use it: in this design a sublayer's output is normed to unit
size before it joins the stream and recurrent states carry every token's output to all later ones, so a single
close call that falls the other way after rounding changes the rest of the sequence by far more than rounding.
The 32-bit runs keep the lively router, and the router's kernels are tested on lively inputs by themselves.

The per-layer token input norms a vector of ``token_side.dim`` gated components; where all of them lie deep in the
negative tail of the gelu (1 + tanh(...) cancels) its direction is lost to rounding in any 32-bit arithmetic, so the
test configurations keep that width at 8 or more and the gate's input near unit size.
"""
import json
import math
import os

import torch

from rustyllm_b200.weights.safetensors_io import write_safetensors


def left(heads, kv_heads, dim, vdim, scale, conv=0, softcap=None, window=None, keep_first=0, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if rot is not None:
        m["rot"] = rot
    return m


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def parallel(l, r, ls, rs, mlp):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def moe(experts, top, ff, groups=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": r, "expert": {"ff": ff}}


CONFIGS = {
    # value heads wider than key heads (the any-shape attention), a window shorter than a page with two kept tokens, a
    # small soft cap, a quarter of the head rotated with stretched frequencies; a lightning layer without a feed-forward
    "T": {"architecture": "Mogutar", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8},
          "layers": [parallel(left(4, 2, 16, 24, 0.3, conv=3, softcap=4.0, window=9, keep_first=2, rot=rot(8, 10000.0, (2.0, 64, 8.0, 1.0))),
                              right(3, 8, 16, 1, 2, 1), 1.3, 0.7, moe(6, 2, 24, groups=(3, 2))),
                     lightning(2, 16, 8, [0.5, 0.97], None),
                     parallel(left(2, 2, 32, 32, 0.2, conv=2, window=70, keep_first=5, rot=rot(32, 500.0)),
                              right(4, 16, 8, 2, 4, 2), 0.8, 1.1, moe(4, 1, 16))]},
    # key and value heads of 64 (a tensor-core attention shape), one key/value head, windows across one and two page
    # borders and none, no token input, four taps, experts with all groups kept and with top = all
    "U": {"architecture": "Mogutar", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
          "layers": [parallel(left(4, 1, 64, 64, 0.125, conv=4, softcap=30.0, window=130, keep_first=3, rot=rot(16, 1.0e6, (8.0, 128, 16.0, 2.0))),
                              right(2, 32, 24, 2, 4, 2), 1.0, 1.0, moe(8, 2, 32, groups=(4, 4))),
                     lightning(4, 32, 16, [0.6, 0.9, 0.99, 0.999], moe(3, 3, 24)),
                     parallel(left(2, 1, 64, 64, 0.11, conv=4, window=None, rot=rot(64, 10000.0)),
                              right(8, 8, 32, 4, 3, 1), 1.1, 0.8, None),
                     parallel(left(4, 2, 64, 64, 0.125, conv=4, softcap=8.0, window=65, keep_first=0, rot=rot(32, 50000.0, (4.0, 256, 24.0, 1.0))),
                              right(2, 32, 24, 1, 4, 2), 0.5, 1.5, moe(6, 3, 16, groups=(2, 1)))]},
    # a width that is no multiple of 64, an odd vocabulary, value heads narrower than key heads, one tap (a gain a
    # channel) and no convolution, no rotation, a window of 1 and of 2, lightning layers first
    "W": {"architecture": "Mogutar", "vocab": 53, "width": 48, "norm": {"eps": 1e-6}, "token_side": {"dim": 12},
          "layers": [lightning(3, 24, 12, [0.7, 0.95, 0.995], moe(5, 5, 8)),
                     parallel(left(6, 3, 32, 8, 0.18, conv=1, window=1, keep_first=1), right(1, 24, 12, 1, 1, 3), 1.0, 0.6, moe(9, 2, 8, groups=(3, 1))),
                     parallel(left(3, 3, 16, 16, 0.25, softcap=2.0, window=2, keep_first=4, rot=rot(4, 100.0)), right(6, 4, 40, 3, 4, 1), 0.9, 1.0, None),
                     lightning(1, 40, 48, [0.9], moe(2, 1, 16))]},
}


def tensor_shapes(cfg):
    d, V, n = cfg["width"], cfg["vocab"], len(cfg["layers"])
    out = {"embed": (V, d), "final.norm": (d,), "head": (V, d)}
    side = cfg.get("token_side")
    if side:
        out["side.embed"] = (V, n * side["dim"])
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        out[p + "norm1"] = (d,)
        if l["type"] == "parallel":
            a, s = m["left"], m["right"]
            q = p + "mix.left."
            for name, rows in (("q", a["heads"] * a["dim"]), ("k", a["kv_heads"] * a["dim"]), ("v", a["kv_heads"] * a["vdim"])):
                out[q + name], out[q + name + ".b"] = (rows, d), (rows,)
                if a.get("conv"):
                    out[q + name + ".conv"] = (rows, a["conv"])
            out[q + "q.norm"], out[q + "k.norm"] = (a["dim"],), (a["dim"],)
            out[q + "o"] = (d, a["heads"] * a["vdim"])
            r = p + "mix.right."
            inner, gn = s["heads"] * s["vdim"], s["groups"] * s["state"]
            out[r + "in"] = (2 * inner + 2 * gn + s["heads"], d)
            out[r + "conv"], out[r + "conv.b"] = (inner + 2 * gn, s["conv"]), (inner + 2 * gn,)
            out[r + "dt_bias"] = out[r + "A_log"] = out[r + "D"] = (s["heads"],)
            out[r + "norm"], out[r + "o"] = (inner,), (d, inner)
        else:
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            q = p + "mix."
            out[q + "q"], out[q + "k"], out[q + "v"], out[q + "g"] = (H * dk, d), (H * dk, d), (H * dv, d), (H * dv, d)
            out[q + "o"], out[q + "norm"] = (d, H * dv), (H * dv,)
        mlp = l["mlp"]
        if mlp is not None:
            out[p + "norm2"] = (d,)
            E, f = mlp["router"]["experts"], mlp["expert"]["ff"]
            out[p + "mlp.router"], out[p + "mlp.correction"] = (E, d), (E,)
            for e in range(E):
                out[f"{p}mlp.e{e}.gate"], out[f"{p}mlp.e{e}.up"], out[f"{p}mlp.e{e}.down"] = (f, d), (f, d), (d, f)
        if side:
            out[p + "side.gate"], out[p + "side.proj"], out[p + "side.norm"] = (side["dim"], d), (d, side["dim"]), (d,)
    return out


def calm_corrections(router, g):
    """Corrections that settle the choice whatever the token: 0.4 apart (scores stay within 0.5 +- 0.06 with the calm
    router's logits, the stream's size growing with depth included), and the groups' scores - the sum of a
    group's two largest - at least 0.4 apart too."""
    E, groups = router["experts"], (router.get("groups") or {}).get("count", 1)
    size = E // groups
    while True:
        t = 0.4 * torch.randperm(E, generator=g).float() + 0.04 * (torch.rand(E, generator=g) - 0.5) - 1.0
        sums = sorted(float(t[i * size:(i + 1) * size].topk(min(2, size)).values.sum()) for i in range(groups))
        if all(b - a >= 0.4 for a, b in zip(sums, sums[1:])):
            return t


def draw_weights(cfg, seed, calm_router=False):
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        z = torch.randn(shape, generator=g, dtype=torch.float32)
        leaf = name.split(".")[-1]
        two = ".".join(name.split(".")[-2:])
        if leaf in ("norm1", "norm2") or name == "final.norm" or two in ("side.norm", "right.norm", "mix.norm"):
            t = 1.0 + 0.1 * z
        elif two in ("q.norm", "k.norm"):
            a = cfg["layers"][int(name.split(".")[0][1:])]["mixer"]["left"]
            t = (1.0 + 0.1 * z) * math.sqrt(1.6 / (a["scale"] * math.sqrt(a["dim"])))     # scores of standard deviation 1.6
        elif name in ("embed", "side.embed"):
            t = z
        elif name == "head":
            t = 3.0 * z / math.sqrt(d)
        elif leaf == "conv":
            t = 0.6 * z
        elif leaf == "b":
            t = 0.3 * z
        elif leaf == "dt_bias":
            t = -1.0 + 1.5 * z
        elif leaf == "A_log":
            t = -1.0 + 1.2 * z
        elif leaf == "D":
            t = 1.0 + 0.3 * z
        elif leaf == "router":
            t = (0.05 if calm_router else 1.5) * z / math.sqrt(d)
        elif leaf == "correction":
            t = calm_corrections(cfg["layers"][int(name.split(".")[0][1:])]["mlp"]["router"], g) if calm_router else 0.3 * z
        elif two == "side.gate":
            t = z / (3.0 * math.sqrt(d))
        elif leaf in ("o", "down", "proj"):
            t = 0.7 * z / math.sqrt(shape[1])
        else:
            t = z / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16)
    return out


def random_config(seed):
    """A configuration with every size drawn at random."""
    import random
    rng = random.Random(seed)
    width = rng.choice([24, 40, 56, 72, 100, 136, 192])
    n = rng.randrange(1, 5)
    layers = []

    def some_mlp():
        if rng.random() < 0.25:
            return None
        count = rng.choice([1, 1, 2, 3, 4])
        size = rng.randrange(1, 4)
        keep = rng.randrange(1, count + 1)
        top = rng.randrange(1, keep * size + 1)
        return moe(count * size, top, rng.choice([8, 12, 16, 40]), groups=None if count == 1 and rng.random() < 0.5 else (count, keep))
    for _ in range(n):
        if rng.random() < 0.6:
            heads = rng.choice([1, 2, 3, 4, 6])
            kv = rng.choice([g for g in range(1, heads + 1) if heads % g == 0])
            dim = rng.choice([8, 16, 18, 24, 32, 48, 64, 128])
            vdim = dim if rng.random() < 0.5 else rng.choice([8, 16, 20, 32, 64])
            window = rng.choice([None, 1, 2, 5, 33, 63, 64, 65, 100, 129])
            r = None
            if rng.random() < 0.8:
                dims = rng.choice([x for x in (2, 4, 8, 16, dim) if x <= dim and x % 2 == 0])
                r = rot(dims, rng.choice([100.0, 10000.0, 200000.0]),
                        rng.choice([None, (2.0, 64, 8.0, 1.0), (4.0, 512, 24.0, 1.0), (16.0, 100, 4.0, 0.5)]))
            l = left(heads, kv, dim, vdim, rng.choice([0.05, 0.125, 0.3, 1.0 / math.sqrt(dim)]), conv=rng.choice([0, 1, 2, 3, 4]),
                     softcap=rng.choice([None, 1.5, 10.0, 40.0]), window=window, keep_first=rng.choice([0, 1, 3, 7, 64, 70]), rot=r)
            sh = rng.choice([1, 2, 3, 4, 8])
            sg = rng.choice([g for g in range(1, sh + 1) if sh % g == 0])
            sp = rng.choice([8, 12, 16, 32])
            ng = rng.choice([g for g in (1, 2, 3, 4) if (sh * sp) % g == 0 and (g == 1 or sh * sp // g >= 24)])   # a norm over a dozen values turns rounding into direction
            layers.append(parallel(l, right(sh, sp, rng.choice([8, 16, 20, 48, 64]), sg, rng.choice([1, 2, 3, 4]), ng),
                                   rng.choice([0.5, 1.0, 1.2]), rng.choice([0.7, 1.0, 1.4]), some_mlp()))
        else:
            heads = rng.choice([1, 2, 3, 5])
            layers.append(lightning(heads, rng.choice([8, 20, 32, 64, 72]), rng.choice([8, 16, 24, 40]),
                                    [rng.choice([0.3, 0.8, 0.95, 0.99, 0.9995]) for _ in range(heads)], some_mlp()))
    cfg = {"architecture": "Mogutar", "vocab": rng.choice([17, 64, 101, 300]), "width": width,
           "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "layers": layers}
    if rng.random() < 0.7:
        cfg["token_side"] = {"dim": rng.choice([8, 10, 12, 16])}
    return cfg


def write_model(name, path, seed=None, cfg=None, calm_router=False):
    cfg = cfg or CONFIGS[name]
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), draw_weights(cfg, seed if seed is not None else sum(map(ord, name)), calm_router))
    return path
