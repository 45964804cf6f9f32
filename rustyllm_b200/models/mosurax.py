"""The Mosurax decoder as a ``ModelSpec``: which parts, with which constants and which tensor names.

    x = embed[token] + pos[position]
    layers in the order of config "layers"; layers loop.start .. loop.stop - 1 run loop.times times in
    a row with the same weights (every pass with a cache of its own); before each pass but the first
    the embedding's output is added to x again, and before every pass the pass's row of "loop.step"
    a layer:  x += attention(rms_norm(x) * norm1);  x += feed_forward(rms_norm(x) * norm2)
    attention: grouped-query, no rotation, scores (q . k) * scale, a sliding window, a softmax with one
               more term of score 0 in its denominator, an output gate sigmoid(Wg h) in front of Wo
    feed_forward: a gated SiLU feed-forward, or a mixture of such experts with a shared one, or none
    logits = head (rms_norm(x) * final.norm), then softcap * tanh(logits / softcap)

Tensor names: "embed", "pos", "loop.step", "l<i>.norm1", "l<i>.norm2", "l<i>.mix.{q,k,v,g,o}",
"l<i>.mlp.{gate,up,down}" or "l<i>.mlp.router", "l<i>.mlp.router.b", "l<i>.mlp.e<j>.{gate,up,down}",
"l<i>.mlp.shared.{gate,up,down}", "final.norm", "head"; matrices [out, in].
"""
from __future__ import annotations

from ..config.mosurax import MosuraxConfig
from ..config.registry import register_architecture
from ..config.spec import Injection, LayerSpec, ModelSpec, PartSpec


def mosurax_spec(cfg: MosuraxConfig) -> ModelSpec:
    d = cfg.width
    layers, ignored = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = l.mixer
        mixer = PartSpec("gqa_attention", {
            "hidden_size": d, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
            "value_dim": m.vdim, "window": m.window, "scale": m.scale, "sink": True,
            "position": PartSpec("none", {"head_dim": m.dim}),
            "names": {"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "g": p + "mix.g", "o": p + "mix.o", "suffix": ""},
        })
        if l.mlp is None:
            ff, ff_norm = PartSpec("none"), PartSpec("none")
            ignored.append(p + "norm2")
        elif l.mlp.kind == "dense":
            ff = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": l.mlp.ff, "activation": "silu",
                                        "names": {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down", "suffix": ""}})
            ff_norm = PartSpec("rms_norm", {"size": d, "eps": cfg.norm_eps, "name": p + "norm2"})
        else:
            shared = None
            if l.mlp.shared_ff is not None:
                shared = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": l.mlp.shared_ff, "activation": "silu",
                                                "names": {"gate": p + "mlp.shared.gate", "up": p + "mlp.shared.up",
                                                          "down": p + "mlp.shared.down", "suffix": ""}})
            ff = PartSpec("moe_mlp", {"hidden_size": d, "expert_size": l.mlp.ff, "num_experts": l.mlp.experts, "top": l.mlp.top,
                                      "router_bias": True, "shared": shared,
                                      "names": {"router": p + "mlp.router", "bias_suffix": ".b", "expert": p + "mlp.e{e}", "suffix": ""}})
            ff_norm = PartSpec("rms_norm", {"size": d, "eps": cfg.norm_eps, "name": p + "norm2"})
        layers.append(LayerSpec(block=PartSpec("pre_norm"), mixer=mixer,
                                mixer_norm=PartSpec("rms_norm", {"size": d, "eps": cfg.norm_eps, "name": p + "norm1"}),
                                feed_forward=ff, feed_forward_norm=ff_norm))
    n = len(layers)
    schedule, injections, inject_parts = list(range(n)), (), ()
    if cfg.loop is not None:
        a, b, times = cfg.loop.start, cfg.loop.stop, cfg.loop.times
        schedule = list(range(a))
        inj = []
        for t in range(times):
            # what is added before pass t stands before the run that follows it (the pass's first layer, or,
            # where the looped range is empty, the first layer behind it)
            inj.append((len(schedule), t))
            schedule += list(range(a, b))
        schedule += list(range(b, n))
        if any(at >= len(schedule) for at, _ in inj):
            raise ValueError("a loop at the very end of the layers over an empty range has no layer to stand before")
        inject_parts = (PartSpec("pass_entry", {"hidden_size": d, "passes": times, "name": "loop.step"}),)
        injections = tuple(Injection(before_run=at, part=0, args={"row": t, "again": t > 0}) for at, t in inj)
    spec = ModelSpec(
        architecture="Mosurax", vocab_size=cfg.vocab, hidden_size=d, max_position_embeddings=cfg.max_positions,
        embedding=PartSpec("token_position_embedding", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed",
                                                        "max_positions": cfg.max_positions, "position_name": "pos"}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("rms_norm", {"size": d, "eps": cfg.norm_eps, "name": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "head", "softcap": cfg.logit_softcap}),
        ignored_tensors=tuple(ignored), inject_parts=inject_parts, injections=injections)
    spec.validate()
    return spec


MOSURAX = register_architecture(("Mosurax", "mosurax"), MosuraxConfig.from_dict, mosurax_spec)
