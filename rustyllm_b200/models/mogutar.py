"""The Mogutar decoder as a ``ModelSpec``: which parts, with which constants and which tensor names.

    x = embed[token]
    a layer:  x += rms_norm(mixer(x)) * norm1;  x += rms_norm(experts(x)) * norm2;  then the per-layer token input
              x += rms_norm(P (gelu_tanh(G x) * side.embed[token, layer's columns])) * side.norm
              (the sublayers read x itself; the norms sit on what they return)
    mixer "parallel":  left_scale * attention(x) + right_scale * state_space(x)
              attention: biased q, k, v; a short convolution over time behind the projections; a norm a head on
              q and k; partial rotary positions with stretched frequencies; soft-capped scores; a sliding window
              that keeps the sequence's first tokens
              state space: a selective state-space layer with a matrix state a head (parts/recurrent.py)
    mixer "lightning": linear attention with a fixed decay a head, a norm over the heads and a sigmoid gate
    experts:  sigmoid scores, a correction of the choice, groups of experts, weights not renormalised
    logits = head (rms_norm(x) * final.norm)

Tensor names: "embed", "side.embed", "l<i>.norm1", "l<i>.norm2", "l<i>.mix.*", "l<i>.mlp.router",
"l<i>.mlp.correction", "l<i>.mlp.e<j>.{gate,up,down}", "l<i>.side.{gate,proj,norm}", "final.norm", "head";
matrices [out, in].
"""
from __future__ import annotations

from ..config.mogutar import MogutarConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec


def _attention_spec(d: int, a, p: str, eps: float) -> PartSpec:
    if a.rot is not None and a.rot.dims:
        position = PartSpec("rope_yarn", {"head_dim": a.dim, "rotary_dim": a.rot.dims, "base": a.rot.base, "factor": a.rot.factor,
                                          "original": a.rot.original, "fast": a.rot.fast, "slow": a.rot.slow})
    else:
        position = PartSpec("none", {"head_dim": a.dim})
    return PartSpec("gqa_attention", {
        "hidden_size": d, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim,
        "scale": a.scale, "window": a.window, "keep_first": a.keep_first, "softcap": a.softcap, "conv_taps": a.conv,
        "qk_norm_eps": eps, "bias": True, "bias_o": False, "position": position,
        "names": {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_norm": p + "q.norm", "k_norm": p + "k.norm",
                  "suffix": "", "bias_suffix": ".b", "conv_suffix": ".conv"}})


def _state_space_spec(d: int, s, p: str, eps: float) -> PartSpec:
    return PartSpec("selective_state_space", {
        "hidden_size": d, "num_heads": s.heads, "head_dim": s.vdim, "state_size": s.state, "groups": s.groups,
        "conv_taps": s.conv, "norm_groups": s.norm_groups, "norm_eps": eps,
        "names": {"in": p + "in", "o": p + "o", "conv": p + "conv", "bias_suffix": ".b", "dt_bias": p + "dt_bias",
                  "A_log": p + "A_log", "D": p + "D", "norm": p + "norm", "suffix": ""}})


def mogutar_spec(cfg: MogutarConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers, ignored = [], []
    n_layers = len(cfg.layers)
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = l.mixer
        if l.type == "parallel":
            mixer = PartSpec("parallel_mixers", {"left": _attention_spec(d, m.left, p + "mix.left.", eps),
                                                 "right": _state_space_spec(d, m.right, p + "mix.right.", eps),
                                                 "left_scale": m.left_scale, "right_scale": m.right_scale})
        else:
            mixer = PartSpec("decay_linear_attention", {
                "hidden_size": d, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "decay": tuple(m.decay),
                "norm_eps": eps,
                "names": {"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "g": p + "mix.g", "o": p + "mix.o",
                          "norm": p + "mix.norm", "suffix": ""}})
        if l.mlp is None:
            ff, ff_norm = PartSpec("none"), PartSpec("none")
            ignored.append(p + "norm2")
        else:
            e = l.mlp
            ff = PartSpec("moe_mlp", {"hidden_size": d, "expert_size": e.ff, "num_experts": e.experts, "top": e.top,
                                      "router_bias": False, "scoring": "sigmoid", "groups": e.groups, "keep_groups": e.keep,
                                      "names": {"router": p + "mlp.router", "correction": p + "mlp.correction",
                                                "expert": p + "mlp.e{e}", "suffix": ""}})
            ff_norm = PartSpec("rms_norm", {"size": d, "eps": eps, "name": p + "norm2"})
        block = {}
        if cfg.side_dim is not None:
            block["after"] = PartSpec("token_side_input", {
                "hidden_size": d, "vocab_size": cfg.vocab, "columns": n_layers * cfg.side_dim, "offset": i * cfg.side_dim,
                "size": cfg.side_dim, "eps": eps, "table_owner": None if i == 0 else "layers.0.after.table",
                "names": {"table": "side.embed", "gate": p + "side.gate", "proj": p + "side.proj", "norm": p + "side.norm",
                          "suffix": ""}})
        layers.append(LayerSpec(block=PartSpec("post_norm", block), mixer=mixer,
                                mixer_norm=PartSpec("rms_norm", {"size": d, "eps": eps, "name": p + "norm1"}),
                                feed_forward=ff, feed_forward_norm=ff_norm))
    spec = ModelSpec(
        architecture="Mogutar", vocab_size=cfg.vocab, hidden_size=d, max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed"}),
        layers=tuple(layers), schedule=tuple(range(n_layers)),
        final_norm=PartSpec("rms_norm", {"size": d, "eps": eps, "name": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "head"}),
        ignored_tensors=tuple(ignored))
    spec.validate()
    return spec


MOGUTAR = register_architecture(("Mogutar", "mogutar"), MogutarConfig.from_dict, mogutar_spec)
