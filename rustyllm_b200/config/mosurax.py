"""Typed configuration of the Mosurax decoder, read from its config.json.

The file describes the model layer by layer:

    {"architecture": "Mosurax", "vocab": V, "width": d, "max_positions": P,
     "norm": {"eps": e}, "logit_softcap": c,
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": hd, "vdim": vd, "scale": s, "mask": {"size": W}},
                 "mlp": {"kind": "dense", "ff": I}
                      | {"kind": "moe", "router": {"experts": E, "top": k}, "expert": {"ff": F}, "shared": {"ff": S}}
                      | null}, ...]}

Every size and every constant that can differ between two models of the design is read here;
nothing downstream hard-codes one.  ``loop`` may be absent (no layer repeats), a layer's ``mlp`` may
be null (a mixer alone), ``mask`` may be absent (all earlier positions are seen), ``shared`` may be
absent (no shared expert), ``logit_softcap`` may be absent or null (logits as they are).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .files import ConfigError


def _int(d: Mapping[str, Any], key: str, where: str, least: int = 1) -> int:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"{where}: '{key}' must be an integer, got {v!r}")
    if v < least:
        raise ConfigError(f"{where}: '{key}' must be >= {least}, got {v}")
    return v


def _num(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: '{key}' must be a number, got {v!r}")
    return float(v)


def _obj(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: '{key}' must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int                 # width of a query/key head
    vdim: int                # width of a value head
    scale: float             # scores are (q . k) * scale
    window: Optional[int]    # mask.size: position i sees j with 0 <= i - j < window; None: all j <= i

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                          # "dense" or "moe"
    ff: int = 0                        # dense: intermediate size; moe: an expert's
    experts: int = 0
    top: int = 0
    shared_ff: Optional[int] = None    # moe: the shared expert's intermediate size, None: no shared expert

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class MosuraxLayer:
    type: str
    mixer: AttentionMixer
    mlp: Optional[FeedForwardConfig]

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class MosuraxConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: Tuple[MosuraxLayer, ...]
    loop: Optional[Loop] = None
    logit_softcap: Optional[float] = None

    # the names other parts of the library read from any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def to_dict(self) -> dict:
        d = {"architecture": "Mosurax", "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
             "norm": {"eps": self.norm_eps}, "layers": [l.to_dict() for l in self.layers]}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MosuraxConfig":
        where = "config.json"
        layers_in = d.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(layers_in):
            lw = f"{where}: layers[{i}]"
            if not isinstance(l, Mapping):
                raise ConfigError(f"{lw} must be an object")
            kind = l.get("type")
            if kind != "attention":
                raise ConfigError(f"{lw}: mixer type {kind!r} is not known; known: 'attention'")
            m = _obj(l, "mixer", lw)
            mask = m.get("mask")
            window = None
            if mask is not None:
                window = _int(_obj(m, "mask", lw + ".mixer"), "size", lw + ".mixer.mask")
            mixer = AttentionMixer(heads=_int(m, "heads", lw + ".mixer"), kv_heads=_int(m, "kv_heads", lw + ".mixer"),
                                   dim=_int(m, "dim", lw + ".mixer"), vdim=_int(m, "vdim", lw + ".mixer"),
                                   scale=_num(m, "scale", lw + ".mixer"), window=window)
            if mixer.heads % mixer.kv_heads:
                raise ConfigError(f"{lw}.mixer: {mixer.heads} heads are no multiple of {mixer.kv_heads} kv_heads")
            mlp_in = l.get("mlp")
            mlp = None
            if mlp_in is not None:
                mw = lw + ".mlp"
                if not isinstance(mlp_in, Mapping):
                    raise ConfigError(f"{mw} must be an object or null")
                fk = mlp_in.get("kind")
                if fk == "dense":
                    mlp = FeedForwardConfig("dense", ff=_int(mlp_in, "ff", mw))
                elif fk == "moe":
                    r = _obj(mlp_in, "router", mw)
                    shared = mlp_in.get("shared")
                    mlp = FeedForwardConfig("moe", ff=_int(_obj(mlp_in, "expert", mw), "ff", mw + ".expert"),
                                            experts=_int(r, "experts", mw + ".router"), top=_int(r, "top", mw + ".router"),
                                            shared_ff=None if shared is None else _int(_obj(mlp_in, "shared", mw), "ff", mw + ".shared"))
                    if mlp.top > mlp.experts:
                        raise ConfigError(f"{mw}.router: top {mlp.top} exceeds experts {mlp.experts}")
                else:
                    raise ConfigError(f"{mw}: kind {fk!r} is not known; known: 'dense', 'moe'")
            layers.append(MosuraxLayer(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lo = _obj(d, "loop", where)
            loop = Loop(start=_int(lo, "start", where + ": loop", 0), stop=_int(lo, "stop", where + ": loop", 0),
                        times=_int(lo, "times", where + ": loop", 1))
            if not (loop.start <= loop.stop <= len(layers)):
                raise ConfigError(f"{where}: loop {loop.start}..{loop.stop} does not lie within the {len(layers)} layers")
        cap = d.get("logit_softcap")
        if cap is not None:
            cap = _num(d, "logit_softcap", where)
            if not cap > 0:
                raise ConfigError(f"{where}: 'logit_softcap' must be > 0, got {cap}")
        return cls(vocab=_int(d, "vocab", where), width=_int(d, "width", where),
                   max_positions=_int(d, "max_positions", where), norm_eps=_num(_obj(d, "norm", where), "eps", where + ": norm"),
                   layers=tuple(layers), loop=loop, logit_softcap=cap)
