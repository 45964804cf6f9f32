"""Typed configuration of the Mogutar decoder, read from its config.json.

The file describes the model layer by layer; every layer names its mixer by "type":

    {"architecture": "Mogutar", "vocab": V, "width": d, "norm": {"eps": e}, "token_side": {"dim": n},
     "layers": [
       {"type": "parallel",
        "mixer": {"left_scale": a, "right_scale": b,
                  "left":  {"heads": H, "kv_heads": G, "dim": hd, "vdim": vd, "conv": taps, "scale": s, "softcap": c,
                            "mask": {"size": W, "keep_first": F},
                            "rot": {"base": B, "dims": r,
                                    "scaling": {"factor": f, "original": L, "fast": t1, "slow": t0}}},
                  "right": {"heads": Hs, "vdim": P, "state": N, "groups": Gs, "conv": taps, "norm_groups": ng}},
        "mlp": {"kind": "moe", "router": {"experts": E, "top": k, "groups": {"count": c, "keep": m}},
                "expert": {"ff": F}} | null},
       {"type": "lightning", "mixer": {"heads": H, "dim": dk, "vdim": dv, "decay": [a_0 .. a_{H-1}]}, "mlp": ...}]}

Every size and constant that can differ between two models of the design is read here; nothing downstream
hard-codes one.  May be absent (or null): ``token_side`` (no per-layer token input), a layer's ``mlp`` (a mixer
alone), ``mask`` (all earlier positions are seen) and its ``keep_first``, ``rot`` (no rotation) and its
``scaling``, ``softcap``, ``conv`` of the left mixer (no convolution), the router's ``groups``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .files import ConfigError
from .mosurax import _int, _num, _obj


def _opt_obj(d: Mapping[str, Any], key: str, where: str) -> Optional[Mapping[str, Any]]:
    return None if d.get(key) is None else _obj(d, key, where)


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    factor: Optional[float] = None      # with a factor: the stretched frequencies, from (original, fast, slow)
    original: Optional[float] = None
    fast: Optional[float] = None
    slow: Optional[float] = None

    def to_dict(self) -> dict:
        d = {"base": self.base, "dims": self.dims}
        if self.factor is not None:
            d["scaling"] = {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}
        return d


@dataclass(frozen=True)
class WindowedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int = 0                        # taps of the convolution behind the q, k, v projections; 0: none
    softcap: Optional[float] = None
    window: Optional[int] = None         # mask.size
    keep_first: int = 0                  # mask.keep_first
    rot: Optional[RotaryConfig] = None

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.conv:
            d["conv"] = self.conv
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.window is not None:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class StateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class ParallelMixer:
    left: WindowedAttention
    right: StateSpace
    left_scale: float
    right_scale: float

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1

    def to_dict(self) -> dict:
        r = {"experts": self.experts, "top": self.top}
        if self.groups > 1:
            r["groups"] = {"count": self.groups, "keep": self.keep}
        return {"kind": "moe", "router": r, "expert": {"ff": self.ff}}


@dataclass(frozen=True)
class MogutarLayer:
    type: str                                        # "parallel" or "lightning"
    mixer: Union[ParallelMixer, LightningMixer]
    mlp: Optional[ExpertsConfig]

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class MogutarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[MogutarLayer, ...]
    side_dim: Optional[int] = None                   # token_side.dim; None: no per-layer token input

    # the names other parts of the library read from any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def max_position_embeddings(self) -> int:
        return 1 << 24           # the design sets no limit; positions stay exact in float32 up to here

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def to_dict(self) -> dict:
        d = {"architecture": "Mogutar", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [l.to_dict() for l in self.layers]}
        if self.side_dim is not None:
            d["token_side"] = {"dim": self.side_dim}
        return d

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MogutarConfig":
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
            m = _obj(l, "mixer", lw)
            if kind == "parallel":
                mixer = ParallelMixer(left=_attention(_obj(m, "left", lw + ".mixer"), lw + ".mixer.left"),
                                      right=_state_space(_obj(m, "right", lw + ".mixer"), lw + ".mixer.right"),
                                      left_scale=_num(m, "left_scale", lw + ".mixer"), right_scale=_num(m, "right_scale", lw + ".mixer"))
            elif kind == "lightning":
                heads = _int(m, "heads", lw + ".mixer")
                decay = m.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != heads or \
                        any(isinstance(a, bool) or not isinstance(a, (int, float)) for a in decay):
                    raise ConfigError(f"{lw}.mixer: 'decay' must list one number for each of the {heads} heads")
                mixer = LightningMixer(heads=heads, dim=_int(m, "dim", lw + ".mixer"), vdim=_int(m, "vdim", lw + ".mixer"),
                                       decay=tuple(float(a) for a in decay))
            else:
                raise ConfigError(f"{lw}: mixer type {kind!r} is not known; known: 'parallel', 'lightning'")
            layers.append(MogutarLayer(kind, mixer, _experts(l.get("mlp"), lw + ".mlp")))
        side = _opt_obj(d, "token_side", where)
        return cls(vocab=_int(d, "vocab", where), width=_int(d, "width", where),
                   norm_eps=_num(_obj(d, "norm", where), "eps", where + ": norm"), layers=tuple(layers),
                   side_dim=None if side is None else _int(side, "dim", where + ": token_side"))


def _attention(m: Mapping[str, Any], w: str) -> WindowedAttention:
    mask = _opt_obj(m, "mask", w)
    window, keep = None, 0
    if mask is not None:
        window = _int(mask, "size", w + ".mask")
        keep = 0 if mask.get("keep_first") is None else _int(mask, "keep_first", w + ".mask", 0)
    rot_in = _opt_obj(m, "rot", w)
    rot = None
    if rot_in is not None:
        sc = _opt_obj(rot_in, "scaling", w + ".rot")
        kw = {}
        if sc is not None:
            kw = {k: _num(sc, k, w + ".rot.scaling") for k in ("factor", "original", "fast", "slow")}
            if kw["factor"] < 1.0 or kw["original"] <= 0 or kw["fast"] <= 0 or kw["slow"] <= 0:
                raise ConfigError(f"{w}.rot.scaling: factor must be >= 1, original, fast and slow positive")
        rot = RotaryConfig(base=_num(rot_in, "base", w + ".rot"), dims=_int(rot_in, "dims", w + ".rot", 0), **kw)
        if rot.dims % 2 or rot.base <= 1.0:
            raise ConfigError(f"{w}.rot: 'dims' must be even and 'base' above 1")
    cap = None if m.get("softcap") is None else _num(m, "softcap", w)
    if cap is not None and not cap > 0:
        raise ConfigError(f"{w}: 'softcap' must be > 0, got {cap}")
    a = WindowedAttention(heads=_int(m, "heads", w), kv_heads=_int(m, "kv_heads", w), dim=_int(m, "dim", w), vdim=_int(m, "vdim", w),
                          scale=_num(m, "scale", w), conv=0 if m.get("conv") is None else _int(m, "conv", w, 0), softcap=cap,
                          window=window, keep_first=keep, rot=rot)
    if a.heads % a.kv_heads:
        raise ConfigError(f"{w}: {a.heads} heads are no multiple of {a.kv_heads} kv_heads")
    if rot is not None and rot.dims > a.dim:
        raise ConfigError(f"{w}.rot: {rot.dims} rotated dimensions exceed the head's {a.dim}")
    return a


def _state_space(m: Mapping[str, Any], w: str) -> StateSpace:
    s = StateSpace(heads=_int(m, "heads", w), vdim=_int(m, "vdim", w), state=_int(m, "state", w), groups=_int(m, "groups", w),
                   conv=_int(m, "conv", w), norm_groups=_int(m, "norm_groups", w))
    if s.heads % s.groups:
        raise ConfigError(f"{w}: {s.heads} heads are no multiple of {s.groups} groups")
    if (s.heads * s.vdim) % s.norm_groups:
        raise ConfigError(f"{w}: {s.norm_groups} norm_groups do not divide {s.heads * s.vdim} channels")
    return s


def _experts(mlp_in: Any, w: str) -> Optional[ExpertsConfig]:
    if mlp_in is None:
        return None
    if not isinstance(mlp_in, Mapping):
        raise ConfigError(f"{w} must be an object or null")
    if mlp_in.get("kind") != "moe":
        raise ConfigError(f"{w}: kind {mlp_in.get('kind')!r} is not known; known: 'moe'")
    r = _obj(mlp_in, "router", w)
    g = _opt_obj(r, "groups", w + ".router")
    e = ExpertsConfig(experts=_int(r, "experts", w + ".router"), top=_int(r, "top", w + ".router"),
                      ff=_int(_obj(mlp_in, "expert", w), "ff", w + ".expert"),
                      groups=1 if g is None else _int(g, "count", w + ".router.groups"),
                      keep=1 if g is None else _int(g, "keep", w + ".router.groups"))
    if e.top > e.experts:
        raise ConfigError(f"{w}.router: top {e.top} exceeds experts {e.experts}")
    if e.experts % e.groups or e.keep > e.groups:
        raise ConfigError(f"{w}.router.groups: {e.groups} groups (keep {e.keep}) do not fit {e.experts} experts")
    if e.keep * (e.experts // e.groups) < e.top:
        raise ConfigError(f"{w}.router.groups: the {e.keep} kept groups hold fewer than top = {e.top} experts")
    return e
