"""Typed configuration of the Nelovik decoder, read from config.json.

Nelovik is a decoder of parallel blocks with two norms: x += mixer(n1(x)) + ff(n2(x)), both RMS norms of the same x.
config.json lists the layers; a layer's `type` says which mixer it has:

* `delta`, `delta_2`: the gated delta rule.  q and k (kv_heads x dim) and v (heads x vdim) each pass a short causal
  convolution and silu; q and k become unit vectors; a decay and a write strength per head and token; a 32-bit state.
* `parallel`: softmax attention (`left`) beside the state space of Mamba-2 (`right`), each normed over the model
  width, half their sum.  The attention has biases, a norm over the whole q and k projections, rotation of the first
  rot.dims entries of a head, a capped score, a sliding window of mask.size tokens with one mean key and value for every
  block of mask.pool tokens behind it, and a sink per head.

The feed-forward is dense without a gate, down(xIELU(up h)).

    architecture   "Nelovik"
    vocab, width
    norm           {eps}
    layers         [{type, mixer: {...}, mlp: {kind: "dense", ff} | null}, ...]
        delta, delta_2:  mixer: heads, kv_heads, dim, vdim, conv
        parallel:        mixer: left:  heads, kv_heads, dim, vdim, scale, softcap, rot: {dims, base}, mask: {size, pool}
                                right: heads, vdim, state, groups, norm_groups, conv

Every size and constant comes from the file; a missing one is an error, an unknown layer type or feed-forward kind is
refused.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from .model_config import ConfigError, _as_float, _as_int
from .riruzen_config import _need, _section

DELTA_TYPES = ("delta", "delta_2")
PARALLEL = "parallel"
DENSE = "dense"


@dataclass(frozen=True)
class DeltaRuleSpec:
    heads: int
    kv_heads: int                   # heads of q and k; heads / kv_heads value heads share one
    dim: int
    vdim: int
    conv: int                       # taps of the short convolutions


@dataclass(frozen=True)
class PooledAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    rot_dims: int
    rot_base: float
    window: int                     # mask.size
    pool: int                       # mask.pool


@dataclass(frozen=True)
class StateSpaceSpec:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int


@dataclass(frozen=True)
class NelovikLayer:
    type: str
    delta: Optional[DeltaRuleSpec] = None
    left: Optional[PooledAttentionSpec] = None
    right: Optional[StateSpaceSpec] = None
    ff: Optional[int] = None        # None: no feed-forward


@dataclass(frozen=True)
class NelovikConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[NelovikLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Nelovik"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "NelovikConfig":
        _need(d, ("vocab", "width", "norm", "layers"), "config.json")
        norm = _section(d, "norm")
        _need(norm, ("eps",), "config.json: norm")
        if not isinstance(d["layers"], (list, tuple)) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with one entry a layer")
        layers = []
        for i, entry in enumerate(d["layers"]):
            where = f"config.json: layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where} must be an object")
            _need(entry, ("type", "mixer"), where)
            m = _section(entry, "mixer", where)
            ff = None
            if entry.get("mlp") is not None:
                mlp = _section(entry, "mlp", where)
                _need(mlp, ("kind", "ff"), f"{where}.mlp")
                if mlp["kind"] != DENSE:
                    raise ConfigError(f"{where}.mlp: unknown kind {mlp['kind']!r}; known: {DENSE}")
                ff = _as_int(mlp, "ff")
            if entry["type"] in DELTA_TYPES:
                _need(m, ("heads", "kv_heads", "dim", "vdim", "conv"), f"{where}.mixer")
                spec = DeltaRuleSpec(_as_int(m, "heads"), _as_int(m, "kv_heads"), _as_int(m, "dim"), _as_int(m, "vdim"), _as_int(m, "conv"))
                layers.append(NelovikLayer(entry["type"], delta=spec, ff=ff))
            elif entry["type"] == PARALLEL:
                _need(m, ("left", "right"), f"{where}.mixer")
                L, R = _section(m, "left", f"{where}.mixer"), _section(m, "right", f"{where}.mixer")
                _need(L, ("heads", "kv_heads", "dim", "vdim", "scale", "softcap", "rot", "mask"), f"{where}.mixer.left")
                rot, mask = _section(L, "rot", f"{where}.mixer.left"), _section(L, "mask", f"{where}.mixer.left")
                _need(rot, ("dims", "base"), f"{where}.mixer.left.rot")
                _need(mask, ("size", "pool"), f"{where}.mixer.left.mask")
                _need(R, ("heads", "vdim", "state", "groups", "norm_groups", "conv"), f"{where}.mixer.right")
                left = PooledAttentionSpec(_as_int(L, "heads"), _as_int(L, "kv_heads"), _as_int(L, "dim"), _as_int(L, "vdim"),
                                           _as_float(L, "scale"), _as_float(L, "softcap"), _as_int(rot, "dims"), _as_float(rot, "base"),
                                           _as_int(mask, "size"), _as_int(mask, "pool"))
                right = StateSpaceSpec(_as_int(R, "heads"), _as_int(R, "vdim"), _as_int(R, "state"), _as_int(R, "groups"),
                                       _as_int(R, "norm_groups"), _as_int(R, "conv"))
                layers.append(NelovikLayer(PARALLEL, left=left, right=right, ff=ff))
            else:
                raise ConfigError(f"{where}: unknown layer type {entry['type']!r}; known: {', '.join(DELTA_TYPES)}, {PARALLEL}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(architecture=cls.ARCHITECTURE, vocab=_as_int(d, "vocab"), width=_as_int(d, "width"),
                  norm_eps=_as_float(norm, "eps"), layers=tuple(layers), eos_token_ids=eos_ids, raw=dict(d))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"vocab and width must be positive, got {self.vocab}, {self.width}")
        if not (self.norm_eps > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        for i, l in enumerate(self.layers):
            where = f"layers[{i}]"
            if l.ff is not None and l.ff <= 0:
                raise ConfigError(f"{where}.mlp: ff must be positive, got {l.ff}")
            if l.delta is not None:
                s = l.delta
                if min(s.heads, s.kv_heads, s.dim, s.vdim, s.conv) <= 0:
                    raise ConfigError(f"{where}: every size must be positive, got {s}")
                if s.heads % s.kv_heads:
                    raise ConfigError(f"{where}: {s.heads} heads are not a multiple of {s.kv_heads} kv heads")
                continue
            a, r = l.left, l.right
            if min(a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.pool) <= 0 or a.rot_dims < 0:
                raise ConfigError(f"{where}.left: every size must be positive, got {a}")
            if a.heads % a.kv_heads:
                raise ConfigError(f"{where}.left: {a.heads} query heads are not a multiple of {a.kv_heads} kv heads")
            if a.rot_dims % 2 or a.rot_dims > a.dim:
                raise ConfigError(f"{where}.left: rot.dims {a.rot_dims} must be even and at most dim {a.dim}")
            if not (a.softcap > 0) or not (a.rot_base > 0):
                raise ConfigError(f"{where}.left: softcap and rot.base must be positive")
            if min(r.heads, r.vdim, r.state, r.groups, r.norm_groups, r.conv) <= 0:
                raise ConfigError(f"{where}.right: every size must be positive, got {r}")
            if r.heads % r.groups or (r.heads * r.vdim) % r.norm_groups:
                raise ConfigError(f"{where}.right: {r.heads} heads of {r.vdim} do not fit {r.groups} groups and {r.norm_groups} norm groups")

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for l in self.layers:
            if l.delta is not None:
                s = l.delta
                mixer: dict[str, Any] = {"heads": s.heads, "kv_heads": s.kv_heads, "dim": s.dim, "vdim": s.vdim, "conv": s.conv}
            else:
                a, r = l.left, l.right
                mixer = {"left": {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
                                  "softcap": a.softcap, "rot": {"dims": a.rot_dims, "base": a.rot_base},
                                  "mask": {"size": a.window, "pool": a.pool}},
                         "right": {"heads": r.heads, "vdim": r.vdim, "state": r.state, "groups": r.groups,
                                   "norm_groups": r.norm_groups, "conv": r.conv}}
            layers.append({"type": l.type, "mixer": mixer, "mlp": None if l.ff is None else {"kind": DENSE, "ff": l.ff}})
        d: dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
