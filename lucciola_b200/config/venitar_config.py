"""Typed configuration of the Venitar decoder, read from config.json.

Venitar is a pre-norm decoder, x += mixer(n1(x)); x += ff(n2(x)) (a layer may have no feed-forward), whose embedding is
scaled, whose output head is the embedding table itself, and of which a run of layers may be repeated: layers
loop.start .. loop.stop - 1 run loop.times times in a row with the same weights and a cache of their own for every
pass, and before every pass but the first the embedding's output is added to the stream.  A layer's `type` names its
mixer:

* `retention`: linear attention with one fixed decay a head (`decay`), no softmax and no denominator, on rotated q and
  k; each head's output is RMS-normed without a weight and gated by silu.
* `attention`: softmax attention whose values are the keys as projected, with per-head norms of q and k, rotation,
  a mask of chunks of mask.size positions, and one more term of score 0 in the denominator.
* `parallel`: softmax attention (`left`: biases, rotation with optional YaRN scaling, a sliding window of mask.size
  tokens, an elementwise sigmoid gate) beside the gated delta rule with a decay for every key channel (`right`: short
  convolutions, maps of low rank for the decay and for the output gate), added as left_scale * left + right_scale * right.

The feed-forward is dense without a gate, down(relu(up h)^2).

    architecture   "Venitar"
    vocab, width
    embedding      {scale}
    norm           {eps}
    loop           {start, stop, times}                      (optional)
    layers         [{type, mixer: {...}, mlp: {kind: "dense", ff} | null}, ...]
        retention:  heads, dim, vdim, decay: [..], rot: {dims, base}
        attention:  heads, kv_heads, dim, vdim, scale, rot: {dims, base}, mask: {size}
        parallel:   left:  heads, kv_heads, dim, vdim, scale, rot: {dims, base, scaling: {factor, original, fast, slow}}, mask: {size}
                    right: heads, kv_heads, dim, vdim, conv
                    left_scale, right_scale

Every size and constant comes from the file; an unknown layer type or feed-forward kind is refused.  The ranks of the
low-rank maps are the shapes of their tensors (`a1`, `g1`), which the model reads when the weights are bound; a
configuration may name them (`decay_rank`, `gate_rank`) when there is no checkpoint to read them from.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from .model_config import ConfigError, _as_float, _as_int
from .riruzen_config import _need, _section

RETENTION = "retention"
ATTENTION = "attention"
PARALLEL = "parallel"
DENSE = "dense"


@dataclass(frozen=True)
class RotarySpec:
    dims: int = 0                   # 0: no rotation
    base: float = 10000.0
    factor: float = 0.0             # > 0: YaRN scaling with the three numbers below
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0


@dataclass(frozen=True)
class RetentionSpec:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: RotarySpec


@dataclass(frozen=True)
class SoftmaxAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotarySpec
    mask: int                       # mask.size: the chunk's or the window's length; 0: plain causal


@dataclass(frozen=True)
class ChannelDeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int = 0             # 0: read from the checkpoint's tensors
    gate_rank: int = 0


@dataclass(frozen=True)
class VenitarLayer:
    type: str
    retention: Optional[RetentionSpec] = None
    attention: Optional[SoftmaxAttentionSpec] = None
    left: Optional[SoftmaxAttentionSpec] = None
    right: Optional[ChannelDeltaSpec] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    ff: Optional[int] = None        # None: no feed-forward


def _rotary(m: Mapping[str, Any], where: str) -> RotarySpec:
    if m.get("rot") is None:
        return RotarySpec()
    rot = _section(m, "rot", where)
    _need(rot, ("dims", "base"), f"{where}.rot")
    sc = rot.get("scaling")
    if sc is None:
        return RotarySpec(_as_int(rot, "dims"), _as_float(rot, "base"))
    if not isinstance(sc, Mapping):
        raise ConfigError(f"{where}.rot.scaling must be an object")
    _need(sc, ("factor", "original", "fast", "slow"), f"{where}.rot.scaling")
    return RotarySpec(_as_int(rot, "dims"), _as_float(rot, "base"), _as_float(sc, "factor"), _as_float(sc, "original"),
                      _as_float(sc, "fast"), _as_float(sc, "slow"))


def _mask(m: Mapping[str, Any], where: str) -> int:
    if m.get("mask") is None:
        return 0
    mask = _section(m, "mask", where)
    _need(mask, ("size",), f"{where}.mask")
    return _as_int(mask, "size")


def _softmax(m: Mapping[str, Any], where: str) -> SoftmaxAttentionSpec:
    _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
    return SoftmaxAttentionSpec(_as_int(m, "heads"), _as_int(m, "kv_heads"), _as_int(m, "dim"), _as_int(m, "vdim"),
                                _as_float(m, "scale"), _rotary(m, where), _mask(m, where))


@dataclass(frozen=True)
class VenitarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[VenitarLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_ids: tuple[int, ...] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Venitar"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "VenitarConfig":
        _need(d, ("vocab", "width", "norm", "layers"), "config.json")
        norm = _section(d, "norm")
        _need(norm, ("eps",), "config.json: norm")
        scale = 1.0
        if d.get("embedding") is not None:
            emb = _section(d, "embedding")
            _need(emb, ("scale",), "config.json: embedding")
            scale = _as_float(emb, "scale")
        start, stop, times = 0, 0, 1
        if d.get("loop") is not None:
            loop = _section(d, "loop")
            _need(loop, ("start", "stop", "times"), "config.json: loop")
            start, stop, times = _as_int(loop, "start"), _as_int(loop, "stop"), _as_int(loop, "times")
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
            kind = entry["type"]
            if kind == RETENTION:
                _need(m, ("heads", "dim", "vdim", "decay"), f"{where}.mixer")
                if not isinstance(m["decay"], (list, tuple)):
                    raise ConfigError(f"{where}.mixer.decay must be a list with one number a head")
                spec = RetentionSpec(_as_int(m, "heads"), _as_int(m, "dim"), _as_int(m, "vdim"),
                                     tuple(float(x) for x in m["decay"]), _rotary(m, f"{where}.mixer"))
                layers.append(VenitarLayer(kind, retention=spec, ff=ff))
            elif kind == ATTENTION:
                layers.append(VenitarLayer(kind, attention=_softmax(m, f"{where}.mixer"), ff=ff))
            elif kind == PARALLEL:
                _need(m, ("left", "right", "left_scale", "right_scale"), f"{where}.mixer")
                L, R = _section(m, "left", f"{where}.mixer"), _section(m, "right", f"{where}.mixer")
                _need(R, ("heads", "kv_heads", "dim", "vdim", "conv"), f"{where}.mixer.right")
                right = ChannelDeltaSpec(_as_int(R, "heads"), _as_int(R, "kv_heads"), _as_int(R, "dim"), _as_int(R, "vdim"),
                                         _as_int(R, "conv"), _as_int(R, "decay_rank") if R.get("decay_rank") is not None else 0,
                                         _as_int(R, "gate_rank") if R.get("gate_rank") is not None else 0)
                layers.append(VenitarLayer(kind, left=_softmax(L, f"{where}.mixer.left"), right=right,
                                           left_scale=_as_float(m, "left_scale"), right_scale=_as_float(m, "right_scale"), ff=ff))
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {RETENTION}, {ATTENTION}, {PARALLEL}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(architecture=cls.ARCHITECTURE, vocab=_as_int(d, "vocab"), width=_as_int(d, "width"),
                  norm_eps=_as_float(norm, "eps"), embedding_scale=scale, layers=tuple(layers), loop_start=start, loop_stop=stop,
                  loop_times=times, eos_token_ids=eos_ids, raw=dict(d))
        cfg.validate()
        return cfg

    def with_tensor_shapes(self, shape_of) -> "VenitarConfig":
        """The same configuration with the ranks of the low-rank maps taken from the checkpoint where config.json does
        not name them: shape_of(name) is a tensor's shape, or None if the checkpoint lacks it."""
        import dataclasses
        layers = []
        for i, l in enumerate(self.layers):
            if l.right is not None:
                r = l.right
                a1, g1 = shape_of(f"l{i}.mix.right.a1"), shape_of(f"l{i}.mix.right.g1")
                r = dataclasses.replace(r, decay_rank=r.decay_rank or (a1[0] if a1 else 0), gate_rank=r.gate_rank or (g1[0] if g1 else 0))
                l = dataclasses.replace(l, right=r)
            layers.append(l)
        return dataclasses.replace(self, layers=tuple(layers))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"vocab and width must be positive, got {self.vocab}, {self.width}")
        if not (self.norm_eps > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if not (0 <= self.loop_start <= self.loop_stop <= len(self.layers)) or self.loop_times < 1:
            raise ConfigError(f"loop {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit {len(self.layers)} layers")

        def rotary(r: RotarySpec, dim: int, where: str) -> None:
            if r.dims < 0 or r.dims % 2 or r.dims > dim:
                raise ConfigError(f"{where}: rot.dims {r.dims} must be even and at most dim {dim}")
            if r.dims and not (r.base > 1):
                raise ConfigError(f"{where}: rot.base must be above 1, got {r.base}")
            if r.factor and not (r.factor >= 1 and r.original > 0 and r.fast > 0 and r.slow > 0):
                raise ConfigError(f"{where}: rot.scaling wants factor >= 1 and positive original, fast, slow")

        def softmax(a: SoftmaxAttentionSpec, where: str) -> None:
            if min(a.heads, a.kv_heads, a.dim, a.vdim) <= 0 or a.mask < 0:
                raise ConfigError(f"{where}: every size must be positive, got {a}")
            if a.heads % a.kv_heads:
                raise ConfigError(f"{where}: {a.heads} query heads are not a multiple of {a.kv_heads} kv heads")
            rotary(a.rot, a.dim, where)

        for i, l in enumerate(self.layers):
            where = f"layers[{i}]"
            if l.ff is not None and l.ff <= 0:
                raise ConfigError(f"{where}.mlp: ff must be positive, got {l.ff}")
            if l.retention is not None:
                s = l.retention
                if min(s.heads, s.dim, s.vdim) <= 0 or len(s.decay) != s.heads:
                    raise ConfigError(f"{where}: sizes must be positive and decay hold one number a head, got {s}")
                rotary(s.rot, s.dim, where)
            elif l.attention is not None:
                softmax(l.attention, where)
                if l.attention.vdim != l.attention.dim:
                    raise ConfigError(f"{where}: the values are the keys, so vdim {l.attention.vdim} must equal dim {l.attention.dim}")
            else:
                softmax(l.left, f"{where}.left")
                r = l.right
                if min(r.heads, r.kv_heads, r.dim, r.vdim, r.conv) <= 0 or r.heads % r.kv_heads:
                    raise ConfigError(f"{where}.right: sizes must be positive and heads a multiple of kv_heads, got {r}")

    def to_dict(self) -> dict[str, Any]:
        def rot(r: RotarySpec) -> dict[str, Any]:
            out: dict[str, Any] = {"dims": r.dims, "base": r.base}
            if r.factor:
                out["scaling"] = {"factor": r.factor, "original": r.original, "fast": r.fast, "slow": r.slow}
            return out

        def softmax(a: SoftmaxAttentionSpec) -> dict[str, Any]:
            out = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale, "rot": rot(a.rot)}
            if a.mask:
                out["mask"] = {"size": a.mask}
            return out

        layers = []
        for l in self.layers:
            if l.retention is not None:
                s = l.retention
                mixer: dict[str, Any] = {"heads": s.heads, "dim": s.dim, "vdim": s.vdim, "decay": list(s.decay), "rot": rot(s.rot)}
            elif l.attention is not None:
                mixer = softmax(l.attention)
            else:
                r = l.right
                right = {"heads": r.heads, "kv_heads": r.kv_heads, "dim": r.dim, "vdim": r.vdim, "conv": r.conv}
                if r.decay_rank:
                    right["decay_rank"] = r.decay_rank
                if r.gate_rank:
                    right["gate_rank"] = r.gate_rank
                mixer = {"left": softmax(l.left), "right": right, "left_scale": l.left_scale, "right_scale": l.right_scale}
            layers.append({"type": l.type, "mixer": mixer, "mlp": None if l.ff is None else {"kind": DENSE, "ff": l.ff}})
        d: dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": layers,
                             "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
