"""Tiny Nelovik configurations with weights made here, model folders of them, and the comparison of what the engine
returns with the plain implementation (plain_nelovik.py)."""
from __future__ import annotations

import json
import random

import torch

from plain_nelovik import PlainNelovik


def _delta(heads, kv_heads, dim, vdim, conv, ff, kind="delta"):
    return {"type": kind, "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _left(heads, kv_heads, dim, vdim, scale, softcap, rot, base, size, pool):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
            "rot": {"dims": rot, "base": base}, "mask": {"size": size, "pool": pool}}


def _right(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def _pair(left, right, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _config(vocab, width, eps, layers):
    return {"architecture": "Nelovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# A: sizes that are no multiples of 8 (the bfloat16 engine falls back to its plain products), values smaller and larger
#    than keys, one kv head for several heads, a window shorter than two pages with blocks of 5 tokens, blocks longer
#    than the window, two and three taps, a layer without feed-forward, rotation of part of a head.
# B: everything that can be 1 is 1: one head each, one tap (no convolution state), a window of one token with blocks of
#    one token (every earlier token is its own block), one group, one norm group, the whole head rotated.
# C: sizes at which the bfloat16 engine takes its tensor-core products (multiples of 64), windows and blocks across
#    several pages, as many kv heads as heads, no rotation at all, state rows of 128.
# D: heads of 128, a window longer than any test sequence (no block is ever seen) beside a window of 7 tokens with
#    blocks of 3, a state space with as many groups as heads, state rows of 200 and value columns that fill no tile.
CONFIGS = {
    "A": _config(211, 72, 1e-5, [
        _delta(3, 1, 20, 12, 3, 100),
        _pair(_left(4, 2, 24, 16, 0.22, 20.0, 10, 10000.0, 24, 5), _right(3, 20, 12, 1, 3, 2), 60),
        _delta(2, 2, 36, 40, 4, None, "delta_2"),
        _pair(_left(3, 1, 12, 28, 0.3, 5.0, 12, 500.0, 6, 9), _right(2, 8, 40, 2, 1, 4), 44)]),
    "B": _config(97, 40, 1e-6, [
        _delta(1, 1, 40, 40, 1, 64),
        _pair(_left(1, 1, 16, 16, 0.25, 50.0, 16, 100.0, 1, 1), _right(1, 24, 8, 1, 1, 1), 32)]),
    "C": _config(331, 256, 1e-5, [
        _pair(_left(4, 4, 64, 64, 0.125, 30.0, 0, 10000.0, 40, 16), _right(4, 64, 128, 2, 4, 4), 512),
        _delta(4, 2, 128, 64, 4, 512),
        _delta(8, 8, 32, 32, 2, 256, "delta_2"),
        _pair(_left(8, 2, 64, 32, 0.125, 15.0, 32, 1000000.0, 33, 32), _right(8, 32, 64, 1, 2, 3), 256)]),
    "D": _config(150, 256, 1e-6, [
        _pair(_left(4, 2, 128, 128, 0.09, 30.0, 64, 10000.0, 1000, 64), _right(4, 40, 200, 4, 1, 4), 128),
        _delta(2, 1, 200, 48, 4, 256),
        _pair(_left(2, 1, 128, 128, 0.09, 8.0, 128, 10000.0, 7, 3), _right(2, 64, 16, 1, 8, 4), None)]),
}
PAGE = {"A": 16, "B": 8, "C": 16, "D": 16}


def make_weights(cfg: dict, seed: int, sharp: float = 1.0) -> dict[str, torch.Tensor]:
    """Random weights, rounded to bfloat16 as a checkpoint holds them.  `sharp` multiplies the weights of the query
    norm, so that a few keys (or blocks) carry a query's whole weight and one that is lost, misplaced or wrongly let
    through an edge changes the output by its full size."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    rnd = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    lin = lambda o, i, gain=1.0: rnd(o, i, std=gain / i ** 0.5)
    w = {"embed": rnd(cfg["vocab"], W), "final.norm": 1 + rnd(W, std=0.2), "head": lin(cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        w[p + "norm1"] = 1 + rnd(W, std=0.2)
        m = layer["mixer"]
        if layer["type"] in ("delta", "delta_2"):
            H, G, D, V, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = lin(G * D, W, 2.0), lin(G * D, W, 2.0), lin(H * V, W, 2.0)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * V)):
                w[p + f"mix.{n}.conv"] = rnd(c, taps, std=0.6)
            w[p + "mix.b"], w[p + "mix.a"], w[p + "mix.g"] = lin(H, W, 2.0), lin(H, W, 2.0), lin(H * V, W, 2.0)
            w[p + "mix.A_log"], w[p + "mix.dt_bias"] = rnd(H) - 1.5, rnd(H)             # decays from nearly 1 to well below
            w[p + "mix.norm"], w[p + "mix.o"] = 1 + rnd(V, std=0.2), lin(W, H * V)
        else:
            L, R = m["left"], m["right"]
            H, G, D, V = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
            q = p + "mix.left."
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * D, W), lin(G * D, W), lin(G * V, W)
            w[q + "q.b"], w[q + "k.b"], w[q + "v.b"] = rnd(H * D, std=0.3), rnd(G * D, std=0.3), rnd(G * V, std=0.3)
            w[q + "q.norm"], w[q + "k.norm"] = (1 + rnd(H * D, std=0.2)) * sharp, 1 + rnd(G * D, std=0.2)
            w[q + "sink"], w[q + "o"], w[q + "out"] = rnd(H), lin(W, H * V), 1 + rnd(W, std=0.2)
            H, V, N, Gr, taps = R["heads"], R["vdim"], R["state"], R["groups"], R["conv"]
            inner, r = H * V, p + "mix.right."
            w[r + "in"] = lin(2 * inner + 2 * Gr * N + H, W, 2.0)
            w[r + "conv"], w[r + "conv.b"] = rnd(inner + 2 * Gr * N, taps, std=0.6), rnd(inner + 2 * Gr * N, std=0.3)
            w[r + "dt_bias"], w[r + "A_log"], w[r + "D"] = rnd(H), rnd(H) - 1.0, 1 + rnd(H, std=0.3)
            w[r + "norm"], w[r + "o"], w[r + "out"] = 1 + rnd(inner, std=0.2), lin(W, inner), 1 + rnd(W, std=0.2)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            w[p + "norm2"] = 1 + rnd(W, std=0.2)
            w[p + "mlp.up"], w[p + "mlp.down"], w[p + "mlp.act"] = lin(ff, W, 1.5), lin(W, ff), rnd(2)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write_model(folder, cfg: dict, weights: dict[str, torch.Tensor]):
    from lucciola_b200.weights.safetensors_io import write_safetensors
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", weights)
    return folder


def tokens(cfg: dict, n: int, salt: int = 0) -> list[int]:
    g = torch.Generator().manual_seed(7919 * salt + n)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


_plain: dict = {}


def plain_logits(key, cfg: dict, weights: dict, ids: list[int]) -> torch.Tensor:
    """Float64 logits of the whole sequence at every position, by the plain implementation (cached)."""
    k = (key, tuple(ids))
    if k not in _plain:
        _plain[k] = PlainNelovik(cfg, weights).forward(ids)
    return _plain[k]


# Largest |engine - plain| as a fraction of the sequence's largest |logit|.
TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def compare(got: dict, key, cfg: dict, weights: dict, reqs: dict[str, list[int]], dtype: str, tol=None) -> float:
    """`tol`: one bound, or one for each request (see bound)."""
    bounds = tol if isinstance(tol, dict) else {rid: (TOL[dtype] if tol is None else tol) for rid in reqs}
    worst = 0.0
    assert got, "the trace asked for no logits"
    for rid, ids in reqs.items():
        ref = plain_logits(key, cfg, weights, ids)
        scale = ref.abs().max().item()
        tol = bounds[rid]
        for p in range(len(ids)):
            if (rid, p) not in got:
                continue
            row = got[(rid, p)]
            assert torch.isfinite(row).all(), f"request {rid} position {p}: logits are not finite"
            err = (row - ref[p]).abs().max().item() / scale
            assert err <= tol, f"request {rid}: first wrong position {p} (error {err:.3g} of scale, allowed {tol:.3g})"
            worst = max(worst, err)
    return worst


def rounding_alone(cfg: dict, weights: dict, ids: list[int]) -> float:
    """What rounding alone does to this model's logits: the largest change, as a fraction of the largest |logit|, when
    the plain implementation rounds to bfloat16 wherever a 16-bit engine may (the inputs of products, what the cache
    holds: plain_nelovik.ROUND) and nothing else."""
    import plain_nelovik as plain
    exact = PlainNelovik(cfg, weights).forward(ids)
    try:
        plain.ROUND = lambda x: x.to(torch.bfloat16).to(torch.float64)
        rounded = PlainNelovik(cfg, weights).forward(ids)
    finally:
        plain.ROUND = None
    return ((rounded - exact).abs().max() / exact.abs().max()).item()


def bound(dtype: str, cfg: dict, weights: dict, reqs: dict, base: float | None = None) -> dict:
    """The bound of a comparison, request by request: the type's own, or for bfloat16 three times what rounding alone
    does to this model on that request if that is more (a sequence of one or two tokens, whose mixers return next to
    nothing that the norms behind them then blow up, can be far more sensitive than a long one)."""
    base = TOL[dtype] if base is None else base
    if dtype != "bfloat16":
        return {rid: base for rid in reqs}
    out = {}
    for rid, ids in reqs.items():
        k = (id(weights), tuple(ids))
        if k not in _rounding:
            _rounding[k] = (weights, rounding_alone(cfg, weights, ids))      # the weights are held so that their id stays theirs
        out[rid] = max(base, 3 * _rounding[k][1])
    return out


_rounding: dict = {}


def random_config(seed: int) -> dict:
    """A configuration whose every size is drawn: widths, the number and order of layers, head counts and groupings,
    sizes that are no multiples of 4 or 8, values larger and smaller than keys, windows from one token to longer than
    the sequences, blocks shorter and longer than windows and pages, taps from 1 to 5, layers without feed-forward."""
    rng = random.Random(seed)
    width = rng.choice([24, 36, 40, 64, 72, 100, 128, 200])
    layers = []
    for _ in range(rng.randint(1, 4)):
        ff = rng.choice([None, 24, 64, 100, 128, 192])
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            layers.append(_delta(kv * rng.choice([1, 2, 4]), kv, rng.choice([4, 10, 16, 33, 64, 130]), rng.choice([3, 8, 20, 32, 40, 70]),
                                 rng.randint(1, 5), ff, rng.choice(["delta", "delta_2"])))
        else:
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([4, 8, 10, 16, 24, 64])
            rot = rng.choice([0, 2, dim // 2 * 2, dim // 4 * 2])
            left = _left(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([4, 8, 12, 20, 32, 72]), rng.choice([0.1, 0.2, 0.3]),
                         rng.choice([2.0, 10.0, 50.0]), rot, rng.choice([100.0, 10000.0, 1e6]), rng.choice([1, 2, 7, 16, 33, 64, 150, 500]),
                         rng.choice([1, 2, 3, 8, 16, 20, 50]))
            groups = rng.choice([1, 2, 3])
            rh = groups * rng.choice([1, 2])
            rv = rng.choice([4, 8, 20, 33, 64])
            ng = rng.choice([g for g in (1, 2, 4, rh) if (rh * rv) % g == 0])
            layers.append(_pair(left, _right(rh, rv, rng.choice([4, 16, 33, 64, 140]), groups, ng, rng.randint(1, 5)), ff))
    return _config(rng.choice([64, 97, 300]), width, rng.choice([1e-5, 1e-6]), layers)
