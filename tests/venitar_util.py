"""Tiny Venitar configurations with weights made here, model folders of them, and the comparison of what the engine
returns with the plain implementation (plain_venitar.py)."""
from __future__ import annotations

import json
import random

import torch

from plain_venitar import PlainVenitar


def _mlp(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def _rot(dims, base, yarn=None):
    r = {"dims": dims, "base": base}
    if yarn is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    return r


def _retention(heads, dim, vdim, decay, rot, ff):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": rot}, "mlp": _mlp(ff)}


def _attention(heads, kv_heads, dim, scale, rot, chunk, ff):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rot,
                                           "mask": {"size": chunk}}, "mlp": _mlp(ff)}


def _left(heads, kv_heads, dim, vdim, scale, rot, window):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot, "mask": {"size": window}}


def _right(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank, "gate_rank": gate_rank}


def _pair(left, right, left_scale, right_scale, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}, "mlp": _mlp(ff)}


def _config(vocab, width, eps, scale, loop, layers):
    return {"architecture": "Venitar", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "loop": dict(zip(("start", "stop", "times"), loop)), "layers": layers}


# A: sizes that are no multiples of 8 (the bfloat16 engine falls back to its plain products), values smaller and larger
#    than keys, a window and a chunk shorter than two pages, YaRN on part of a head, two and three taps, odd ranks, a
#    loop over the two middle layers, a layer without feed-forward.
# B: everything that can be 1 is 1: one head each, one tap (no convolution state), a window and a chunk of one token, rank
#    1, one pass of the loop, an embedding scale of 1, no rotation in one mixer and the whole head in another.
# C: sizes at which the bfloat16 engine takes its tensor-core kernels (multiples of 64), windows and chunks across
#    several pages, as many kv heads as heads, three passes over the two middle layers, state rows of 128.
# D: heads of 128, a window and a chunk longer than any test sequence, state rows of 200 and 256, value columns that
#    fill no tile, the loop over all layers.
CONFIGS = {
    "A": _config(211, 72, 1e-5, 0.7, (1, 3, 2), [
        _pair(_left(4, 2, 24, 16, 0.22, _rot(10, 10000.0, (4.0, 64, 8.0, 1.0)), 24), _right(3, 1, 20, 12, 3, 5, 7), 0.6, 1.3, 100),
        _retention(3, 20, 12, (0.9, 0.99, 0.999), _rot(8, 500.0), None),
        _attention(4, 2, 24, 0.25, _rot(24, 10000.0), 10, 60),
        _pair(_left(3, 1, 12, 28, 0.3, _rot(12, 500.0), 6), _right(2, 2, 36, 40, 2, 3, 2), 1.0, 0.5, 44)]),
    "B": _config(97, 40, 1e-6, 1.0, (0, 2, 1), [
        _pair(_left(1, 1, 16, 16, 0.25, _rot(16, 100.0, (1.0, 8, 4.0, 2.0)), 1), _right(1, 1, 40, 40, 1, 1, 1), 1.0, 1.0, 32),
        _retention(1, 16, 24, (0.95,), _rot(0, 100.0), 64),
        _attention(1, 1, 16, 0.3, _rot(16, 100.0), 1, None)]),
    "C": _config(331, 256, 1e-5, 0.25, (1, 3, 3), [
        _attention(4, 4, 64, 0.125, _rot(32, 500000.0), 40, 512),
        _pair(_left(8, 2, 64, 64, 0.125, _rot(64, 10000.0, (3.0, 128, 16.0, 2.0)), 33), _right(4, 2, 128, 64, 4, 16, 8), 0.75, 1.25, 256),
        _retention(4, 64, 64, (0.9, 0.97, 0.995, 0.9995), _rot(64, 10000.0), 256),
        _attention(8, 2, 64, 0.125, _rot(64, 10000.0), 64, None)]),
    "D": _config(150, 256, 1e-6, 2.0, (0, 3, 2), [
        _pair(_left(4, 2, 128, 96, 0.09, _rot(64, 10000.0), 1000), _right(2, 1, 200, 48, 4, 8, 24), 1.2, 0.7, 128),
        _retention(2, 256, 40, (0.98, 0.9999), _rot(128, 300000.0), None),
        _attention(2, 1, 128, 0.09, _rot(128, 10000.0), 1000, 128)]),
}
PAGE = {"A": 16, "B": 8, "C": 16, "D": 16}


def make_weights(cfg: dict, seed: int, sharp: float = 1.0) -> dict[str, torch.Tensor]:
    """Random weights, rounded to bfloat16 as a checkpoint holds them.  `sharp` multiplies the queries of the softmax
    attentions (the query norm's weight, or the query map and its bias where there is no norm), so that a few keys
    carry a query's whole weight and one that is lost, misplaced or wrongly let through an edge changes the output by
    its full size."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    rnd = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    lin = lambda o, i, gain=1.0: rnd(o, i, std=gain / i ** 0.5)
    w = {"embed": rnd(cfg["vocab"], W), "final.norm": 1 + rnd(W, std=0.2)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        w[p + "norm1"] = 1 + rnd(W, std=0.2)
        m = layer["mixer"]
        if layer["type"] == "retention":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = lin(H * D, W, 2.0), lin(H * D, W, 2.0), lin(H * V, W, 2.0)
            w[p + "mix.g"], w[p + "mix.o"] = lin(H * V, W, 2.0), lin(W, H * V)
        elif layer["type"] == "attention":
            H, G, D = m["heads"], m["kv_heads"], m["dim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.o"] = lin(H * D, W), lin(G * D, W, 2.0), lin(W, H * D)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = (1 + rnd(D, std=0.2)) * sharp, 1 + rnd(D, std=0.2)
        else:
            L, R = m["left"], m["right"]
            H, G, D, V = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
            q = p + "mix.left."
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * D, W, 2.0) * sharp, lin(G * D, W, 2.0), lin(G * V, W)
            w[q + "q.b"], w[q + "k.b"], w[q + "v.b"] = rnd(H * D, std=0.3) * sharp, rnd(G * D, std=0.3), rnd(G * V, std=0.3)
            w[q + "g"], w[q + "o"] = lin(H * V, W, 2.0), lin(W, H * V)
            H, G, D, V, taps = R["heads"], R["kv_heads"], R["dim"], R["vdim"], R["conv"]
            ra, rg = R["decay_rank"], R["gate_rank"]
            r = p + "mix.right."
            w[r + "q"], w[r + "k"], w[r + "v"] = lin(G * D, W, 2.0), lin(G * D, W, 2.0), lin(H * V, W, 2.0)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * V)):
                w[r + f"{n}.conv"] = rnd(c, taps, std=0.6)
            w[r + "b"], w[r + "a1"], w[r + "a2"] = lin(H, W, 2.0), lin(ra, W, 2.0), lin(H * D, ra, 2.0)
            w[r + "g1"], w[r + "g2"] = lin(rg, W, 2.0), lin(H * V, rg, 2.0)
            w[r + "A_log"], w[r + "dt_bias"] = rnd(H) - 1.5, rnd(H * D)               # decays from nearly 1 to well below
            w[r + "norm"], w[r + "o"] = 1 + rnd(V, std=0.2), lin(W, H * V)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            w[p + "norm2"] = 1 + rnd(W, std=0.2)
            w[p + "mlp.up"], w[p + "mlp.down"] = lin(ff, W, 1.5), lin(W, ff)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write_model(folder, cfg: dict, weights: dict[str, torch.Tensor], name_ranks: bool = True):
    """A model folder.  name_ranks=False leaves the ranks of the low-rank maps out of config.json: the engine then has
    them from the shapes of the checkpoint's tensors."""
    from lucciola_b200.weights.safetensors_io import write_safetensors
    folder.mkdir(parents=True, exist_ok=True)
    cfg = json.loads(json.dumps(cfg))
    if not name_ranks:
        for layer in cfg["layers"]:
            if layer["type"] == "parallel":
                del layer["mixer"]["right"]["decay_rank"], layer["mixer"]["right"]["gate_rank"]
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
        _plain[k] = PlainVenitar(cfg, weights).forward(ids)
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
    holds: plain_venitar.ROUND) and nothing else."""
    import plain_venitar as plain
    exact = PlainVenitar(cfg, weights).forward(ids)
    try:
        plain.ROUND = lambda x: x.to(torch.bfloat16).to(torch.float64)
        rounded = PlainVenitar(cfg, weights).forward(ids)
    finally:
        plain.ROUND = None
    return ((rounded - exact).abs().max() / exact.abs().max()).item()


_rounding: dict = {}


def bound(dtype: str, cfg: dict, weights: dict, reqs: dict, base: float | None = None) -> dict:
    """The bound of a comparison, request by request: the type's own, or for bfloat16 three times what rounding alone
    does to this model on that request if that is more."""
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


def random_config(seed: int) -> dict:
    """A configuration whose every size is drawn: widths, the number and order of layers, the loop, head counts and
    groupings, sizes that are no multiples of 4 or 8, values larger and smaller than keys, windows and chunks from one
    token to longer than the sequences, taps from 1 to 5, ranks, layers without feed-forward, YaRN or not."""
    rng = random.Random(seed)
    width = rng.choice([24, 36, 40, 64, 72, 100, 128, 200])
    layers = []
    for _ in range(rng.randint(1, 4)):
        ff = rng.choice([None, 24, 64, 100, 128, 192])
        kind = rng.choice(["retention", "attention", "parallel"])
        dim = rng.choice([4, 8, 10, 16, 24, 64, 130])
        rot = _rot(rng.choice([0, 2, dim // 2 * 2, dim // 4 * 2]), rng.choice([100.0, 10000.0, 1e6]))
        if kind == "retention":
            heads = rng.choice([1, 2, 3, 5])
            layers.append(_retention(heads, dim, rng.choice([3, 8, 20, 32, 40, 70]), [rng.choice([0.5, 0.9, 0.99, 0.9995]) for _ in range(heads)], rot, ff))
        elif kind == "attention":
            kv = rng.choice([1, 2, 3])
            layers.append(_attention(kv * rng.choice([1, 2, 4]), kv, min(dim, 64), rng.choice([0.1, 0.2, 0.3]), _rot(min(rot["dims"], min(dim, 64) // 2 * 2), rot["base"]),
                                     rng.choice([1, 2, 7, 16, 33, 64, 150, 500]), ff))
        else:
            kv = rng.choice([1, 2, 3])
            ldim = min(dim, 64)
            lrot = _rot(min(rot["dims"], ldim // 2 * 2), rot["base"], rng.choice([None, (rng.choice([1.5, 4.0, 16.0]), rng.choice([16, 64, 300]), rng.choice([4.0, 32.0]), rng.choice([0.5, 1.0]))]))
            left = _left(kv * rng.choice([1, 2, 4]), kv, ldim, rng.choice([4, 8, 12, 20, 32, 72]), rng.choice([0.1, 0.2, 0.3]), lrot,
                         rng.choice([1, 2, 7, 16, 33, 64, 150, 500]))
            rkv = rng.choice([1, 2, 3])
            right = _right(rkv * rng.choice([1, 2]), rkv, rng.choice([4, 10, 16, 33, 64, 130]), rng.choice([3, 8, 20, 32, 40, 70]), rng.randint(1, 5),
                           rng.choice([1, 3, 8, 24]), rng.choice([1, 2, 8, 16]))
            layers.append(_pair(left, right, rng.choice([0.5, 1.0, 1.5]), rng.choice([0.5, 1.0, 1.5]), ff))
    start = rng.randint(0, len(layers))
    stop = rng.randint(start, len(layers))
    return _config(rng.choice([64, 97, 300]), width, rng.choice([1e-5, 1e-6]), rng.choice([0.5, 1.0, 3.0]), (start, stop, rng.randint(1, 3)), layers)
