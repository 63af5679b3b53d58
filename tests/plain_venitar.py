"""The Venitar decoder, plainly: one slow function per mechanism, on the CPU, in float64 unless told otherwise.

This file is what the engine's kernels are compared with.  It shares no code with the package: it takes a
configuration as the dictionary of config.json and the weights as a dictionary of tensors by checkpoint name,
and runs one sequence at a time, either whole or in portions with an explicit state.

Notation.  x: residual stream [T, width].  A layer computes x <- x + mixer(n1(x)) and then, if it has a feed-forward,
x <- x + ff(n2(x)).  Linear weights are [out, in].  Every function that keeps something of the past takes it as `past`
(None at a sequence's start) and returns what the next call needs.  Layers `loop.start .. loop.stop - 1` run
`loop.times` times in a row with the same weights and a past of their own for every pass; before every pass but the
first the embedding's output is added to x.
"""
from __future__ import annotations

import math

import torch


# Where an engine that serves in 16 bits may round: the inputs of products and what a cache holds.  None: nowhere (this
# file's own arithmetic is exact to its type); the tests set it to see what such rounding alone does to a model's logits.
ROUND = None


def _r(x: torch.Tensor) -> torch.Tensor:
    return x if ROUND is None else ROUND(x)


def rms_norm(x: torch.Tensor, weight, eps: float) -> torch.Tensor:
    y = x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(z, torch.zeros_like(z))


def rotary_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """The dims / 2 frequencies of a rotation and the factor on its sines and cosines.  Without `scaling` they are
    base^(-2i/dims) and 1.  With it (YaRN): slow frequencies are divided by `factor`, fast ones kept, with a linear ramp
    between the pair indices at which `original` positions make `fast` and `slow` turns."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0
    turns_at = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turns_at(sc["fast"])), 0)
    hi = min(math.ceil(turns_at(sc["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, dim]: entry i < dims/2 is paired with entry i + dims/2 and the pair turned by p * f_i; entries from
    dims on pass unchanged."""
    dims = rot["dims"]
    if dims == 0:
        return x
    half = dims // 2
    f, mag = rotary_frequencies(rot)
    a = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :].to(x.dtype), (torch.sin(a) * mag)[:, None, :].to(x.dtype)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def short_conv(x: torch.Tensor, w: torch.Tensor, past):
    """Causal convolution over time, one filter a channel.  x [T, C], w [C, taps] whose last column weighs the current
    token, zeros before the start; past [taps - 1, C] are the inputs before x.  Returns (y, the last taps - 1 inputs)."""
    taps = w.shape[1]
    if past is None:
        past = torch.zeros(taps - 1, x.shape[1], dtype=x.dtype)
    full = torch.cat([past, x], dim=0)
    T = x.shape[0]
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + full[j:j + T] * w[:, j]
    return y, full[full.shape[0] - (taps - 1):]


def retention(h: torch.Tensor, w: dict, m: dict, eps: float, past):
    """Linear attention with one fixed decay a head, no softmax and no denominator, on rotated q and k.
    w: q, k, v, g, o.  past: (tokens seen, state [heads, dim, vdim]) or None."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    start, S = past if past is not None else (0, torch.zeros(H, D, V, dtype=h.dtype))
    pos = torch.arange(start, start + T)
    h = _r(h)
    q = rotate_half((h @ w["q"].T).reshape(T, H, D), pos, m["rot"])
    k = rotate_half((h @ w["k"].T).reshape(T, H, D), pos, m["rot"]) * D ** -0.5
    v = (h @ w["v"].T).reshape(T, H, V)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = S.clone()
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t, :, :, None] * v[t, :, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, None, eps).reshape(T, H * V) * silu(h @ w["g"].T)
    return _r(o) @ w["o"].T, (start + T, S)


def softmax_attention(q, k, v, start: int, scale: float, lo_of, sink: bool):
    """q [T, H, D] at positions start .. start + T - 1 over keys k [n, G, D] and values v [n, G, V] at positions 0 ..
    n - 1.  Position i sees the keys lo_of(i) .. i.  With `sink`, one more term of score 0 and no value stands in the
    denominator."""
    T, H, _ = q.shape
    G, V = k.shape[1], v.shape[2]
    per = H // G
    out = torch.zeros(T, H, V, dtype=q.dtype)
    for t in range(T):
        i = start + t
        lo = lo_of(i)
        for hd in range(H):
            g = hd // per
            s = (k[lo:i + 1, g] @ q[t, hd]) * scale
            mx = s.max().clamp(min=0.0) if sink else s.max()
            e = torch.exp(s - mx)
            den = e.sum() + (torch.exp(-mx) if sink else 0.0)
            out[t, hd] = (e[:, None] * v[lo:i + 1, g]).sum(dim=0) / den
    return out


def chunked_attention(h: torch.Tensor, w: dict, m: dict, eps: float, past):
    """Softmax attention inside chunks of mask.size positions counted from the sequence's start, whose values are the
    keys as projected (before their norm and rotation), with per-head norms of q and k and a sink of score 0.
    w: q, k, q.norm, k.norm, o.  past: (keys as the cache holds them [n, G, D], values [n, G, D]) or None."""
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    C = m["mask"]["size"]
    T = h.shape[0]
    start = 0 if past is None else past[0].shape[0]
    pos = torch.arange(start, start + T)
    h = _r(h)
    q = (h @ w["q"].T).reshape(T, H, D)
    v = (h @ w["k"].T).reshape(T, G, D)
    k = rotate_half(rms_norm(v, w["k.norm"], eps), pos, m["rot"])
    q = rotate_half(rms_norm(q, w["q.norm"], eps), pos, m["rot"])
    q, k, v = _r(q), _r(k), _r(v)
    if past is not None:
        k, v = torch.cat([past[0], k], dim=0), torch.cat([past[1], v], dim=0)
    out = softmax_attention(q, k, v, start, m["scale"], lambda i: (i // C) * C, sink=True)
    return _r(out.reshape(T, -1)) @ w["o"].T, (k, v)


def window_attention(h: torch.Tensor, w: dict, m: dict, past):
    """Softmax attention over the last mask.size tokens with biases on q, k and v, rotation (optionally with YaRN
    scaling) and an elementwise sigmoid gate on the heads.  w: q, q.b, k, k.b, v, v.b, g, o.  past: (keys, values) or None."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = m["mask"]["size"]
    T = h.shape[0]
    start = 0 if past is None else past[0].shape[0]
    pos = torch.arange(start, start + T)
    h = _r(h)
    q = rotate_half((h @ w["q"].T + w["q.b"]).reshape(T, H, D), pos, m["rot"])
    k = rotate_half((h @ w["k"].T + w["k.b"]).reshape(T, G, D), pos, m["rot"])
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, V)
    q, k, v = _r(q), _r(k), _r(v)
    if past is not None:
        k, v = torch.cat([past[0], k], dim=0), torch.cat([past[1], v], dim=0)
    out = softmax_attention(q, k, v, start, m["scale"], lambda i: max(0, i - size + 1), sink=False)
    out = out.reshape(T, H * V) * torch.sigmoid(h @ w["g"].T)
    return _r(out) @ w["o"].T, (k, v)


def channel_delta_rule(h: torch.Tensor, w: dict, m: dict, eps: float, past):
    """The gated delta rule with a decay for every key channel, through two maps of low rank, and an output gate of low
    rank.  w: q, k, v, q.conv, k.conv, v.conv, b, a1, a2, A_log, dt_bias, g1, g2, norm, o.  past: (conv inputs of q, k, v,
    state [heads, dim, vdim]) or None."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    h = _r(h)
    cq, ck, cv, S = past if past is not None else (None, None, None, torch.zeros(H, D, V, dtype=h.dtype))
    q, cq = short_conv(h @ w["q"].T, w["q.conv"], cq)
    k, ck = short_conv(h @ w["k"].T, w["k.conv"], ck)
    v, cv = short_conv(h @ w["v"].T, w["v.conv"], cv)
    q, k, v = silu(q).reshape(T, G, D), silu(k).reshape(T, G, D), silu(v).reshape(T, H, V)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)                                                          # [T, H]
    step = softplus(_r(h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).reshape(T, H, D)
    decay = torch.exp(-torch.exp(w["A_log"])[None, :, None] * step)                             # [T, H, D]
    S = S.clone()
    o = torch.zeros(T, H, V, dtype=h.dtype)
    per = H // G
    for t in range(T):
        for hd in range(H):
            kk, qq = k[t, hd // per], q[t, hd // per]
            S[hd] = decay[t, hd][:, None] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ kk)
            S[hd] = S[hd] + torch.outer(kk, u)
            o[t, hd] = S[hd].T @ qq
    gate = torch.sigmoid(_r(h @ w["g1"].T) @ w["g2"].T).reshape(T, H, V)
    o = rms_norm(o, w["norm"], eps) * gate
    return _r(o.reshape(T, H * V)) @ w["o"].T, (cq, ck, cv, S)


def side_by_side(h: torch.Tensor, w: dict, m: dict, eps: float, past):
    """left_scale * window attention + right_scale * delta rule, both of the same input."""
    sub = lambda p: {k[len(p):]: v for k, v in w.items() if k.startswith(p)}
    pl, pr = past if past is not None else (None, None)
    a, pl = window_attention(h, sub("left."), m["left"], pl)
    b, pr = channel_delta_rule(h, sub("right."), m["right"], eps, pr)
    return m["left_scale"] * a + m["right_scale"] * b, (pl, pr)


def dense_feed_forward(h: torch.Tensor, w: dict) -> torch.Tensor:
    """down( relu(up h)^2 ); w: up, down."""
    return _r(torch.relu(_r(_r(h) @ w["up"].T)).pow(2)) @ w["down"].T


def mixer(kind: str, h, w, m, eps, past):
    if kind == "retention":
        return retention(h, w, m, eps, past)
    if kind == "attention":
        return chunked_attention(h, w, m, eps, past)
    if kind == "parallel":
        return side_by_side(h, w, m, eps, past)
    raise ValueError(f"unknown layer type {kind!r}")


def layer_runs(cfg: dict) -> list[tuple[int, bool]]:
    """The layers in the order they run: (layer, whether the embedding's output is added before it)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for p in range(times):
        runs += [(i, p > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


class PlainVenitar:
    def __init__(self, cfg: dict, weights: dict, dtype=torch.float64):
        self.cfg = cfg
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
        self.dtype = dtype
        self.runs = layer_runs(cfg)

    def _sub(self, prefix: str) -> dict:
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def run(self, ids, past=None, layers_out: list | None = None):
        """Logits [T, vocab] of the tokens `ids`, which follow what `past` holds (None: a sequence's start), and the
        new past (one entry for every layer run).  layers_out, if a list, receives the residual stream after every run."""
        eps = self.cfg["norm"]["eps"]
        e = self.w["embed"][torch.as_tensor(ids, dtype=torch.long)] * self.cfg["embedding"]["scale"]
        x = e.clone()
        past = past if past is not None else [None] * len(self.runs)
        new_past = []
        for r, (i, add) in enumerate(self.runs):
            layer, p = self.cfg["layers"][i], f"l{i}."
            if add:
                x = x + e
            a, state = mixer(layer["type"], rms_norm(x, self.w[p + "norm1"], eps), self._sub(p + "mix."), layer["mixer"], eps, past[r])
            new_past.append(state)
            x = x + a
            if layer.get("mlp") is not None:
                x = x + dense_feed_forward(rms_norm(x, self.w[p + "norm2"], eps), self._sub(p + "mlp."))
            if layers_out is not None:
                layers_out.append(x.clone())
        return _r(rms_norm(x, self.w["final.norm"], eps)) @ self.w["embed"].T, new_past

    def forward(self, ids, layers_out: list | None = None) -> torch.Tensor:
        return self.run(ids, None, layers_out)[0]
