"""The Nelovik decoder, plainly: one slow function per mechanism, on the CPU, in float64 unless told otherwise.

This file is what the engine's kernels are compared with.  It shares no code with the package: it takes a
configuration as the dictionary of config.json and the weights as a dictionary of tensors by checkpoint name,
and runs one sequence at a time, either whole or in portions with an explicit state.

Notation.  x: residual stream [T, width].  A layer computes x <- x + mixer(n1(x)) + ff(n2(x)) with two RMS norms of the
same x.  Linear weights are [out, in].  Every function that keeps something of the past takes it as `past` (None at a
sequence's start) and returns what the next call needs.
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


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    """z > 0: sp(p) z^2 + z / 2;  z <= 0: (1/2 + sp(q)) (e^z - 1 - z) + z / 2;  sp = softplus."""
    ap = math.log1p(math.exp(p))
    an = 0.5 + math.log1p(math.exp(q))
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(z) - z) + 0.5 * z)


def short_conv(x: torch.Tensor, w: torch.Tensor, bias, past):
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
    if bias is not None:
        y = y + bias
    return y, full[full.shape[0] - (taps - 1):]


def gated_delta_rule(h: torch.Tensor, w: dict, m: dict, eps: float, past):
    """The gated delta rule with convolved, unit-length queries and keys.  w: q, k, v, q.conv, k.conv, v.conv, b, a,
    A_log, dt_bias, g, norm, o.  past: (conv inputs of q, k, v, state [heads, dim, vdim]) or None."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    h = _r(h)
    cq, ck, cv, S = past if past is not None else (None, None, None, torch.zeros(H, D, V, dtype=h.dtype))
    q, cq = short_conv(h @ w["q"].T, w["q.conv"], None, cq)
    k, ck = short_conv(h @ w["k"].T, w["k.conv"], None, ck)
    v, cv = short_conv(h @ w["v"].T, w["v.conv"], None, cv)
    q, k, v = silu(q).reshape(T, G, D), silu(k).reshape(T, G, D), silu(v).reshape(T, H, V)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)                                              # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))   # [T, H]
    S = S.clone()
    o = torch.zeros(T, H, V, dtype=h.dtype)
    per = H // G
    for t in range(T):
        for hd in range(H):
            kk, qq = k[t, hd // per], q[t, hd // per]
            S[hd] = decay[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ kk)
            S[hd] = S[hd] + torch.outer(kk, u)
            o[t, hd] = S[hd].T @ qq
    o = rms_norm(o, w["norm"], eps) * silu(h @ w["g"].T).reshape(T, H, V)
    return _r(o.reshape(T, H * V)) @ w["o"].T, (cq, ck, cv, S)


def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, dim]: entry i < dims/2 is paired with entry i + dims/2 and the pair turned by p * base^(-2i/dims)."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)
    a = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :].to(x.dtype), torch.sin(a)[:, None, :].to(x.dtype)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def pooled_window_attention(h: torch.Tensor, w: dict, m: dict, eps: float, past):
    """Softmax attention over the last `size` tokens and over one mean key and value for every block of `pool` tokens
    that lies wholly before them, with a capped score and a sink in the denominator.  w: q, q.b, k, k.b, v, v.b, q.norm,
    k.norm, sink, o.  past: (keys [n, kv_heads, dim] as the cache holds them, values [n, kv_heads, vdim]) or None."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, P = m["mask"]["size"], m["mask"]["pool"]
    T = h.shape[0]
    start = 0 if past is None else past[0].shape[0]
    pos = torch.arange(start, start + T)
    h = _r(h)
    q = rms_norm(h @ w["q"].T + w["q.b"], w["q.norm"], eps).reshape(T, H, D)
    k = rms_norm(h @ w["k"].T + w["k.b"], w["k.norm"], eps).reshape(T, G, D)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, V)
    q = rotate_half(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half(k, pos, m["rot"]["dims"], m["rot"]["base"])
    q, k, v = _r(q), _r(k), _r(v)                               # as the cache holds them
    if past is not None:
        k, v = torch.cat([past[0], k], dim=0), torch.cat([past[1], v], dim=0)
    cap = m["softcap"]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    per = H // G
    for t in range(T):
        i = start + t
        lo = max(0, i - size + 1)                               # 0 <= i - j < size
        nb = max(0, (i - size + 1) // P)                        # blocks whose last token is at most i - size
        for hd in range(H):
            g = hd // per
            keys = torch.cat([k[:nb * P, g].reshape(nb, P, D).mean(dim=1), k[lo:i + 1, g]], dim=0)
            vals = torch.cat([v[:nb * P, g].reshape(nb, P, V).mean(dim=1), v[lo:i + 1, g]], dim=0)
            s = (keys @ q[t, hd]) * m["scale"]
            s = cap * torch.tanh(s / cap)
            mx = torch.maximum(s.max(), w["sink"][hd])
            e = torch.exp(s - mx)
            out[t, hd] = (e[:, None] * vals).sum(dim=0) / (e.sum() + torch.exp(w["sink"][hd] - mx))
    return _r(out.reshape(T, H * V)) @ w["o"].T, (k, v)


def mamba2(h: torch.Tensor, w: dict, m: dict, eps: float, past):
    """The selective state space of Mamba-2.  w: in, conv, conv.b, dt_bias, A_log, D, norm, o.  past: (conv inputs,
    state [heads, N, vdim]) or None."""
    H, V, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * V
    T = h.shape[0]
    conv_in, S = past if past is not None else (None, torch.zeros(H, N, V, dtype=h.dtype))
    zxbcdt = _r(h) @ w["in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc, conv_in = short_conv(xbc, w["conv"], w["conv.b"], conv_in)
    xbc = silu(xbc)
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])                                                # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)
    S = S.clone()
    y = torch.zeros(T, H, V, dtype=h.dtype)
    per = H // G
    for t in range(T):
        for hd in range(H):
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, hd // per], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, hd // per] + w["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = (rms_norm(y.reshape(T, NG, inner // NG), None, eps)).reshape(T, inner) * w["norm"]
    return _r(y) @ w["o"].T, (conv_in, S)


def side_by_side(h: torch.Tensor, w: dict, m: dict, eps: float, past):
    """Half the sum of attention and state space, each normed over the model width first.  w holds both mixers' tensors
    under 'left.' and 'right.' and the two norm weights 'left.out', 'right.out'."""
    sub = lambda p: {k[len(p):]: v for k, v in w.items() if k.startswith(p)}
    pl, pr = past if past is not None else (None, None)
    a, pl = pooled_window_attention(h, sub("left."), m["left"], eps, pl)
    b, pr = mamba2(h, sub("right."), m["right"], eps, pr)
    return 0.5 * (rms_norm(a, w["left.out"], eps) + rms_norm(b, w["right.out"], eps)), (pl, pr)


def dense_feed_forward(h: torch.Tensor, w: dict) -> torch.Tensor:
    """down( xielu(up h) ); w: up, down, act = (p, q)."""
    return _r(xielu(_r(_r(h) @ w["up"].T), float(w["act"][0]), float(w["act"][1]))) @ w["down"].T


MIXERS = {"delta": gated_delta_rule, "delta_2": gated_delta_rule, "parallel": side_by_side}


class PlainNelovik:
    def __init__(self, cfg: dict, weights: dict, dtype=torch.float64):
        self.cfg = cfg
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
        self.dtype = dtype

    def _sub(self, prefix: str) -> dict:
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def run(self, ids, past=None, layers_out: list | None = None):
        """Logits [T, vocab] of the tokens `ids`, which follow what `past` holds (None: a sequence's start), and the
        new past.  layers_out, if a list, receives the residual stream after every layer."""
        eps = self.cfg["norm"]["eps"]
        x = self.w["embed"][torch.as_tensor(ids, dtype=torch.long)]
        past = past if past is not None else [None] * len(self.cfg["layers"])
        new_past = []
        for i, layer in enumerate(self.cfg["layers"]):
            p = f"l{i}."
            a, state = MIXERS[layer["type"]](rms_norm(x, self.w[p + "norm1"], eps), self._sub(p + "mix."), layer["mixer"], eps, past[i])
            new_past.append(state)
            if layer.get("mlp") is not None:
                a = a + dense_feed_forward(rms_norm(x, self.w[p + "norm2"], eps), self._sub(p + "mlp."))
            x = x + a
            if layers_out is not None:
                layers_out.append(x.clone())
        return _r(rms_norm(x, self.w["final.norm"], eps)) @ self.w["head"].T, new_past

    def forward(self, ids, layers_out: list | None = None) -> torch.Tensor:
        return self.run(ids, None, layers_out)[0]
