"""The gated delta rule: linear attention that takes what its state already predicts for a key off the value before it
writes, with a decay and a write strength per head and token.  Per head, with a 32-bit state S [dim, vdim]:

    q, k, v = silu(conv(W_q x)), silu(conv(W_k x)), silu(conv(W_v x))       short causal convolutions, a filter a channel
    q <- q / sqrt(sum q^2 + 1e-6) * dim^-1/2      k <- k / sqrt(sum k^2 + 1e-6)
    w = sigmoid(W_b x)      g = exp(-exp(A_log) * softplus(W_a x + dt_bias))
    S <- g S;   u = w (v - S^T k);   S <- S + k u^T;   o = S^T q           (the read-out sees the token's own write)
    out = W_o concat_h( o / rms(o) * n * silu(W_g x)_h )                    (n [vdim], shared by the heads)

q and k come in `kv_heads` heads that heads / kv_heads value heads share.  The state and the last taps - 1 inputs of
the convolutions are all this mixer keeps of the past: prompts, portions and decoded tokens go through the same
kernels, which walk a sequence's tokens of the step in order from what the step before left.  W_q | W_k | W_v | W_g |
W_b | W_a are one product with 32-bit output; everything behind it up to the output product is computed in 32-bit.

Two variants, by constructor arguments.  `decay_rank` R > 0: a decay for every key channel instead of one a head,
g[h, d] = exp(-exp(A_log_h) * softplus((W_a2 W_a1 x)[h, d] + dt_bias[h, d])) with W_a1 [R, width], W_a2 [heads * dim, R] and
dt_bias [heads * dim]; S <- diag(g) S.  `gate_rank` R > 0: the output gate is act(W_g2 W_g1 x) with W_g1 [R, width] and
W_g2 [heads * vdim, R]; `gate_act` is "silu" or "sigmoid".  The first stages of the low-rank maps are rows of the one
input product; their second stages are ONE product over [a1 | g1] with the two second maps on a block diagonal (zeros
contribute exact zeros), fed by the first stage rounded to the activation type.

Beside forward(), the mixer offers its steps apart (in_names / in_sizes, inner, `o`), so that a mixer that runs it
beside another may stack their input products.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .. import ops
from .base import Mixer, ParamSpec, Part, Runtime, StateSlot, StepContext
from .linear import Linear
from .short_conv import ShortConv

UNIT_EPS = 1e-6          # inside the root of the unit norm of q and k


class GatedDeltaRule(Mixer):
    recordable = True

    def __init__(self, rt: Runtime, prefix: str, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 decay_rank: int = 0, gate_rank: int = 0, gate_act: str = "silu"):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        if decay_rank < 0 or gate_rank < 0 or gate_act not in ("silu", "sigmoid"):
            raise ValueError("ranks are 0 (no low-rank map) or positive; the gate passes silu or sigmoid")
        self.decay_rank, self.gate_rank, self.gate_act = int(decay_rank), int(gate_rank), gate_act
        self.rt, self.prefix, self.width = rt, prefix, width
        self.heads, self.kv_heads, self.dim, self.vdim, self.eps = heads, kv_heads, dim, vdim, float(eps)
        self.qk_size, self.inner_size = kv_heads * dim, heads * vdim
        self.proj = Linear(rt, self.in_names(), width, self.in_sizes())
        self.conv = ShortConv(rt, [f"{prefix}.q.conv", f"{prefix}.k.conv", f"{prefix}.v.conv"],
                              [self.qk_size, self.qk_size, self.inner_size], taps)
        self.o = Linear(rt, f"{prefix}.o", self.inner_size, width)
        self.A_log = self.dt_bias = self.norm_w = None
        # the second stages of the low-rank maps: [a2 0; 0 g2] over the input [a1 | g1]
        self.low_rank = self.decay_rank + self.gate_rank
        self.low_sizes = [n for n, r in ((heads * dim, self.decay_rank), (self.inner_size, self.gate_rank)) if r]
        self.low: Linear | None = Linear(rt, f"{prefix}.low", self.low_rank, sum(self.low_sizes)) if self.low_rank else None

    def in_names(self) -> list[str]:
        """q | k | v | g | b | a, where g is the gate's map (or g1, the first stage of a low-rank one) and a the decay's
        (or a1); the low-rank first stages stand last, side by side: q | k | v | [g] | b | [a] | [a1] | [g1]."""
        p = self.prefix
        names = [f"{p}.q", f"{p}.k", f"{p}.v"]
        if not self.gate_rank:
            names.append(f"{p}.g")
        names.append(f"{p}.b")
        if not self.decay_rank:
            names.append(f"{p}.a")
        else:
            names.append(f"{p}.a1")
        if self.gate_rank:
            names.append(f"{p}.g1")
        return names

    def in_sizes(self) -> list[int]:
        sizes = [self.qk_size, self.qk_size, self.inner_size]
        if not self.gate_rank:
            sizes.append(self.inner_size)
        sizes.append(self.heads)
        sizes.append(self.decay_rank or self.heads)
        if self.gate_rank:
            sizes.append(self.gate_rank)
        return sizes

    def children(self) -> list[Part]:
        # the second-stage product owns no checkpoint tensor: this part binds it from a2 and g2
        return [self.proj, self.conv, self.o]

    def param_specs(self) -> list[ParamSpec]:
        p = self.prefix
        specs = [ParamSpec(f"{p}.A_log", (self.heads,), "linear"),
                 ParamSpec(f"{p}.dt_bias", (self.heads * self.dim if self.decay_rank else self.heads,), "linear"),
                 ParamSpec(f"{p}.norm", (self.vdim,), "norm")]
        if self.decay_rank:
            specs.append(ParamSpec(f"{p}.a2", (self.heads * self.dim, self.decay_rank), "linear"))
        if self.gate_rank:
            specs.append(ParamSpec(f"{p}.g2", (self.inner_size, self.gate_rank), "linear"))
        return specs

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        p = self.prefix
        self.A_log = get(f"{p}.A_log").to(torch.float32).contiguous()
        self.dt_bias = get(f"{p}.dt_bias").to(torch.float32).contiguous()
        self.norm_w = get(f"{p}.norm").to(torch.float32).contiguous()
        if self.low is not None:
            seconds = [get(f"{p}.{n}") for n, r in (("a2", self.decay_rank), ("g2", self.gate_rank)) if r]
            w = torch.zeros((sum(self.low_sizes), self.low_rank), dtype=seconds[0].dtype, device=seconds[0].device)
            row = col = 0
            for t in seconds:
                w[row:row + t.shape[0], col:col + t.shape[1]] = t
                row, col = row + t.shape[0], col + t.shape[1]
            self.low.bind_tensor(w.contiguous())

    def cache_request(self) -> tuple:
        """(the convolutions' last inputs, the state); without the first when there is one tap."""
        state = StateSlot((self.heads, self.dim, self.vdim), torch.float32)
        conv = self.conv.cache_request()
        return (conv, state) if conv is not None else (state,)

    def inner(self, pre: torch.Tensor, step: StepContext, cache: tuple, out: torch.Tensor, out_scale: float = 1.0,
              write_cache: bool = True) -> None:
        """pre: float32 [T, >= sum(in_sizes())], the columns q | k | v | g | b | a of this mixer; out: [T, inner_size] in the
        activation type receives the normed, gated heads times out_scale."""
        if not write_cache:
            raise ops.KernelError("a recurrent mixer has no cache another call could have written")
        rt, n, m = self.rt, self.qk_size, self.inner_size
        conv_cache, state = (cache[0], cache[1]) if len(cache) == 2 else (None, cache[0])
        qkv = self.conv.forward(pre[:, :2 * n + m], step, conv_cache)
        T, H = pre.shape[0], self.heads
        c = 2 * n + m                                      # columns behind q | k | v
        gate = None
        if not self.gate_rank:
            gate, c = pre[:, c:c + m], c + m
        b, c = pre[:, c:c + H], c + H
        a = None
        if not self.decay_rank:
            a, c = pre[:, c:c + H], c + H
        if self.low is not None:
            first = rt.empty((T, self.low_rank))
            ops.round_cols(first, pre[:, c:c + self.low_rank], rt.stream)
            second = self.low.forward(first, out_dtype=torch.float32)
            at = 0
            if self.decay_rank:
                a, at = second[:, :H * self.dim], H * self.dim
            if self.gate_rank:
                gate = second[:, at:at + m]
        o = rt.empty((T, m), torch.float32)
        ops.state_recurrence(qkv[:, :n], qkv[:, n:2 * n], qkv[:, 2 * n:], a, b, self.A_log, self.dt_bias, None, state.state, o, step,
                             H, self.kv_heads, self.dim, self.vdim, rt.stream, delta=True, unit_norm=True, q_scale=self.dim ** -0.5,
                             unit_eps=UNIT_EPS, rows_decay=bool(self.decay_rank), by_shape=rt.fast_kernels)
        ops.gated_group_norm(out, o, gate, self.norm_w, H, self.eps, rt.stream, gate_first=False, act=self.gate_act, scale=out_scale)

    def forward(self, h: torch.Tensor, step: StepContext, cache: tuple, write_cache: bool = True) -> torch.Tensor:
        pre = self.proj.forward(h, out_dtype=torch.float32)
        inner = self.rt.empty((h.shape[0], self.inner_size))
        self.inner(pre, step, cache, inner, 1.0, write_cache)
        return self.o.forward(inner, out_dtype=torch.float32)
