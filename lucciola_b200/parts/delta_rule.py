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

    def __init__(self, rt: Runtime, prefix: str, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        self.rt, self.prefix, self.width = rt, prefix, width
        self.heads, self.kv_heads, self.dim, self.vdim, self.eps = heads, kv_heads, dim, vdim, float(eps)
        self.qk_size, self.inner_size = kv_heads * dim, heads * vdim
        self.proj = Linear(rt, self.in_names(), width, self.in_sizes())
        self.conv = ShortConv(rt, [f"{prefix}.q.conv", f"{prefix}.k.conv", f"{prefix}.v.conv"],
                              [self.qk_size, self.qk_size, self.inner_size], taps)
        self.o = Linear(rt, f"{prefix}.o", self.inner_size, width)
        self.A_log = self.dt_bias = self.norm_w = None

    def in_names(self) -> list[str]:
        p = self.prefix
        return [f"{p}.q", f"{p}.k", f"{p}.v", f"{p}.g", f"{p}.b", f"{p}.a"]

    def in_sizes(self) -> list[int]:
        return [self.qk_size, self.qk_size, self.inner_size, self.inner_size, self.heads, self.heads]

    def children(self) -> list[Part]:
        return [self.proj, self.conv, self.o]

    def param_specs(self) -> list[ParamSpec]:
        p = self.prefix
        return [ParamSpec(f"{p}.A_log", (self.heads,), "linear"), ParamSpec(f"{p}.dt_bias", (self.heads,), "linear"),
                ParamSpec(f"{p}.norm", (self.vdim,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        p = self.prefix
        self.A_log = get(f"{p}.A_log").to(torch.float32).contiguous()
        self.dt_bias = get(f"{p}.dt_bias").to(torch.float32).contiguous()
        self.norm_w = get(f"{p}.norm").to(torch.float32).contiguous()

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
        g0 = 2 * n + m
        o = rt.empty((pre.shape[0], m), torch.float32)
        ops.state_recurrence(qkv[:, :n], qkv[:, n:2 * n], qkv[:, 2 * n:], pre[:, g0 + m + self.heads:g0 + m + 2 * self.heads],
                             pre[:, g0 + m:g0 + m + self.heads], self.A_log, self.dt_bias, None, state.state, o, step, self.heads,
                             self.kv_heads, self.dim, self.vdim, rt.stream, delta=True, unit_norm=True, q_scale=self.dim ** -0.5,
                             unit_eps=UNIT_EPS)
        ops.gated_group_norm(out, o, pre[:, g0:g0 + m], self.norm_w, self.heads, self.eps, rt.stream, gate_first=False,
                             act="silu", scale=out_scale)

    def forward(self, h: torch.Tensor, step: StepContext, cache: tuple, write_cache: bool = True) -> torch.Tensor:
        pre = self.proj.forward(h, out_dtype=torch.float32)
        inner = self.rt.empty((h.shape[0], self.inner_size))
        self.inner(pre, step, cache, inner, 1.0, write_cache)
        return self.o.forward(inner, out_dtype=torch.float32)
