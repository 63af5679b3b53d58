"""The selective state space of Mamba-2.  With inner = heads * vdim, N = state, G = groups, the input product is laid out
[z: inner | x: inner | B: G N | C: G N | dt: heads]; x, B and C together pass a short causal convolution (with a bias)
and silu.  Per head (head h uses group h / (heads / G)), with a 32-bit state S [N, vdim]:

    dt <- softplus(dt + dt_bias)                       (no clamp)
    S <- exp(-exp(A_log) dt) S + B (dt x)^T            y = S^T C + D x
    out = W_o ( rmsnorm_parts(y * silu(z)) * w )       (the gate comes BEFORE the norm; norm_groups equal parts of the row)

The state and the last taps - 1 inputs of the convolution are all this mixer keeps of the past.  The recurrence is the
kernel of the gated delta rule without the delta rule's correction (csrc/state_recurrence.cu); everything between the
two products is computed in 32-bit.

Beside forward(), the mixer offers its steps apart (in_names / in_sizes, inner, `o`).
"""
from __future__ import annotations

from typing import Callable

import torch

from .. import ops
from .base import Mixer, ParamSpec, Part, Runtime, StateSlot, StepContext
from .linear import Linear
from .short_conv import ShortConv


class SelectiveStateSpace(Mixer):
    recordable = True

    def __init__(self, rt: Runtime, prefix: str, width: int, heads: int, vdim: int, state: int, groups: int, norm_groups: int,
                 taps: int, eps: float):
        if heads % groups or (heads * vdim) % norm_groups:
            raise ValueError(f"{heads} heads of {vdim} do not fit {groups} groups and {norm_groups} norm groups")
        self.rt, self.prefix, self.width = rt, prefix, width
        self.heads, self.vdim, self.state, self.groups, self.norm_groups, self.eps = heads, vdim, state, groups, norm_groups, float(eps)
        self.inner_size = heads * vdim
        self.bc_size = groups * state
        self.proj = Linear(rt, self.in_names(), width, self.in_sizes())
        self.conv = ShortConv(rt, f"{prefix}.conv", self.inner_size + 2 * self.bc_size, taps, bias_name=f"{prefix}.conv.b")
        self.o = Linear(rt, f"{prefix}.o", self.inner_size, width)
        self.A_log = self.dt_bias = self.D = self.norm_w = None

    def in_names(self) -> list[str]:
        return [f"{self.prefix}.in"]

    def in_sizes(self) -> list[int]:
        return [2 * self.inner_size + 2 * self.bc_size + self.heads]

    def children(self) -> list[Part]:
        return [self.proj, self.conv, self.o]

    def param_specs(self) -> list[ParamSpec]:
        p = self.prefix
        return [ParamSpec(f"{p}.A_log", (self.heads,), "linear"), ParamSpec(f"{p}.dt_bias", (self.heads,), "linear"),
                ParamSpec(f"{p}.D", (self.heads,), "norm"), ParamSpec(f"{p}.norm", (self.inner_size,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        p = self.prefix
        self.A_log = get(f"{p}.A_log").to(torch.float32).contiguous()
        self.dt_bias = get(f"{p}.dt_bias").to(torch.float32).contiguous()
        self.D = get(f"{p}.D").to(torch.float32).contiguous()
        self.norm_w = get(f"{p}.norm").to(torch.float32).contiguous()

    def cache_request(self) -> tuple:
        state = StateSlot((self.heads, self.state, self.vdim), torch.float32)
        conv = self.conv.cache_request()
        return (conv, state) if conv is not None else (state,)

    def inner(self, pre: torch.Tensor, step: StepContext, cache: tuple, out: torch.Tensor, out_scale: float = 1.0,
              write_cache: bool = True) -> None:
        """pre: float32 [T, >= in_sizes()[0]], the columns z | x | B | C | dt; out: [T, inner_size] in the activation type
        receives the gated, normed heads times out_scale."""
        if not write_cache:
            raise ops.KernelError("a recurrent mixer has no cache another call could have written")
        rt, m, bc = self.rt, self.inner_size, self.bc_size
        conv_cache, state = (cache[0], cache[1]) if len(cache) == 2 else (None, cache[0])
        xbc = self.conv.forward(pre[:, m:2 * m + 2 * bc], step, conv_cache)
        y = rt.empty((pre.shape[0], m), torch.float32)
        dt0 = 2 * m + 2 * bc
        ops.state_recurrence(xbc[:, m + bc:], xbc[:, m:m + bc], xbc[:, :m], pre[:, dt0:dt0 + self.heads], None, self.A_log,
                             self.dt_bias, self.D, state.state, y, step, self.heads, self.groups, self.state, self.vdim, rt.stream,
                             delta=False, by_shape=rt.fast_kernels)
        ops.gated_group_norm(out, y, pre[:, :m], self.norm_w, self.norm_groups, self.eps, rt.stream, gate_first=True, act="silu",
                             scale=out_scale)

    def forward(self, h: torch.Tensor, step: StepContext, cache: tuple, write_cache: bool = True) -> torch.Tensor:
        pre = self.proj.forward(h, out_dtype=torch.float32)
        inner = self.rt.empty((h.shape[0], self.inner_size))
        self.inner(pre, step, cache, inner, 1.0, write_cache)
        return self.o.forward(inner, out_dtype=torch.float32)
