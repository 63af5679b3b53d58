"""Dense gated feed-forward: down( act(gate(h)) * up(h) ), act = silu (src/qwen.cc:762-794,
src/kernels/swiglu.cu:30-36 of lucciola), relu, the tanh form of gelu, or a clamped swish with its limit (ops.GATE_ACTS).  gate and up are one product over the stacked weights; on
the bfloat16 path, when the intermediate size is a multiple of 64, their rows are interleaved in blocks of 64
and act(gate) * up is formed in that product's epilogue, so the [T, 2 * intermediate] matrix is never written.

GatedFeedForward takes the three tensor names and the activation; SwiGLUFeedForward is the silu one with the
tensor names of the Qwen3 checkpoints."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from .base import FeedForward, NormSink, Part, RowScaled, Runtime, StepContext
from .linear import Linear


class GatedFeedForward(FeedForward):
    recordable = True

    def __init__(self, rt: Runtime, gate_name: str, up_name: str, down_name: str, hidden_size: int, intermediate_size: int,
                 act: str = "silu", limit: float = 0.0, out_dtype: Optional[torch.dtype] = None):
        if act not in ops.GATE_ACTS:
            raise ValueError(f"activation {act!r} of a gated feed-forward is not one of {sorted(ops.GATE_ACTS)}")
        self.rt, self.act, self.limit = rt, act, float(limit)
        self.out_dtype = out_dtype          # type of the down product's output (None: the activation type)
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_up = Linear(rt, [gate_name, up_name], hidden_size, [intermediate_size, intermediate_size])
        self.down = Linear(rt, down_name, intermediate_size, hidden_size)
        self.fused = False

    def children(self) -> list[Part]:
        return [self.gate_up, self.down]

    def bind_all(self, get) -> None:
        super().bind_all(get)
        w = self.gate_up.weight
        self.fused = (self.rt.fast_kernels and w.is_cuda and w.dtype == torch.bfloat16 and self.intermediate_size % 64 == 0
                      and self.hidden_size % 8 == 0)
        if self.fused:
            inter = self.intermediate_size
            self.gate_up.weight = ops.interleave_gate_up(w[:inter], w[inter:])

    accepts_sink = True

    def row_scaled_ok(self, num_tokens: int) -> bool:
        """The products with the activation in their epilogue also apply a row's norm factor there."""
        return self.fused

    def _down(self, act: torch.Tensor, sink: Optional[NormSink]):
        if sink is not None and self.out_dtype is None and self.down.sink_ok(act):
            return self.down.forward_into(act, sink)
        return self.down.forward(act, out_dtype=self.out_dtype)

    def forward(self, h, step: StepContext, sink: Optional[NormSink] = None):
        inter = self.intermediate_size
        if isinstance(h, RowScaled):
            if not self.row_scaled_ok(h.shape[0]):
                raise ops.KernelError("this feed-forward was handed rows without their norm factor for a step it cannot take them in")
            act = self.rt.empty((h.shape[0], inter))
            ops.gemm_tcgen05(act, h.x, self.gate_up.weight, self.rt.stream, swiglu=True, sumsq=h.sumsq, eps=h.eps, act=self.act, limit=self.limit)
            return self._down(act, sink)
        if self.fused and ops.gemm_tcgen05_ok(h, h, self.gate_up.weight):
            act = self.rt.empty((h.shape[0], inter))
            ops.gemm_tcgen05(act, h, self.gate_up.weight, self.rt.stream, swiglu=True, act=self.act, limit=self.limit)
            return self._down(act, sink)
        if self.fused:
            raise ops.KernelError("the interleaved gate|up weights need the tensor-core product (bfloat16, 16-byte aligned input)")
        gu = self.gate_up.forward(h)
        act = self.rt.empty((h.shape[0], inter))
        ops.swiglu(act, gu[:, :inter], gu[:, inter:], self.rt.stream, act=self.act, limit=self.limit)
        return self._down(act, sink)


class SwiGLUFeedForward(GatedFeedForward):
    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, intermediate_size: int):
        super().__init__(rt, f"{prefix}.gate_proj.weight", f"{prefix}.up_proj.weight", f"{prefix}.down_proj.weight",
                         hidden_size, intermediate_size, "silu")


class DenseFeedForward(FeedForward):
    """A feed-forward without a gate: down( act(up(h)) ).  `act` is one of ops.PLAIN_ACTS ("relu2" is relu(z)^2); xIELU,

        z > 0: softplus(p) z^2 + z / 2        z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2,

    takes its two learned numbers (p, q) from the tensor `act_name` [2]; the two positive factors are formed once, when
    the weights are bound."""
    recordable = True

    def __init__(self, rt: Runtime, up_name: str, down_name: str, hidden_size: int, intermediate_size: int, act: str = "xielu",
                 act_name: Optional[str] = None, out_dtype: Optional[torch.dtype] = None):
        if act not in ops.PLAIN_ACTS:
            raise ValueError(f"activation {act!r} of a dense feed-forward is not one of {sorted(ops.PLAIN_ACTS)}")
        if (act == "xielu") != (act_name is not None):
            raise ValueError("xielu, and only xielu, takes a tensor with its two numbers")
        self.rt, self.act, self.act_name, self.out_dtype = rt, act, act_name, out_dtype
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.up = Linear(rt, up_name, hidden_size, intermediate_size)
        self.down = Linear(rt, down_name, intermediate_size, hidden_size)
        self.p0 = self.p1 = 0.0

    def children(self) -> list[Part]:
        return [self.up, self.down]

    def param_specs(self):
        from .base import ParamSpec
        return [ParamSpec(self.act_name, (2,), "linear")] if self.act_name is not None else []

    def bind(self, get) -> None:
        if self.act_name is not None:
            p, q = get(self.act_name).to(torch.float64).cpu().tolist()
            sp = lambda x: max(x, 0.0) + math.log1p(math.exp(-abs(x)))
            self.p0, self.p1 = sp(p), 0.5 + sp(q)

    def forward(self, h, step: StepContext):
        u = self.up.forward(h)
        a = self.rt.empty(u.shape)
        ops.activation(a, u, self.act, self.rt.stream, self.p0, self.p1)
        return self.down.forward(a, out_dtype=self.out_dtype)
