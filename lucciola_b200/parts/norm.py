"""RMSNorm with a weight: y = x * rsqrt(mean(x^2) + eps) * w, statistics and product in 32-bit
(src/kernels/rmsnorm.cu:57-97 of lucciola; eps is a literal 1e-6 there, a parameter here).

GroupRMSNorm cuts the row into equal consecutive parts with a root mean square each; with one group it is the
same function (it does not offer itself as a sink of a product's epilogue, which forms one sum a row).

LayerNorm is the centred norm with a weight and no bias, y = (x - mean) / sqrt(var + eps) * w; it can also sit BEHIND a
sublayer (add_normed), for blocks that norm what a sublayer returns."""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .. import ops
from .base import Norm, NormSink, ParamSpec, Runtime


class RMSNorm(Norm):
    recordable = True

    def __init__(self, rt: Runtime, name: str, size: int, eps: float):
        self.rt, self.name, self.size, self.eps = rt, name, size, float(eps)
        self.weight: torch.Tensor | None = None     # float32 on the device

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.size,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        # bfloat16 -> float32 is exact; the kernels read norm weights as float32.
        self.weight = get(self.name).to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return self.add_forward(x, None, out_dtype)

    def as_sink(self, residual: torch.Tensor) -> Optional[NormSink]:
        return NormSink(residual, self.weight, self.eps)

    def add_forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = self.rt.empty((n, self.size), out_dtype)
        ops.add_rmsnorm(out, residual, delta, self.weight, self.eps, self.rt.stream, rows=rows)
        return out

    def add_forward_pair(self, residual: torch.Tensor, deltas: tuple, other: Optional["RMSNorm"], out_dtype: torch.dtype):
        """residual += the deltas (none, one or two tensors); returns (this norm of the new residual, `other`'s norm of it,
        or None without `other`): two norms of one stream share the row's root mean square when their eps agree, and one
        kernel adds, norms and applies both weights."""
        if other is not None and (other.size != self.size or other.eps != self.eps):
            raise ValueError("two norms of one stream in one pass need one size and one eps")
        a = self.rt.empty(residual.shape, out_dtype)
        b = self.rt.empty(residual.shape, out_dtype) if other is not None else None
        ops.add_rmsnorm_pair(a, b, residual, tuple(deltas), self.weight, other.weight if other is not None else None, self.eps,
                             self.rt.stream)
        return a, b


class GroupRMSNorm(Norm):
    """y = concat_g( x_g / sqrt(mean(x_g^2) + eps) ) * w over `groups` equal consecutive parts x_g of the row.
    add_forward() takes one delta or a tuple of two (the outputs of sublayers that run side by side) and adds
    them to the residual stream in 32-bit."""
    recordable = True
    takes_delta_parts = True

    def __init__(self, rt: Runtime, name: str, size: int, groups: int, eps: float):
        if groups <= 0 or size % groups:
            raise ValueError(f"a row of {size} cannot be cut into {groups} equal parts")
        self.rt, self.name, self.size, self.groups, self.eps = rt, name, size, int(groups), float(eps)
        self.weight: torch.Tensor | None = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.size,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.weight = get(self.name).to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return self.add_forward(x, None, out_dtype)

    def add_forward(self, residual: torch.Tensor, delta, out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = self.rt.empty((n, self.size), out_dtype)
        deltas = delta if isinstance(delta, tuple) else (delta,)
        ops.add_group_rmsnorm(out, residual, deltas, self.weight, self.groups, self.eps, self.rt.stream, rows=rows)
        return out


class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w, no bias, in 32-bit."""
    recordable = True

    def __init__(self, rt: Runtime, name: str, size: int, eps: float):
        self.rt, self.name, self.size, self.eps = rt, name, size, float(eps)
        self.weight: torch.Tensor | None = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.size,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.weight = get(self.name).to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return self.add_forward(x, None, out_dtype)

    def add_forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if delta is not None:
            ops.add_into(residual, delta, self.rt.stream)
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = self.rt.empty((n, self.size), out_dtype)
        ops.layernorm(out, residual, self.weight, self.eps, self.rt.stream, rows=rows)
        return out

    def add_normed(self, residual: torch.Tensor, outputs, scales, mult: float, copy_dtype: Optional[torch.dtype] = None):
        """residual += mult * layernorm(sum_i scales[i] * outputs[i]) * w for one or two outputs, one kernel; the copy of
        the new residual in `copy_dtype` comes out of the same kernel."""
        if not 1 <= len(outputs) <= 2 or len(scales) != len(outputs):
            raise ValueError("a layer norm behind a sublayer takes one or two outputs, with a scale each")
        copy = self.rt.empty(residual.shape, copy_dtype) if copy_dtype is not None else None
        ops.layernorm_add(residual, outputs[0], outputs[1] if len(outputs) > 1 else None, float(scales[0]),
                          float(scales[1]) if len(outputs) > 1 else 0.0, self.weight, float(mult), self.eps, self.rt.stream, copy=copy)
        return copy
