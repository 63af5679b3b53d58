"""Two mixers side by side: both read the same input, and the result is a * left(x) + b * right(x).

What each mixer keeps of the past stays its own: the pair asks for (left's cache, right's cache) and hands each its view.
Mixers that offer their steps apart (in_names / in_sizes, inner, `o`, as GatedBiasAttention and DecayLinearAttention do)
are run with stacked products: ONE input product over the rows of both (32-bit output), each mixer's inner step writing
its scaled result into its columns of one matrix, and ONE output product over that matrix with the two output maps laid
side by side along the input, which is the weighted sum: [W_l | W_r] [a y_l ; b y_r] = a W_l y_l + b W_r y_r.  The
weights a and b multiply in 32-bit inside the inner steps' last kernels, before the one rounding there, so they cost
neither a kernel nor a rounding.
"""
from __future__ import annotations

from typing import Callable, Hashable, Optional

import torch

from .. import ops
from .base import BatchShape, Mixer, ParamSpec, Part, Runtime, StepContext, StepPlan
from .linear import Linear


class SideBySideMixer(Mixer):
    def __init__(self, rt: Runtime, width: int, left: Mixer, right: Mixer, left_scale: float, right_scale: float):
        for m in (left, right):
            if not all(hasattr(m, a) for a in ("in_names", "in_sizes", "inner", "inner_size", "o")):
                raise ValueError(f"{type(m).__name__} does not offer its steps apart (in_names, in_sizes, inner, inner_size, o)")
        self.rt, self.width = rt, width
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.n_left = sum(left.in_sizes())
        self.proj = Linear(rt, left.in_names() + right.in_names(), width, left.in_sizes() + right.in_sizes())
        self.o = Linear(rt, [left.o.names[0], right.o.names[0]], [left.inner_size, right.inner_size], width)
        # a mixer may keep several things (a tuple): the pair asks for the two laid end to end and hands each its share
        self._left_tuple, self._right_tuple = isinstance(left.cache_request(), tuple), isinstance(right.cache_request(), tuple)
        self._n_left_caches = len(left.cache_request()) if self._left_tuple else 1

    @property
    def recordable(self) -> bool:
        return bool(self.left.recordable and self.right.recordable)

    def children(self) -> list[Part]:
        # the mixers' own children (a convolution, say) but for their input and output products, which this part's replace
        own = [c for m in (self.left, self.right) for c in m.children()
               if c is not m.o and not (isinstance(c, Linear) and c.names == list(m.in_names()))]
        return [self.proj, self.o, *own]

    def param_specs(self) -> list[ParamSpec]:
        # the two mixers' own tensors (norm weights and the like); their products' tensors are this part's
        return list(self.left.param_specs()) + list(self.right.param_specs())

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.left.bind(get)
        self.right.bind(get)

    def cache_request(self) -> tuple:
        a, b = self.left.cache_request(), self.right.cache_request()
        return (a if self._left_tuple else (a,)) + (b if self._right_tuple else (b,))

    def plan_key(self) -> Optional[Hashable]:
        a, b = self.left.plan_key(), self.right.plan_key()
        if a is not None and b is not None and a != b:
            raise NotImplementedError("two mixers side by side that both plan work on the host")
        return a if a is not None else b

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        return (self.left if self.left.plan_key() is not None else self.right).plan(batch)

    def forward(self, h: torch.Tensor, step: StepContext, cache, write_cache: bool = True) -> torch.Tensor:
        left_cache, right_cache = cache[:self._n_left_caches], cache[self._n_left_caches:]
        left_cache = left_cache if self._left_tuple else left_cache[0]
        right_cache = right_cache if self._right_tuple else right_cache[0]
        pre = self.proj.forward(h, out_dtype=torch.float32)
        kl = self.left.inner_size
        inner = self.rt.empty((h.shape[0], kl + self.right.inner_size))
        self.left.inner(pre[:, :self.n_left], step, left_cache, inner[:, :kl], self.left_scale, write_cache)
        self.right.inner(pre[:, self.n_left:], step, right_cache, inner[:, kl:], self.right_scale, write_cache)
        return self.o.forward(inner, out_dtype=torch.float32)


class NormedPairMixer(Mixer):
    """Two mixers side by side whose outputs are normed before they are added:

        out = a * rmsnorm(left(x)) * w_l + b * rmsnorm(right(x)) * w_r          (norms over the model width, plain weights)

    A norm does not commute with the output products, so unlike SideBySideMixer each mixer keeps its own output product
    (32-bit sums, never rounded before the norm); what is shared is the INPUT product, one over the rows of both, and
    one kernel norms both outputs and adds them.  Each mixer's cache request is a tuple; the pair asks for the two laid
    end to end and hands each mixer its share."""

    def __init__(self, rt: Runtime, width: int, left: Mixer, right: Mixer, left_norm_name: str, right_norm_name: str,
                 left_scale: float, right_scale: float, eps: float):
        for m in (left, right):
            if not all(hasattr(m, a) for a in ("in_names", "in_sizes", "inner", "inner_size", "o")):
                raise ValueError(f"{type(m).__name__} does not offer its steps apart (in_names, in_sizes, inner, inner_size, o)")
        self.rt, self.width, self.eps = rt, width, float(eps)
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.names = (left_norm_name, right_norm_name)
        self.n_left = sum(left.in_sizes())
        self.proj = Linear(rt, left.in_names() + right.in_names(), width, left.in_sizes() + right.in_sizes())
        self._n_left_caches = len(self._as_tuple(left.cache_request()))
        self.w_left: torch.Tensor | None = None
        self.w_right: torch.Tensor | None = None

    @staticmethod
    def _as_tuple(r) -> tuple:
        return r if isinstance(r, tuple) else (r,)

    @property
    def recordable(self) -> bool:
        return bool(self.left.recordable and self.right.recordable)

    def children(self) -> list[Part]:
        # the mixers' own children but for their input products, which this part's one product replaces
        own = [c for m in (self.left, self.right) for c in m.children() if c is not getattr(m, "proj", None)]
        return [self.proj, *own]

    def param_specs(self) -> list[ParamSpec]:
        return (list(self.left.param_specs()) + list(self.right.param_specs())
                + [ParamSpec(self.names[0], (self.width,), "norm"), ParamSpec(self.names[1], (self.width,), "norm")])

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.left.bind(get)
        self.right.bind(get)
        self.w_left = get(self.names[0]).to(torch.float32).contiguous()
        self.w_right = get(self.names[1]).to(torch.float32).contiguous()

    def cache_request(self) -> tuple:
        return self._as_tuple(self.left.cache_request()) + self._as_tuple(self.right.cache_request())

    def plan_key(self) -> Optional[Hashable]:
        a, b = self.left.plan_key(), self.right.plan_key()
        if a is not None and b is not None and a != b:
            raise NotImplementedError("two mixers side by side that both plan work on the host")
        return a if a is not None else b

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        return (self.left if self.left.plan_key() is not None else self.right).plan(batch)

    def forward(self, h: torch.Tensor, step: StepContext, cache, write_cache: bool = True) -> torch.Tensor:
        left_cache, right_cache = cache[:self._n_left_caches], cache[self._n_left_caches:]
        pre = self.proj.forward(h, out_dtype=torch.float32)
        T = h.shape[0]
        a_in, b_in = self.rt.empty((T, self.left.inner_size)), self.rt.empty((T, self.right.inner_size))
        self.left.inner(pre[:, :self.n_left], step, left_cache, a_in, 1.0, write_cache)
        self.right.inner(pre[:, self.n_left:], step, right_cache, b_in, 1.0, write_cache)
        a = self.left.o.forward(a_in, out_dtype=torch.float32)
        b = self.right.o.forward(b_in, out_dtype=torch.float32)
        out = self.rt.empty((T, self.width), torch.float32)
        ops.rmsnorm_mix2(out, a, b, self.w_left, self.w_right, self.left_scale, self.right_scale, self.eps, self.rt.stream)
        return out
