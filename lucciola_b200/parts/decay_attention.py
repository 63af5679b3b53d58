"""Linear attention with a fixed decay per head ("lightning attention").  Per head, with a state S [dim, vdim]:

    q = silu(W_q x)    k = silu(W_k x)    v = silu(W_v x)
    S_t = decay_h S_(t-1) + k_t v_t^T        o_t = S_t^T q_t
    out = W_o ( rmsnorm(concat_h o_t) * w * sigmoid(W_g x) )       (one norm over all heads, w [heads * vdim])

The state is 32-bit, one slot a request, zero for a new request, and is all this mixer keeps of the past: prompts,
portions and decoded tokens go through the same kernel, which walks a sequence's tokens of the step in order from the
state the step before left.  W_q | W_k | W_v | W_g are one product with 32-bit output; the activations, the recurrence,
the norm and the gate are computed in 32-bit.  In the bfloat16 engine steps with many tokens a sequence form the
outputs of 16 tokens side by side (still 32-bit, the same state); the 32-bit engine walks every step token by token,
so its results do not depend on how a prompt was cut.

The form is a parameter, so that a relative of the design above can use the same part and kernels ("retention"):
`act` ("silu", or None: q, k, v as projected), `position_encoding` (q and k are rotated in 32-bit, in place, after the
product), `k_scale` (k is multiplied by it after the rotation), `head_norm` (True: each head's output is RMS-normed on
its own, not all heads together), `norm_weight` (False: the norm has no weight and the checkpoint no tensor for it) and
`gate_act` ("sigmoid" or "silu").

Beside forward(), the mixer offers its three steps apart (in_names / in_sizes, inner, `o`), so that a mixer that runs
it beside another may stack their products (see SideBySideMixer).
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from .. import ops
from .base import Mixer, ParamSpec, Part, PositionEncoding, Runtime, StateCacheView, StateSlot, StepContext
from .linear import Linear


class DecayLinearAttention(Mixer):
    def __init__(self, rt: Runtime, prefix: str, width: int, heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float,
                 names: Optional[dict] = None, act: Optional[str] = "silu", position_encoding: Optional[PositionEncoding] = None,
                 k_scale: float = 1.0, head_norm: bool = False, norm_weight: bool = True, gate_act: str = "sigmoid",
                 out_dtype: Optional[torch.dtype] = None):
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        if act not in ("silu", None) or gate_act not in ("sigmoid", "silu"):
            raise ValueError(f"activation {act!r} or gate {gate_act!r}: q, k, v pass silu or nothing, the gate sigmoid or silu")
        if position_encoding is not None and position_encoding.rotary_table() is None:
            raise ValueError("q and k of a decay attention are rotated by a table of frequencies (rotary_table)")
        self.act, self.position_encoding, self.k_scale = act, position_encoding, float(k_scale)
        self.head_norm, self.norm_weight, self.gate_act = bool(head_norm), bool(norm_weight), gate_act
        self.out_dtype = out_dtype          # type of the output product's sums (None: the activation type)
        self.rt, self.prefix = rt, prefix
        self.width, self.heads, self.dim, self.vdim, self.eps = width, heads, dim, vdim, float(eps)
        self.names = {"q": f"{prefix}.q", "k": f"{prefix}.k", "v": f"{prefix}.v", "g": f"{prefix}.g", "o": f"{prefix}.o",
                      "norm": f"{prefix}.norm"}
        self.names.update(names or {})
        self._decay = [float(x) for x in decay]
        self.inner_size = heads * vdim
        self.qkvg = Linear(rt, self.in_names(), width, self.in_sizes())
        self.o = Linear(rt, self.names["o"], self.inner_size, width)
        self.decay: torch.Tensor | None = None
        self.norm_w: torch.Tensor | None = None

    def in_names(self) -> list[str]:
        return [self.names["q"], self.names["k"], self.names["v"], self.names["g"]]

    def in_sizes(self) -> list[int]:
        n = self.heads * self.dim
        return [n, n, self.inner_size, self.inner_size]

    def children(self) -> list[Part]:
        return [self.qkvg, self.o]

    @property
    def recordable(self) -> bool:
        return self.position_encoding is None or self.position_encoding.recordable

    def param_specs(self) -> list[ParamSpec]:
        if not self.norm_weight:
            return []
        return [ParamSpec(self.names["norm"], (self.vdim if self.head_norm else self.inner_size,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        if self.norm_weight:
            self.norm_w = get(self.names["norm"]).to(torch.float32).contiguous()
        self.decay = torch.tensor(self._decay, dtype=torch.float32, device=self.rt.device)

    def cache_request(self) -> StateSlot:
        return StateSlot((self.heads, self.dim, self.vdim), torch.float32)

    def inner(self, pre: torch.Tensor, step: StepContext, cache: StateCacheView, out: torch.Tensor, out_scale: float,
              write_cache: bool = True) -> None:
        """pre: float32 [T, >= sum(in_sizes())], the columns q | k | v | g of this mixer; out: [T, inner_size] in the
        activation type (may be a column range of a wider matrix) receives the normed, gated heads times out_scale."""
        if not write_cache:
            raise ops.KernelError("a recurrent mixer has no cache another call could have written")
        rt, n = self.rt, self.heads * self.dim
        T = pre.shape[0]
        if self.position_encoding is not None or self.k_scale != 1.0:
            inv_freq, rot = self.position_encoding.rotary_table() if self.position_encoding is not None else (None, 0)
            ops.rotate_rows(pre, step.positions, inv_freq, self.dim, rot, [(0, self.heads, 1.0), (n, self.heads, self.k_scale)], rt.stream,
                            rot_scale=getattr(self.position_encoding, "magnitude", 1.0))
        # the bfloat16 engine forms the outputs of long steps 16 tokens at a time, the rows of the state shared out over CTAs
        split = ops.decay_row_split(step.num_seqs, self.heads, self.dim, self.vdim, step.max_q_len) if rt.fast_kernels else 0
        o = rt.empty((split, T, self.inner_size) if split else (T, self.inner_size), torch.float32)
        ops.decay_recurrence(pre, 0, n, 2 * n, self.decay, cache.state, o, step, self.heads, self.dim, self.vdim, rt.stream,
                             max_tokens_a_seq=step.max_q_len, row_split=split, act=self.act is not None)
        g0 = 2 * n + self.inner_size
        if self.head_norm or not self.norm_weight or self.gate_act != "sigmoid":
            ops.gated_group_norm(out, o, pre[:, g0:g0 + self.inner_size], self.norm_w, self.heads if self.head_norm else 1, self.eps,
                                 rt.stream, act=self.gate_act, scale=out_scale)
        else:
            ops.rmsnorm_gated(out, o, self.norm_w, pre[:, g0:g0 + self.inner_size], out_scale, self.eps, rt.stream)

    def forward(self, h: torch.Tensor, step: StepContext, cache: StateCacheView, write_cache: bool = True) -> torch.Tensor:
        pre = self.qkvg.forward(h, out_dtype=torch.float32)
        inner = self.rt.empty((h.shape[0], self.inner_size))
        self.inner(pre, step, cache, inner, 1.0, write_cache)
        return self.o.forward(inner, out_dtype=self.out_dtype)
