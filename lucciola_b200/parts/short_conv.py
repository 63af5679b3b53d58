"""A short causal convolution over time, one filter a channel: y_t = act(b + sum_j w[:, j] * x_(t - taps + 1 + j)).

Unlike CausalTaps the input is not added to the result, rows are 32-bit (a product's 32-bit output goes in, what a
recurrence reads comes out) and there may be a bias.  The filter may be made of several checkpoint tensors laid side by
side along the channels ([channels_i, taps] each, last column the current token's), so that q | k | v of a mixer pass
one launch.  Zeros before a sequence's start; the last taps - 1 inputs of a sequence are its state (a slot of
[taps - 1, channels] in 32-bit, zero for a new request), so a portion of a prompt or a single decoded token continues
where the step before stopped.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from .. import ops
from .base import ParamSpec, Part, Runtime, StateCacheView, StateSlot, StepContext


class ShortConv(Part):
    recordable = True

    def __init__(self, rt: Runtime, names: str | Sequence[str], channels: int | Sequence[int], taps: int,
                 bias_name: Optional[str] = None, act: bool = True):
        self.rt = rt
        self.names = [names] if isinstance(names, str) else list(names)
        self.sizes = [channels] if isinstance(channels, int) else list(channels)
        if len(self.names) != len(self.sizes):
            raise ValueError("one channel count for each tensor name")
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        self.channels, self.taps, self.bias_name, self.act = sum(self.sizes), int(taps), bias_name, bool(act)
        self.weight: torch.Tensor | None = None     # float32 [taps, channels]: the checkpoint's tensors, side by side, transposed
        self.bias: torch.Tensor | None = None

    def param_specs(self) -> list[ParamSpec]:
        specs = [ParamSpec(n, (c, self.taps), "linear") for n, c in zip(self.names, self.sizes)]
        if self.bias_name is not None:
            specs.append(ParamSpec(self.bias_name, (self.channels,), "linear"))
        return specs

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.weight = torch.cat([get(n).to(torch.float32) for n in self.names], dim=0).t().contiguous()
        if self.bias_name is not None:
            self.bias = get(self.bias_name).to(torch.float32).contiguous()

    def cache_request(self) -> Optional[StateSlot]:
        return StateSlot((self.taps - 1, self.channels), torch.float32) if self.taps > 1 else None

    def forward(self, x: torch.Tensor, step: StepContext, cache: Optional[StateCacheView]) -> torch.Tensor:
        """x: float32 [T, channels] (may be a column range).  Returns y, float32 [T, channels]; the sequences' states
        move on to the end of the step."""
        out = self.rt.empty(x.shape, torch.float32)
        state = cache.state if self.taps > 1 else None
        ops.short_conv(out, x, self.weight, self.bias, state, step, self.rt.stream, act=self.act)
        if state is not None:
            ops.short_conv_state(state, x, self.taps, step, self.rt.stream)
        return out
