"""Token embedding and output head."""
from __future__ import annotations

from typing import Callable

import torch

from .. import ops
from .base import ParamSpec, Part, Runtime
from .linear import Linear


class TokenEmbedding(Part):
    """residual[t, :] = table[id_t, :], unscaled (src/kernels/embedding.cu:22-38 of lucciola), as float32.
    With `positions_name` the model has a table of learned position vectors [max_positions, hidden], and
    residual[t, :] += positions[p_t, :] (unscaled, added in 32-bit); forward() then takes the tokens' positions.
    With `sinusoid_base` b a sinusoidal vector is added instead, for positions without a limit: entry 2i is
    sin(p * b^(-2i / hidden)), entry 2i + 1 the cosine of the same angle; the frequencies are made once in 64-bit.
    `scale` multiplies the table's row (in 32-bit); an output head tied to the table reads it unscaled."""
    recordable = True

    def __init__(self, rt: Runtime, name: str, vocab_size: int, hidden_size: int, positions_name: str | None = None,
                 max_positions: int = 0, sinusoid_base: float | None = None, scale: float = 1.0):
        self.scale = float(scale)
        if sinusoid_base is not None and self.scale != 1.0:
            raise ValueError("sinusoidal positions come with an unscaled embedding")
        self.rt, self.name, self.vocab_size, self.hidden_size = rt, name, vocab_size, hidden_size
        self.positions_name, self.max_positions = positions_name, max_positions
        if positions_name is not None and max_positions <= 0:
            raise ValueError("a table of position vectors needs its number of rows")
        if positions_name is not None and sinusoid_base is not None:
            raise ValueError("positions are a table of vectors or sinusoids, not both")
        self.sinusoid_base = float(sinusoid_base) if sinusoid_base is not None else None
        self.weight: torch.Tensor | None = None
        self.position_table: torch.Tensor | None = None
        self.sin_freq: torch.Tensor | None = None

    @property
    def uses_positions(self) -> bool:
        return self.positions_name is not None or self.sinusoid_base is not None

    def param_specs(self) -> list[ParamSpec]:
        specs = [ParamSpec(self.name, (self.vocab_size, self.hidden_size), "embedding")]
        if self.positions_name is not None:
            specs.append(ParamSpec(self.positions_name, (self.max_positions, self.hidden_size), "embedding"))
        return specs

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.weight = get(self.name).contiguous()
        if self.positions_name is not None:
            self.position_table = get(self.positions_name).to(self.weight.dtype).contiguous()
        if self.sinusoid_base is not None:
            i = torch.arange((self.hidden_size + 1) // 2, dtype=torch.float64)
            self.sin_freq = (self.sinusoid_base ** (-2.0 * i / self.hidden_size)).to(self.weight.device).contiguous()

    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor | None = None, copy: torch.Tensor | None = None) -> torch.Tensor:
        """`copy` (float32 [T, hidden]) receives the output a second time, for a model that adds it to the stream again."""
        out = self.rt.empty((token_ids.shape[0], self.hidden_size), torch.float32)
        if copy is not None and self.sinusoid_base is not None:
            raise ValueError("no second copy of an embedding with sinusoidal positions")
        if self.uses_positions and positions is None:
            raise ValueError("this embedding adds position vectors and needs the tokens' positions")
        if self.sinusoid_base is not None:
            ops.embedding(out, token_ids, self.weight, self.rt.stream, positions=positions, sin_freq=self.sin_freq)
        elif self.positions_name is not None:
            ops.embedding(out, token_ids, self.weight, self.rt.stream, pos_table=self.position_table, positions=positions,
                          scale=self.scale, copy=copy)
        else:
            ops.embedding(out, token_ids, self.weight, self.rt.stream, scale=self.scale, copy=copy)
        return out


class OutputHead(Part):
    """logits = h . W^T in float32; W is its own tensor or the embedding table when tied
    (src/qwen.cc:80-84 of lucciola falls back to a second copy of the table; here the table is shared)."""
    recordable = True


    def __init__(self, rt: Runtime, name: str, vocab_size: int, hidden_size: int, tied_to: TokenEmbedding | None,
                 scale: float = 1.0):
        self.rt, self.name, self.tied_to = rt, name, tied_to
        self.vocab_size = vocab_size
        self.scale = float(scale)           # the logits are multiplied by this, in 32-bit
        self.proj = Linear(rt, name, hidden_size, vocab_size)

    def param_specs(self) -> list[ParamSpec]:
        return [] if self.tied_to is not None else self.proj.param_specs()

    def ignored_names(self) -> list[str]:
        """A tied head does not need its own tensor; a checkpoint may carry one all the same."""
        return [self.name] if self.tied_to is not None else []

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        if self.tied_to is not None:
            self.proj.bind_tensor(self.tied_to.weight)
        else:
            self.proj.bind(get)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.proj.forward(h, out_dtype=torch.float32)
        if self.scale != 1.0:
            ops.scale_(logits, self.scale, self.rt.stream)
        return logits
