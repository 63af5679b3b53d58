"""A decoder as data: blocks, and the list of calls that runs them.

`calls` gives the order in which blocks run.  A call names a block and a cache; a block may be
called twice (with two caches), and a call may read a cache that an earlier call has written
(`write_cache=False`): then the mixer computes queries only and attends to what is there.  A call may ask for the
embedding's output to be added to the stream before its block runs (`add_embedding`: models that repeat a run of
layers and feed the input in again at the start of every pass).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import ops
from ..parts.base import Block, KVPages, Norm, Part, Runtime, StateSlot, StepContext, StreamCopy
from ..parts.embedding import OutputHead, TokenEmbedding


@dataclass(frozen=True)
class LayerCall:
    block: int
    cache: int
    write_cache: bool = True
    add_embedding: bool = False      # the embedding's output is added to the stream before this call's block runs


class DecoderModel(Part):
    recordable = True

    def __init__(self, rt: Runtime, embedding: TokenEmbedding, blocks: Sequence[Block], calls: Sequence[LayerCall],
                 final_norm: Norm, head: OutputHead, vocab_size: int, max_positions: int, eos_token_ids: Sequence[int] = (),
                 ignored_names: Sequence[str] = ()):
        self.rt = rt
        self.embedding, self.blocks, self.calls = embedding, list(blocks), list(calls)
        self.final_norm, self.head = final_norm, head
        self.vocab_size, self.max_positions = vocab_size, max_positions
        self.eos_token_ids = tuple(eos_token_ids)
        self._ignored = list(ignored_names)      # tensors a checkpoint may carry that this model has no use for
        self._check_calls()

    def _check_calls(self) -> None:
        written: dict[int, int] = {}
        for i, c in enumerate(self.calls):
            if not (0 <= c.block < len(self.blocks)):
                raise ValueError(f"call {i} names block {c.block}, there are {len(self.blocks)}")
            if c.write_cache:
                if c.cache in written:
                    raise ValueError(f"cache {c.cache} is written by calls {written[c.cache]} and {i}")
                written[c.cache] = i
            elif c.cache not in written:
                raise ValueError(f"call {i} reads cache {c.cache} before any call has written it")
            else:
                a, b = self.blocks[self.calls[written[c.cache]].block].cache_request(), self.blocks[c.block].cache_request()
                if a != b:
                    raise ValueError(f"call {i} reads cache {c.cache} but its mixer wants {b}, the cache holds {a}")
        if sorted(written) != list(range(len(written))):
            raise ValueError(f"cache ids must be 0..n-1, got {sorted(written)}")
        self.num_caches = len(written)
        self._writer = written

    def children(self) -> list[Part]:
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def ignored_names(self) -> list[str]:
        return self.head.ignored_names() + self._ignored

    def cache_requests(self) -> list[KVPages | StateSlot | None | tuple]:
        """What each cache id has to hold, as asked by the block that writes it (its mixer's needs, and the block's own)."""
        return [self.blocks[self.calls[self._writer[j]].block].cache_request() for j in range(self.num_caches)]

    def forward(self, token_ids: torch.Tensor, step: StepContext, caches: Sequence[object],
                logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the tokens of one step; float32 logits [R, vocab] for the rows asked for (None if none)."""
        again = None                                     # a second copy of the embedding's output, for the calls that add it
        if any(c.add_embedding for c in self.calls):
            again = self.rt.empty((token_ids.shape[0], self.embedding.hidden_size), torch.float32)
        pos = step.positions if getattr(self.embedding, "uses_positions", False) else None
        residual = self.embedding.forward(token_ids, pos, copy=again) if again is not None else (
            self.embedding.forward(token_ids, pos) if pos is not None else self.embedding.forward(token_ids))
        delta = None
        for i, c in enumerate(self.calls):
            if c.add_embedding:
                # with what the block before left, if this block's first norm adds two things in its pass; else by itself
                if self.blocks[c.block].takes_delta_parts and (delta is None or (torch.is_tensor(delta) and delta.dtype == again.dtype)):
                    delta = (delta, again) if delta is not None else (again,)
                else:
                    if isinstance(delta, tuple):
                        for d in delta:
                            ops.add_into(residual, d, self.rt.stream)
                        delta = None
                    elif torch.is_tensor(delta):
                        ops.add_into(residual, delta, self.rt.stream)
                        delta = None
                    elif delta is not None and not isinstance(delta, StreamCopy):
                        raise ops.KernelError("the embedding cannot be added again behind a block that hands its output on inside a product")
                    ops.add_into(residual, again, self.rt.stream)
                    delta = None
            # what the call after this one offers to take over from this one's last product (see Block.entry_sink)
            nxt = self.calls[i + 1] if i + 1 < len(self.calls) else None
            block = self.blocks[c.block]
            if isinstance(delta, StreamCopy) and not block.takes_stream_copy:
                delta = None                             # nothing is left to be added; this block makes its own input
            next_sink = (self.blocks[nxt.block].entry_sink(residual, step.num_tokens, nxt.write_cache)
                         if nxt is not None and not nxt.add_embedding else None)
            # a block whose sublayers run side by side may leave their outputs unsummed when the norm that adds them
            # to the residual stream takes both (see Block.offers_delta_parts)
            parts_ok = (self.blocks[nxt.block].takes_delta_parts if nxt is not None else self.final_norm.takes_delta_parts)
            if next_sink is not None and block.accepts_next_sink:
                residual, delta = block.forward(residual, delta, step, caches[c.cache], c.write_cache, next_sink=next_sink)
            elif block.offers_delta_parts and parts_ok:
                residual, delta = block.forward(residual, delta, step, caches[c.cache], c.write_cache, delta_parts=True)
            else:
                residual, delta = block.forward(residual, delta, step, caches[c.cache], c.write_cache)
        if logit_rows is None or logit_rows.shape[0] == 0:
            return None
        if isinstance(delta, StreamCopy):
            delta = None
        h = self.final_norm.add_forward(residual, delta, self.rt.act_dtype, rows=logit_rows)
        return self.head.forward(h)
