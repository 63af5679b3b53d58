"""Pre-norm residual block: r += mixer(norm1(r)); r += ffn(norm2(r)) (src/qwen.cc:574-798 of lucciola).  A block may
have no feed-forward: then it is its first half alone.

The residual stream is float32.  A block hands the output of its feed-forward on as `delta`
instead of adding it: the next block's first norm adds it in the same pass (one kernel
instead of the add, copy and norm that lucciola launches at src/qwen.cc:742-759)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Block, FeedForward, Mixer, Norm, NormSink, Part, RowScaled, StepContext, StreamCopy
from .causal_taps import CausalTaps


class PreNormBlock(Block):
    accepts_next_sink = True
    # Where the add and the norm between two products may run inside those products (see forward): "both", or only at
    # the block's "entry" (the block before -> this block's mixer), only in its "middle" (mixer -> feed-forward), or
    # "none": always as a kernel of their own.  For comparisons.
    fuse_norms = "both"
    recordable = True

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], mixer_norm: Norm, ffn_norm: Optional[Norm],
                 act_dtype: torch.dtype):
        if (feed_forward is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.act_dtype = act_dtype

    def children(self) -> list[Part]:
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None]

    @property
    def takes_delta_parts(self) -> bool:
        """A norm that adds two deltas in the pass in which it norms takes what the model wants added before this block
        (the output of the block before and, say, the embedding's output once more) as a tuple."""
        return hasattr(self.mixer_norm, "add_forward_pair")

    def entry_sink(self, residual: torch.Tensor, num_tokens: int, write_cache: bool) -> Optional[NormSink]:
        """The block before may add its output to the residual stream itself and hand it over without the first norm's
        factor, when this block's mixer can take rows in that form for this step."""
        if self.fuse_norms in ("both", "entry") and self.mixer.row_scaled_ok(num_tokens, write_cache):
            return self.mixer_norm.as_sink(residual)
        return None

    def forward(self, residual: torch.Tensor, delta, step: StepContext, cache, write_cache: bool = True,
                next_sink: Optional[NormSink] = None):
        # Between two products, the add into the residual stream and the norm either run as a kernel of their own, or,
        # where the product before and the product after can, inside those two (NormSink, RowScaled).
        if isinstance(delta, RowScaled):
            h = delta
        elif isinstance(delta, tuple):
            h, _ = self.mixer_norm.add_forward_pair(residual, delta, None, self.act_dtype)
        else:
            h = self.mixer_norm.add_forward(residual, delta, self.act_dtype)
        if self.feed_forward is None:
            return residual, self.mixer.forward(h, step, cache, write_cache)
        sink = None
        if self.fuse_norms in ("both", "middle") and self.mixer.accepts_sink and self.feed_forward.row_scaled_ok(step.num_tokens):
            sink = self.ffn_norm.as_sink(residual)
        a = self.mixer.forward(h, step, cache, write_cache, sink=sink) if sink is not None else self.mixer.forward(h, step, cache, write_cache)
        h = a if isinstance(a, RowScaled) else self.ffn_norm.add_forward(residual, a, self.act_dtype)
        if next_sink is not None and self.feed_forward.accepts_sink:
            return residual, self.feed_forward.forward(h, step, sink=next_sink)
        return residual, self.feed_forward.forward(h, step)


class ParallelBlock(Block):
    """One norm, two sublayers side by side: h = norm(r); r += mixer(u) + ffn(h), where the mixer reads
    u = input_taps(h) (a short causal convolution over time added to h) if the block has one, else h.  The
    feed-forward always reads h; a block may have none.  With `ffn_norm` the feed-forward has a norm of its own on the
    same stream, r += mixer(norm(r)) + ffn(ffn_norm(r)); two RMS norms with one eps then run as one kernel that adds what
    the block before left, norms once and applies both weights (RMSNorm.add_forward_pair).

    The block hands its two outputs on unsummed when the norm that follows takes them (`delta_parts`): that norm adds
    both to the 32-bit residual stream in the pass in which it reads it.  The taps' state (the last inputs of each
    sequence) lives beside the mixer's cache: the block asks for (taps' state, mixer's cache)."""
    recordable = True
    offers_delta_parts = True

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], norm: Norm, act_dtype: torch.dtype,
                 input_taps: Optional[CausalTaps] = None, ffn_norm: Optional[Norm] = None):
        self.mixer, self.feed_forward, self.norm, self.input_taps = mixer, feed_forward, norm, input_taps
        if ffn_norm is not None and feed_forward is None:
            raise ValueError("a norm for a feed-forward that is not there")
        self.ffn_norm = ffn_norm
        # two RMS norms of one stream with one eps: one kernel adds the deltas, norms once and applies both weights
        self._paired = hasattr(norm, "add_forward_pair") and (ffn_norm is None or (type(ffn_norm) is type(norm)
                                                               and ffn_norm.eps == norm.eps and ffn_norm.size == norm.size))
        self.act_dtype = act_dtype
        self._taps_state = input_taps.cache_request() if input_taps is not None else None
        self._rt = norm.rt

    @property
    def takes_delta_parts(self) -> bool:
        return self.norm.takes_delta_parts or (self.ffn_norm is not None and self._paired)

    def children(self) -> list[Part]:
        return [p for p in (self.norm, self.ffn_norm, self.input_taps, self.mixer, self.feed_forward) if p is not None]

    def cache_request(self):
        mixer = self.mixer.cache_request()
        return (self._taps_state, mixer) if self._taps_state is not None else mixer

    def forward(self, residual: torch.Tensor, delta, step: StepContext, cache, write_cache: bool = True,
                delta_parts: bool = False):
        if self.ffn_norm is not None and self._paired:
            deltas = delta if isinstance(delta, tuple) else ((delta,) if delta is not None else ())
            h, h_ffn = self.norm.add_forward_pair(residual, deltas, self.ffn_norm, self.act_dtype)
        else:
            h = self.norm.add_forward(residual, delta, self.act_dtype)
            h_ffn = self.ffn_norm.forward(residual, self.act_dtype) if self.ffn_norm is not None else h
        taps_cache, mixer_cache = cache if self._taps_state is not None else (None, cache)
        u = self.input_taps.forward(h, step, taps_cache) if self.input_taps is not None else h
        a = self.mixer.forward(u, step, mixer_cache, write_cache)
        if self.feed_forward is None:
            return residual, a
        b = self.feed_forward.forward(h_ffn, step)
        if delta_parts:
            return residual, (a, b)
        # the norm that follows adds one delta only: the mixer's output goes into the residual stream here
        ops.add_into(residual, a, self._rt.stream)
        return residual, b


class PostNormBlock(Block):
    """Norm on the sublayer's output only: r += m * norm1(mixer(r)); r += m * norm2(ffn(r)).  The sublayers read the
    residual stream itself; `m` is one multiplier for both.  A block may have no feed-forward.

    The stream is 32-bit; what the sublayers' products read is its copy in the activation type, which the kernel that
    adds a normed output writes in the same pass (Norm.add_normed) and which the block hands on as StreamCopy, so only
    the first block of a model makes a copy by a kernel of its own.  In a 32-bit engine the sublayers read the stream
    directly."""
    recordable = True
    takes_stream_copy = True

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], mixer_norm: Norm, ffn_norm: Optional[Norm],
                 residual_mult: float, act_dtype: torch.dtype):
        if (feed_forward is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer, self.feed_forward, self.mixer_norm, self.ffn_norm = mixer, feed_forward, mixer_norm, ffn_norm
        self.residual_mult, self.act_dtype = float(residual_mult), act_dtype
        self._rt = mixer_norm.rt

    def children(self) -> list[Part]:
        return [p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.ffn_norm) if p is not None]

    def forward(self, residual: torch.Tensor, delta, step: StepContext, cache, write_cache: bool = True):
        exact = self.act_dtype == torch.float32
        copy_dtype = None if exact else self.act_dtype
        if isinstance(delta, StreamCopy):
            h = delta.x
        else:
            if delta is not None:                       # a block of another kind left something to be added
                ops.add_into(residual, delta, self._rt.stream)
            h = residual
            if not exact:
                h = self._rt.empty(residual.shape)
                ops.round_copy(h, residual, self._rt.stream)
        a = self.mixer.forward(h, step, cache, write_cache)
        h = self.mixer_norm.add_normed(residual, (a,), (1.0,), self.residual_mult, copy_dtype)
        if self.feed_forward is not None:
            b = self.feed_forward.forward(residual if exact else h, step)
            h = self.ffn_norm.add_normed(residual, (b,), (1.0,), self.residual_mult, copy_dtype)
        return residual, (None if exact else StreamCopy(h))
