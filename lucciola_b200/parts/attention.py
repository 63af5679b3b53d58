"""Grouped-query attention over paged keys and values, with per-head RMSNorm of q and k.

Order of operations as in lucciola's decoder layer (src/qwen.cc:592-742): q, k, v projections
without bias; RMSNorm over each head of q and of k with a weight [head_dim] shared by the heads,
before the rotation; rotary position encoding of q and k; k and v written to the cache at the
token's position; causal attention of every query head h over the keys of kv head
h / (nq / nkv) with scale 1/sqrt(head_dim) unless another scale is given; output projection.
A window W, which lucciola does not have, limits a query at position p to keys p-W+1 .. p.

The attention kernels take their work from lists of tiles that this part makes on the host before a step runs
(`plan`): which tokens of which request form a tile, how many rows a tile has, which tiles go to which kernel.
"""
from __future__ import annotations

import math
from typing import Callable, Hashable, Optional, Sequence

import numpy as np
import torch

from .. import ops
from .base import (BatchShape, KVCacheView, KVPages, Mixer, NormSink, ParamSpec, Part, PositionEncoding, RowScaled, Runtime,
                   StepContext, StepPlan)
from .linear import Linear

# Entries with at least this many tokens in a step go to the tensor-memory attention kernel (128-row tiles).
BIG_PORTION = 16
# Query rows (heads of a group x tokens) of a tile of the mma.sync kernels; tiles of at most DECODE_ROWS rows have
# a kernel of their own, which a launch uses only if all of its tiles are such.
TILE_ROWS, DECODE_ROWS = 64, 16


def tiles_of(q_lens: Sequence[int], group: int, rows: int, take=None) -> list[tuple[int, int, int, int]]:
    """Runs of up to rows // group consecutive tokens of one request: (first token, tokens, request, 0),
    for the requests whose number of tokens passes `take`."""
    per = rows // group
    tiles, t = [], 0
    for i, n in enumerate(q_lens):
        if take is None or take(n):
            for off in range(0, n, per):
                tiles.append((t + off, min(per, n - off), i, 0))
        t += n
    return tiles


def plan_tiles(batch: BatchShape, group: int) -> StepPlan:
    """The tile lists of one step for query groups of `group` heads.  Kinds: "all" = every entry; when the step
    holds portions of prompts of BIG_PORTION tokens or more, also "big" = those portions in work items of up to 256
    rows (two tiles of floor(128 / group) tokens, for the tensor-memory kernel) and "rest" = the other entries.
    Tiles of "all" and "rest" have up to 64 query rows; but where single tokens sit beside portions of a few tokens,
    those lists are cut into tiles of at most 16 rows, so that one launch of the kernel for such tiles serves them all
    (a portion of 8 tokens beside 32 decoded tokens then costs two more tiles, not a launch with key ranges split
    through a workspace and a second kernel to combine them; its keys are read once per tile, which is little for a
    few tokens).  Each array is int32 [n, 4]; host["rows"][kind] is the most query rows of a tile of that kind."""
    q_lens, starts, g = batch.q_lens, batch.start_positions, group
    has_big = batch.max_q_len >= BIG_PORTION
    small = [n for n in q_lens if n < BIG_PORTION]
    fine = (g <= DECODE_ROWS and any(n * g <= DECODE_ROWS for n in small) and any(n * g > DECODE_ROWS for n in small))
    rows_small = DECODE_ROWS if fine else TILE_ROWS
    lists: dict[str, list] = {"all": tiles_of(q_lens, g, TILE_ROWS if has_big else rows_small)}
    if has_big:
        first_token = np.concatenate(([0], np.cumsum(q_lens)[:-1])).tolist()
        big = tiles_of(q_lens, g, 2 * (128 // g) * g, lambda n: n >= BIG_PORTION)
        # tiles that see the most keys first: the short ones then fill the end of the last wave
        big.sort(key=lambda tl: -(starts[tl[2]] + (tl[0] - first_token[tl[2]]) + tl[1]))
        lists["big"] = big
        if small:
            lists["rest"] = tiles_of(q_lens, g, rows_small, lambda n: n < BIG_PORTION)
    return StepPlan({k: np.asarray(tl, dtype=np.int32).reshape(len(tl), 4) for k, tl in lists.items()},
                    {"rows": {k: max(n for _, n, _, _ in tl) * g for k, tl in lists.items()}})


class GQAttention(Mixer):
    _decode_plans: dict[tuple[int, int], StepPlan] = {}      # (group size, batch size) -> plan of a step of single tokens

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position_encoding: Optional[PositionEncoding], qk_norm_eps: Optional[float], window: int = 0,
                 scale: Optional[float] = None, names: Optional[dict] = None, v_head_dim: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        self.rt, self.prefix = rt, prefix
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.position_encoding = position_encoding
        self.qk_norm_eps = qk_norm_eps              # None: no q/k norm
        self.window = int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_size, self.kv_size = num_heads * head_dim, num_kv_heads * head_dim
        # tensor names: those of the Qwen3 checkpoints unless a design gives its own (keys q, k, v, o, q_norm, k_norm)
        self.names = {"q": f"{prefix}.q_proj.weight", "k": f"{prefix}.k_proj.weight", "v": f"{prefix}.v_proj.weight",
                      "o": f"{prefix}.o_proj.weight", "q_norm": f"{prefix}.q_norm.weight", "k_norm": f"{prefix}.k_norm.weight"}
        self.names.update(names or {})
        self.v_head_dim = int(v_head_dim) if v_head_dim else head_dim        # values may have another size than keys
        self.v_size, self.out_size = num_kv_heads * self.v_head_dim, num_heads * self.v_head_dim
        self.qkv = Linear(rt, [self.names["q"], self.names["k"], self.names["v"]],
                          hidden_size, [self.q_size, self.kv_size, self.v_size])
        self.o = Linear(rt, self.names["o"], self.out_size, hidden_size)
        self.q_norm_w: torch.Tensor | None = None
        self.k_norm_w: torch.Tensor | None = None

    def children(self) -> list[Part]:
        return [self.qkv, self.o]

    @property
    def recordable(self) -> bool:
        """This part only launches kernels; a position encoding of its own kind has its own say."""
        return self.position_encoding is None or self.position_encoding.recordable

    def param_specs(self) -> list[ParamSpec]:
        if self.qk_norm_eps is None:
            return []
        return [ParamSpec(self.names["q_norm"], (self.head_dim,), "norm"),
                ParamSpec(self.names["k_norm"], (self.head_dim,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        if self.qk_norm_eps is not None:
            self.q_norm_w = get(self.names["q_norm"]).to(torch.float32).contiguous()
            self.k_norm_w = get(self.names["k_norm"]).to(torch.float32).contiguous()

    def plan_key(self) -> Optional[Hashable]:
        """The tensor-core kernels run on the bfloat16 path for groups of up to 64 query heads; the tile lists
        depend on the group size alone, so all such layers of a model share them."""
        g = self.num_heads // self.num_kv_heads
        return ("attention tiles", g) if self.rt.fast_kernels and g <= TILE_ROWS else None

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        g = self.num_heads // self.num_kv_heads
        if batch.max_q_len == 1:                    # one token each: the same tiles for every step of this size
            key = (g, len(batch.q_lens))
            hit = self._decode_plans.get(key)
            if hit is None:
                hit = self._decode_plans[key] = plan_tiles(batch, g)
            return hit
        return plan_tiles(batch, g)

    def cache_request(self) -> KVPages:
        return KVPages(self.num_kv_heads, self.head_dim, self.window, v_head_dim=self.v_head_dim if self.v_head_dim != self.head_dim else 0)

    accepts_sink = True

    def _heads_in_epilogue(self, num_tokens: int, write_cache: bool) -> bool:
        """Few tokens and heads of 128: the q|k|v product finishes the heads in its own epilogue."""
        rotary = self.position_encoding.rotary_table() if self.position_encoding is not None else None
        return (write_cache and self.rt.fast_kernels and (self.position_encoding is None or rotary is not None)
                and (rotary is None or rotary[1] == self.head_dim)
                and ops.gemm_tcgen05_heads_sizes_ok(num_tokens, self.qkv.out_features, self.hidden_size, self.head_dim))

    def row_scaled_ok(self, num_tokens: int, write_cache: bool = True) -> bool:
        """That epilogue also applies the factor that rows without their norm's factor lack; so does the many-token
        product."""
        return self._heads_in_epilogue(num_tokens, write_cache) or self.qkv.row_scaled_ok(num_tokens)

    def _project_out(self, out: torch.Tensor, sink: Optional[NormSink]):
        if sink is not None and self.o.sink_ok(out):
            return self.o.forward_into(out, sink)
        return self.o.forward(out)

    def forward(self, h, step: StepContext, cache: KVCacheView, write_cache: bool = True, sink: Optional[NormSink] = None):
        rt = self.rt
        T = h.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        table = cache_table = step.block_tables[cache.group]
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        q = rt.empty((T, nq, d))
        rotary = self.position_encoding.rotary_table() if self.position_encoding is not None else None
        scaled = h if isinstance(h, RowScaled) else None
        x = scaled.x if scaled is not None else h
        if self._heads_in_epilogue(T, write_cache) and ops.gemm_tcgen05_heads_ok(x, self.qkv.weight, d, rotary[1] if rotary is not None else None):
            # Norm, rotation, queries into their layout, keys and values into the pages: the product's output never
            # exists as a matrix.
            ops.gemm_tcgen05_heads(x, self.qkv.weight, q, step.positions, step.token_seq, cache_table, cache.k, cache.v,
                                   nq, nkv, cache.page_size, eps, rt.stream, q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w,
                                   inv_freq=rotary[0] if rotary is not None else None,
                                   sumsq=scaled.sumsq if scaled is not None else None, row_eps=scaled.eps if scaled is not None else 0.0)
            out = rt.empty((T, nq, d))
            ops.attention(q, out, cache.k, cache.v, step, cache.group, nq, nkv, d, cache.page_size, self.window,
                          self.scale, rt.stream, plan=step.plans.get(self.plan_key()))
            return self._project_out(out.view(T, self.q_size), sink)
        if scaled is not None and not self.qkv.row_scaled_ok(T):
            raise ops.KernelError("this mixer was handed rows without their norm factor for a step it cannot take them in")
        if write_cache:
            qkv = self.qkv.forward(h)
            q_in, k_in, v_in = qkv[:, :self.q_size], qkv[:, self.q_size:self.q_size + self.kv_size], qkv[:, self.q_size + self.kv_size:]
            n_kv = nkv
        else:
            # This call reads a cache another call has written: only q is needed.
            q_in = k_in = v_in = self.qkv.forward(h, rows=self.q_size)
            n_kv = 0
        if self.position_encoding is None or rotary is not None:
            inv_freq, rot = rotary if rotary is not None else (None, 0)
            ops.rope_kv(q_in, k_in, v_in, q, step.positions, nq, n_kv, d, eps, rt.stream,
                        q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, inv_freq=inv_freq, rot_dim=rot,
                        k_cache=cache.k, v_cache=cache.v, token_seq=step.token_seq, block_table=cache_table,
                        page_size=cache.page_size)
        else:
            # A position encoding the fused kernel does not know: norm first, then the part's own
            # apply(), then the write.
            k_tmp, v_tmp = rt.empty((T, max(n_kv, 1), d)), rt.empty((T, max(n_kv, 1), d))
            ops.rope_kv(q_in, k_in, v_in, q, step.positions, nq, n_kv, d, eps, rt.stream,
                        q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, k_out=k_tmp, v_out=v_tmp)
            self.position_encoding.apply(q, k_tmp, step.positions)
            if n_kv:
                k2, v2 = k_tmp.view(T, n_kv * d), v_tmp.view(T, n_kv * d)
                ops.rope_kv(k2, k2, v2, q, step.positions, 0, n_kv, d, 0.0, rt.stream,
                            k_cache=cache.k, v_cache=cache.v, token_seq=step.token_seq, block_table=cache_table,
                            page_size=cache.page_size)
        out = rt.empty((T, nq, d))
        ops.attention(q, out, cache.k, cache.v, step, cache.group, nq, nkv, d, cache.page_size, self.window,
                      self.scale, rt.stream, plan=step.plans.get(self.plan_key()))
        return self._project_out(out.view(T, self.q_size), sink)


def distance_slopes(num_heads: int, exponent: float = 8.0) -> list[float]:
    """The slopes of a linear distance bias: head h gets 2^(-exponent (h + 1) / num_heads)."""
    return [2.0 ** (-exponent * (h + 1) / num_heads) for h in range(num_heads)]


class GatedBiasAttention(GQAttention):
    """Grouped-query attention without rotation whose positions enter as a linear distance bias, with a sigmoid gate of
    one number a head on the output:

        score(i, j) = (q_i . k_j) * scale - slope_h * (i - j)          for the keys j the window allows
        out_h = softmax(score) V * sigmoid(W_g x)_h                     before the output projection

    Queries and keys are normed per head as in GQAttention; values may have another size than keys (`v_head_dim`).
    q | k | v | g are one product with 32-bit output.  Beside forward(), the mixer offers the three steps apart, so that a
    mixer that runs it beside another may stack their products: in_names() / in_sizes() (the tensors and widths of the
    input product), inner(pre, ...) (from the product's 32-bit columns to the scaled input of the output projection,
    written where the caller says), and `o`."""
    accepts_sink = False

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: int, scale: float, window: int, qk_norm_eps: Optional[float], slopes: Sequence[float],
                 names: Optional[dict] = None):
        base = {"q": f"{prefix}.q", "k": f"{prefix}.k", "v": f"{prefix}.v", "o": f"{prefix}.o", "g": f"{prefix}.g",
                "q_norm": f"{prefix}.q.norm", "k_norm": f"{prefix}.k.norm"}
        base.update(names or {})
        super().__init__(rt, prefix, hidden_size, num_heads, num_kv_heads, head_dim, None, qk_norm_eps, window, scale,
                         names=base, v_head_dim=v_head_dim)
        if len(slopes) != num_heads:
            raise ValueError(f"{len(slopes)} slopes for {num_heads} heads")
        self._slopes = [float(x) for x in slopes]
        self.slopes: torch.Tensor | None = None
        self.qkvg = Linear(rt, self.in_names(), hidden_size, self.in_sizes())
        self.inner_size = self.out_size

    def in_names(self) -> list[str]:
        return [self.names["q"], self.names["k"], self.names["v"], self.names["g"]]

    def in_sizes(self) -> list[int]:
        return [self.q_size, self.kv_size, self.v_size, self.num_heads]

    def children(self) -> list[Part]:
        return [self.qkvg, self.o]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        super().bind(get)
        self.slopes = torch.tensor(self._slopes, dtype=torch.float32, device=self.rt.device)

    def row_scaled_ok(self, num_tokens: int, write_cache: bool = True) -> bool:
        return False

    def inner(self, pre: torch.Tensor, step: StepContext, cache: KVCacheView, out: torch.Tensor, out_scale: float,
              write_cache: bool = True) -> None:
        """pre: float32 [T, >= sum(in_sizes())], the columns q | k | v | g of this mixer; out: [T, inner_size] in the
        activation type (may be a column range of a wider matrix) receives the gated heads times out_scale."""
        rt = self.rt
        T, nq, nkv, d, dv = pre.shape[0], self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        c1, c2, c3 = self.q_size, self.q_size + self.kv_size, self.q_size + self.kv_size + self.v_size
        q = rt.empty((T, nq, d))
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        ops.rope_kv(pre[:, :c1], pre[:, c1:c2], pre[:, c2:c3], q, step.positions, nq, nkv if write_cache else 0, d, eps, rt.stream,
                    q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, k_cache=cache.k, v_cache=cache.v, token_seq=step.token_seq,
                    block_table=step.block_tables[cache.group], page_size=cache.page_size, v_dim=dv)
        heads = rt.empty((T, nq, dv))
        ops.attention(q, heads, cache.k, cache.v, step, cache.group, nq, nkv, d, cache.page_size, self.window, self.scale,
                      rt.stream, plan=step.plans.get(self.plan_key()), v_dim=dv, slopes=self.slopes)
        ops.head_gate(out, heads, pre[:, c3:c3 + nq], out_scale, rt.stream)

    def forward(self, h, step: StepContext, cache: KVCacheView, write_cache: bool = True):
        pre = self.qkvg.forward(h, out_dtype=torch.float32)
        inner = self.rt.empty((h.shape[0], self.inner_size))
        self.inner(pre, step, cache, inner, 1.0, write_cache)
        return self.o.forward(inner)


class PooledWindowAttention(Mixer):
    """Softmax attention over a sliding window and, behind it, over one mean key and value for every whole block of
    `pool` tokens, with biases, a norm over the whole q and k projections, partial rotation, a capped score and a sink:

        q = rmsnorm_all(W_q x + b_q) * n_q     k = rmsnorm_all(W_k x + b_k) * n_k     v = W_v x + b_v
            (the root mean square runs over ALL heads of the projection at once; then the first rot_dims entries of
             each head of q and k are rotated, half-rotation pairing)
        the query at position i sees the keys j with 0 <= i - j < window, and block b (tokens b P .. b P + P - 1) through the
            mean of its P keys and the mean of its P values, as the cache holds them, if b P + P - 1 <= i - window
        s = softcap * tanh((q . k) * scale / softcap)
        out_h = sum_j exp(s_j) v_j / (sum_j exp(s_j) + exp(sink_h))          tokens and blocks in one softmax

    The keys and values of the last max(window, P) tokens stay in pages (a window group, whose pages go back as the
    window passes); the blocks' means live in a second group of pages with one entry for every P tokens
    (KVPages(every=P)), written by the step that completes a block.  W_q | W_k | W_v are one product with 32-bit output.

    Beside forward(), the mixer offers its steps apart (in_names / in_sizes, inner, `o`)."""
    recordable = True

    def __init__(self, rt: Runtime, prefix: str, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 softcap: float, position_encoding: Optional[PositionEncoding], window: int, pool: int, eps: float):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        if window <= 0 or pool <= 0:
            raise ValueError("pooled blocks lie behind a window: both sizes must be positive")
        self.rt, self.prefix, self.width = rt, prefix, width
        self.heads, self.kv_heads, self.dim, self.vdim = heads, kv_heads, dim, vdim
        self.scale, self.softcap, self.window, self.pool, self.eps = float(scale), float(softcap), int(window), int(pool), float(eps)
        self.position_encoding = position_encoding
        self.q_size, self.k_size, self.v_size, self.inner_size = heads * dim, kv_heads * dim, kv_heads * vdim, heads * vdim
        self.proj = Linear(rt, self.in_names(), width, self.in_sizes())
        self.o = Linear(rt, f"{prefix}.o", self.inner_size, width)
        self.q_b = self.k_b = self.v_b = self.q_norm_w = self.k_norm_w = self.sinks = None

    def in_names(self) -> list[str]:
        p = self.prefix
        return [f"{p}.q", f"{p}.k", f"{p}.v"]

    def in_sizes(self) -> list[int]:
        return [self.q_size, self.k_size, self.v_size]

    def children(self) -> list[Part]:
        return [self.proj, self.o]

    def param_specs(self) -> list[ParamSpec]:
        p = self.prefix
        return [ParamSpec(f"{p}.q.b", (self.q_size,), "linear"), ParamSpec(f"{p}.k.b", (self.k_size,), "linear"),
                ParamSpec(f"{p}.v.b", (self.v_size,), "linear"), ParamSpec(f"{p}.q.norm", (self.q_size,), "norm"),
                ParamSpec(f"{p}.k.norm", (self.k_size,), "norm"), ParamSpec(f"{p}.sink", (self.heads,), "linear")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        p = self.prefix
        f = lambda n: get(f"{p}.{n}").to(torch.float32).contiguous()
        self.q_b, self.k_b, self.v_b = f("q.b"), f("k.b"), f("v.b")
        self.q_norm_w, self.k_norm_w, self.sinks = f("q.norm"), f("k.norm"), f("sink")

    def plan_key(self) -> Optional[Hashable]:
        """The tile lists of the tensor-core kernels, as GQAttention's: they depend on the group size alone."""
        g = self.heads // self.kv_heads
        return ("attention tiles", g) if self.rt.fast_kernels and g <= TILE_ROWS and self.vdim == self.dim else None

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        g = self.heads // self.kv_heads
        if batch.max_q_len == 1:
            key = (g, len(batch.q_lens))
            hit = GQAttention._decode_plans.get(key)
            if hit is None:
                hit = GQAttention._decode_plans[key] = plan_tiles(batch, g)
            return hit
        return plan_tiles(batch, g)

    def cache_request(self) -> tuple:
        """(pages of the tokens inside the window, or of a block that is not complete yet; pages of the blocks' means)."""
        v = self.vdim if self.vdim != self.dim else 0
        return (KVPages(self.kv_heads, self.dim, max(self.window, self.pool), v_head_dim=v),
                KVPages(self.kv_heads, self.dim, 0, v_head_dim=v, every=self.pool))

    def inner(self, pre: torch.Tensor, step: StepContext, cache: tuple, out: torch.Tensor, out_scale: float = 1.0,
              write_cache: bool = True) -> None:
        """pre: float32 [T, >= sum(in_sizes())], the columns q | k | v of this mixer, which are changed in place; out:
        [T, inner_size] in the activation type (contiguous) receives the heads."""
        if not write_cache:
            raise ops.KernelError("attention with pooled blocks writes the cache it reads")
        if out_scale != 1.0 or not out.is_contiguous():
            raise ops.KernelError("attention with pooled blocks writes unscaled heads into a matrix of their own")
        rt = self.rt
        near, far = cache
        T, H, G, D, V = pre.shape[0], self.heads, self.kv_heads, self.dim, self.vdim
        c1, c2, c3 = self.q_size, self.q_size + self.k_size, self.q_size + self.k_size + self.v_size
        ops.bias_rmsnorm_cols(pre, [(0, self.q_size, self.q_b, self.q_norm_w), (c1, self.k_size, self.k_b, self.k_norm_w),
                                    (c2, self.v_size, self.v_b, None)], self.eps, rt.stream)
        rotary = self.position_encoding.rotary_table() if self.position_encoding is not None else None
        inv_freq, rot = rotary if rotary is not None else (None, 0)
        table, far_table = step.block_tables[near.group], step.block_tables[far.group]
        q = rt.empty((T, H, D))
        ops.rope_kv(pre[:, :c1], pre[:, c1:c2], pre[:, c2:c3], q, step.positions, H, G, D, 0.0, rt.stream, inv_freq=inv_freq, rot_dim=rot,
                    k_cache=near.k, v_cache=near.v, token_seq=step.token_seq, block_table=table, page_size=near.page_size, v_dim=V)
        ops.pool_kv(near.k, near.v, table, far.k, far.v, far_table, step, G, D, V, near.page_size, self.pool, rt.stream)
        ops.attention(q, out.view(T, H, V), near.k, near.v, step, near.group, H, G, D, near.page_size, self.window, self.scale,
                      rt.stream, plan=step.plans.get(self.plan_key()), v_dim=V if V != D else 0, softcap=self.softcap,
                      sinks=self.sinks, pool=self.pool, pool_k=far.k, pool_v=far.v, pool_group=far.group)

    def forward(self, h: torch.Tensor, step: StepContext, cache: tuple, write_cache: bool = True) -> torch.Tensor:
        pre = self.proj.forward(h, out_dtype=torch.float32)
        inner = self.rt.empty((h.shape[0], self.inner_size))
        self.inner(pre, step, cache, inner, 1.0, write_cache)
        return self.o.forward(inner, out_dtype=torch.float32)


def _attention_plan_key(rt: Runtime, heads: int, kv_heads: int, dim: int, vdim: int) -> Optional[Hashable]:
    """The tile lists of the tensor-core kernels, as GQAttention's: they depend on the group size alone."""
    g = heads // kv_heads
    return ("attention tiles", g) if rt.fast_kernels and g <= TILE_ROWS and vdim == dim else None


def _attention_plan(batch: BatchShape, heads: int, kv_heads: int) -> StepPlan:
    g = heads // kv_heads
    if batch.max_q_len == 1:
        key = (g, len(batch.q_lens))
        hit = GQAttention._decode_plans.get(key)
        if hit is None:
            hit = GQAttention._decode_plans[key] = plan_tiles(batch, g)
        return hit
    return plan_tiles(batch, g)


class TiedChunkAttention(Mixer):
    """Softmax attention whose values are its keys as projected, inside chunks of positions, with a sink of score 0:

        q = rotate(rmsnorm_head(W_q x) * n_q)      k = rotate(rmsnorm_head(c) * n_k)      v = c      with c = W_k x
            (per-head RMS norms with one weight [dim] for all heads; the first rot_dims entries of a head are rotated)
        the query at position i sees the keys j <= i with floor(j / chunk) = floor(i / chunk), chunks counted from the
            sequence's start (chunk 0: every j <= i)
        out_h = sum_j exp(s_j) v_j / (sink + sum_j exp(s_j)),   s_j = (q . k_j) * scale,   sink = 1 (a term of score 0
            without a value) or 0

    There is no value projection: the cache holds the normed, rotated keys and, as values, the same projection before
    norm and rotation.  A chunk's keys never reach back further than `chunk` tokens, so the pages are a window group of
    that length and go back as the chunk passes.  W_q | W_k are one product with 32-bit output.

    Beside forward(), the mixer offers its steps apart (in_names / in_sizes, inner, `o`)."""
    recordable = True

    def __init__(self, rt: Runtime, prefix: str, width: int, heads: int, kv_heads: int, dim: int, scale: float,
                 position_encoding: Optional[PositionEncoding], chunk: int, eps: float, sink: bool = True,
                 out_dtype: Optional[torch.dtype] = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        if position_encoding is not None and position_encoding.rotary_table() is None:
            raise ValueError("this attention rotates by a table of frequencies (rotary_table)")
        self.rt, self.prefix, self.width = rt, prefix, width
        self.heads, self.kv_heads, self.dim = heads, kv_heads, dim
        self.scale, self.chunk, self.eps, self.sink = float(scale), int(chunk), float(eps), bool(sink)
        self.position_encoding, self.out_dtype = position_encoding, out_dtype
        self.q_size, self.k_size, self.inner_size = heads * dim, kv_heads * dim, heads * dim
        self.proj = Linear(rt, self.in_names(), width, self.in_sizes())
        self.o = Linear(rt, f"{prefix}.o", self.inner_size, width)
        self.q_norm_w = self.k_norm_w = self.sinks = None

    def in_names(self) -> list[str]:
        return [f"{self.prefix}.q", f"{self.prefix}.k"]

    def in_sizes(self) -> list[int]:
        return [self.q_size, self.k_size]

    def children(self) -> list[Part]:
        return [self.proj, self.o]

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(f"{self.prefix}.q.norm", (self.dim,), "norm"), ParamSpec(f"{self.prefix}.k.norm", (self.dim,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.q_norm_w = get(f"{self.prefix}.q.norm").to(torch.float32).contiguous()
        self.k_norm_w = get(f"{self.prefix}.k.norm").to(torch.float32).contiguous()
        self.sinks = torch.zeros(self.heads, dtype=torch.float32, device=self.rt.device) if self.sink else None

    def plan_key(self) -> Optional[Hashable]:
        return _attention_plan_key(self.rt, self.heads, self.kv_heads, self.dim, self.dim)

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        return _attention_plan(batch, self.heads, self.kv_heads)

    def cache_request(self) -> KVPages:
        return KVPages(self.kv_heads, self.dim, self.chunk)

    def inner(self, pre: torch.Tensor, step: StepContext, cache: KVCacheView, out: torch.Tensor, out_scale: float = 1.0,
              write_cache: bool = True) -> None:
        """pre: float32 [T, >= sum(in_sizes())], the columns q | k of this mixer; out: [T, inner_size] in the activation type
        (contiguous) receives the heads."""
        if out_scale != 1.0 or not out.is_contiguous():
            raise ops.KernelError("this attention writes unscaled heads into a matrix of their own")
        rt = self.rt
        T, H, G, D = pre.shape[0], self.heads, self.kv_heads, self.dim
        k_in = pre[:, self.q_size:self.q_size + self.k_size]
        rotary = self.position_encoding.rotary_table() if self.position_encoding is not None else None
        inv_freq, rot = rotary if rotary is not None else (None, 0)
        q = rt.empty((T, H, D))
        # the keys' projection goes in twice: normed and rotated as keys, and as it is as values
        ops.rope_kv(pre[:, :self.q_size], k_in, k_in, q, step.positions, H, G if write_cache else 0, D, self.eps, rt.stream,
                    q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, inv_freq=inv_freq, rot_dim=rot, k_cache=cache.k, v_cache=cache.v,
                    token_seq=step.token_seq, block_table=step.block_tables[cache.group], page_size=cache.page_size,
                    rot_scale=getattr(self.position_encoding, "magnitude", 1.0))
        ops.attention(q, out.view(T, H, D), cache.k, cache.v, step, cache.group, H, G, D, cache.page_size, 0, self.scale, rt.stream,
                      plan=step.plans.get(self.plan_key()), sinks=self.sinks, chunk=self.chunk)

    def forward(self, h: torch.Tensor, step: StepContext, cache: KVCacheView, write_cache: bool = True) -> torch.Tensor:
        pre = self.proj.forward(h, out_dtype=torch.float32)
        inner = self.rt.empty((h.shape[0], self.inner_size))
        self.inner(pre, step, cache, inner, 1.0, write_cache)
        return self.o.forward(inner, out_dtype=self.out_dtype)


class GatedWindowAttention(Mixer):
    """Softmax attention over a sliding window with biases on q, k and v, rotation (whose sines and cosines may carry a
    magnitude, as with YaRN) and an elementwise sigmoid gate on the heads:

        q = rotate(W_q x + b_q)      k = rotate(W_k x + b_k)      v = W_v x + b_v
        the query at position i sees the keys j with 0 <= i - j < window (window 0: every j <= i)
        out = softmax(q . k * scale) v * sigmoid(W_g x)           (the gate has heads * vdim entries)

    Values may have another size than keys.  W_q | W_k | W_v | W_g are one product with 32-bit output; the biases are
    added to it in 32-bit.  Beside forward(), the mixer offers its steps apart (in_names / in_sizes, inner, `o`)."""
    recordable = True

    def __init__(self, rt: Runtime, prefix: str, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 position_encoding: Optional[PositionEncoding], window: int, out_dtype: Optional[torch.dtype] = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        if position_encoding is not None and position_encoding.rotary_table() is None:
            raise ValueError("this attention rotates by a table of frequencies (rotary_table)")
        self.rt, self.prefix, self.width = rt, prefix, width
        self.heads, self.kv_heads, self.dim, self.vdim = heads, kv_heads, dim, vdim
        self.scale, self.window = float(scale), int(window)
        self.position_encoding, self.out_dtype = position_encoding, out_dtype
        self.q_size, self.k_size, self.v_size, self.inner_size = heads * dim, kv_heads * dim, kv_heads * vdim, heads * vdim
        self.proj = Linear(rt, self.in_names(), width, self.in_sizes())
        self.o = Linear(rt, f"{prefix}.o", self.inner_size, width)
        self.q_b = self.k_b = self.v_b = None

    def in_names(self) -> list[str]:
        p = self.prefix
        return [f"{p}.q", f"{p}.k", f"{p}.v", f"{p}.g"]

    def in_sizes(self) -> list[int]:
        return [self.q_size, self.k_size, self.v_size, self.inner_size]

    def children(self) -> list[Part]:
        return [self.proj, self.o]

    def param_specs(self) -> list[ParamSpec]:
        p = self.prefix
        return [ParamSpec(f"{p}.q.b", (self.q_size,), "linear"), ParamSpec(f"{p}.k.b", (self.k_size,), "linear"),
                ParamSpec(f"{p}.v.b", (self.v_size,), "linear")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        f = lambda n: get(f"{self.prefix}.{n}").to(torch.float32).contiguous()
        self.q_b, self.k_b, self.v_b = f("q.b"), f("k.b"), f("v.b")

    def plan_key(self) -> Optional[Hashable]:
        return _attention_plan_key(self.rt, self.heads, self.kv_heads, self.dim, self.vdim)

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        return _attention_plan(batch, self.heads, self.kv_heads)

    def cache_request(self) -> KVPages:
        return KVPages(self.kv_heads, self.dim, self.window, v_head_dim=self.vdim if self.vdim != self.dim else 0)

    def inner(self, pre: torch.Tensor, step: StepContext, cache: KVCacheView, out: torch.Tensor, out_scale: float = 1.0,
              write_cache: bool = True) -> None:
        """pre: float32 [T, >= sum(in_sizes())], the columns q | k | v | g of this mixer, of which q, k, v are changed in
        place; out: [T, inner_size] in the activation type (may be a column range of a wider matrix) receives the gated
        heads times out_scale."""
        rt = self.rt
        T, H, G, D, V = pre.shape[0], self.heads, self.kv_heads, self.dim, self.vdim
        c1, c2, c3 = self.q_size, self.q_size + self.k_size, self.q_size + self.k_size + self.v_size
        ops.bias_rmsnorm_cols(pre, [(0, self.q_size, self.q_b, None), (c1, self.k_size, self.k_b, None), (c2, self.v_size, self.v_b, None)],
                              0.0, rt.stream)
        rotary = self.position_encoding.rotary_table() if self.position_encoding is not None else None
        inv_freq, rot = rotary if rotary is not None else (None, 0)
        q = rt.empty((T, H, D))
        ops.rope_kv(pre[:, :c1], pre[:, c1:c2], pre[:, c2:c3], q, step.positions, H, G if write_cache else 0, D, 0.0, rt.stream,
                    inv_freq=inv_freq, rot_dim=rot, k_cache=cache.k, v_cache=cache.v, token_seq=step.token_seq,
                    block_table=step.block_tables[cache.group], page_size=cache.page_size, v_dim=V,
                    rot_scale=getattr(self.position_encoding, "magnitude", 1.0))
        heads = rt.empty((T, H, V))
        ops.attention(q, heads, cache.k, cache.v, step, cache.group, H, G, D, cache.page_size, self.window, self.scale, rt.stream,
                      plan=step.plans.get(self.plan_key()), v_dim=V if V != D else 0)
        # an elementwise gate is a gate of one number a "head" of one entry
        ops.head_gate(out, heads.view(T, H * V, 1), pre[:, c3:c3 + H * V], out_scale, rt.stream)

    def forward(self, h: torch.Tensor, step: StepContext, cache: KVCacheView, write_cache: bool = True) -> torch.Tensor:
        pre = self.proj.forward(h, out_dtype=torch.float32)
        inner = self.rt.empty((h.shape[0], self.inner_size))
        self.inner(pre, step, cache, inner, 1.0, write_cache)
        return self.o.forward(inner, out_dtype=self.out_dtype)
