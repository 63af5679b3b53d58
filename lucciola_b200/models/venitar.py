"""The Venitar decoder, composed from parts.

    e = embed[token] * embedding.scale;   x = e
    the layers in order, of which layers loop.start .. loop.stop - 1 run loop.times times in a row (same weights, a cache
    of its own for every pass; x += e before every pass but the first):
        x += mixer(n1(x));   x += ffn(n2(x))                                       (PreNormBlock; a layer may have no ffn)
        mixer: retention   decay linear attention on rotated q and k, head-wise norm without weight, silu gate
               attention   softmax attention in chunks, values = keys as projected, per-head q/k norms, a sink of score 0
               parallel    left_scale * window attention (biases, YaRN rotation, sigmoid gate)
                           + right_scale * gated delta rule with a decay for every key channel        (SideBySideMixer)
        ffn:   down( relu(up h)^2 )
    logits = embed . rmsnorm(x)                                                      (the table itself, unscaled)

Tensor names: embed, final.norm and, for layer i, l<i>.norm1, l<i>.norm2, l<i>.mlp.{up,down} and
  retention:  l<i>.mix.{q,k,v,g,o}
  attention:  l<i>.mix.{q,k,o}, {q,k}.norm
  parallel:   l<i>.mix.left.{q,k,v,g,o}, {q,k,v}.b;  l<i>.mix.right.{q,k,v,b,a1,a2,g1,g2,o}, {q,k,v}.conv, A_log, dt_bias, norm
The attention layers keep pages of keys and values (window groups: a chunk's or a window's pages go back as it passes),
the recurrent ones a 32-bit state slot, the delta rule also the last inputs of its convolutions.
"""
from __future__ import annotations

import torch

from ..config.model_config import ConfigError
from ..config.registry import register_architecture
from ..config.venitar_config import RotarySpec, VenitarConfig
from ..parts.attention import GatedWindowAttention, TiedChunkAttention
from ..parts.base import Runtime
from ..parts.block import PreNormBlock
from ..parts.decay_attention import DecayLinearAttention
from ..parts.delta_rule import GatedDeltaRule
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.mlp import DenseFeedForward
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEmbedding
from ..parts.side_by_side import SideBySideMixer
from .decoder import DecoderModel, LayerCall


def _rotary(rt: Runtime, dim: int, r: RotarySpec):
    if r.dims <= 0:
        return None
    return RotaryEmbedding(rt, dim, r.base, r.dims, yarn=(r.factor, r.original, r.fast, r.slow) if r.factor else None)


def build_venitar(cfg: VenitarConfig, rt: Runtime) -> DecoderModel:
    W, eps, f32 = cfg.width, cfg.norm_eps, torch.float32
    embedding = TokenEmbedding(rt, "embed", cfg.vocab, W, scale=cfg.embedding_scale)
    blocks = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        if l.retention is not None:
            s = l.retention
            mixer = DecayLinearAttention(rt, f"{p}.mix", W, s.heads, s.dim, s.vdim, s.decay, eps, act=None,
                                         position_encoding=_rotary(rt, s.dim, s.rot), k_scale=s.dim ** -0.5, head_norm=True,
                                         norm_weight=False, gate_act="silu", out_dtype=f32)
        elif l.attention is not None:
            a = l.attention
            mixer = TiedChunkAttention(rt, f"{p}.mix", W, a.heads, a.kv_heads, a.dim, a.scale, _rotary(rt, a.dim, a.rot), a.mask, eps,
                                       sink=True, out_dtype=f32)
        else:
            a, r = l.left, l.right
            if not (r.decay_rank > 0 and r.gate_rank > 0):
                raise ConfigError(f"layers[{i}].right: the ranks of the decay's and the gate's maps are unknown: config.json does "
                                  "not name them (decay_rank, gate_rank) and no checkpoint was read for the shapes of a1 and g1")
            left = GatedWindowAttention(rt, f"{p}.mix.left", W, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, _rotary(rt, a.dim, a.rot),
                                        a.mask)
            right = GatedDeltaRule(rt, f"{p}.mix.right", W, r.heads, r.kv_heads, r.dim, r.vdim, r.conv, eps,
                                   decay_rank=r.decay_rank, gate_rank=r.gate_rank, gate_act="sigmoid")
            mixer = SideBySideMixer(rt, W, left, right, l.left_scale, l.right_scale)
        ffn = ffn_norm = None
        if l.ff is not None:
            ffn = DenseFeedForward(rt, f"{p}.mlp.up", f"{p}.mlp.down", W, l.ff, act="relu2", out_dtype=f32)
            ffn_norm = RMSNorm(rt, f"{p}.norm2", W, eps)
        blocks.append(PreNormBlock(mixer, ffn, RMSNorm(rt, f"{p}.norm1", W, eps), ffn_norm, rt.act_dtype))
    # the order of runs: the layers before the loop, the looped run `times` times, the rest; a cache for every run
    a, b, n = cfg.loop_start, cfg.loop_stop, len(blocks)
    order = [(i, False) for i in range(a)]
    for t in range(cfg.loop_times if b > a else 0):
        order += [(i, t > 0 and i == a) for i in range(a, b)]
    order += [(i, False) for i in range(b, n)]
    calls = [LayerCall(i, j, True, add) for j, (i, add) in enumerate(order)]
    final_norm = RMSNorm(rt, "final.norm", W, eps)
    head = OutputHead(rt, "head", cfg.vocab, W, embedding)
    unused = [f"l{i}.norm2" for i, l in enumerate(cfg.layers) if l.ff is None]       # the norm of a feed-forward that is not there
    return DecoderModel(rt, embedding, blocks, calls, final_norm, head, cfg.vocab, 0, cfg.eos_token_ids, ignored_names=unused)


register_architecture(VenitarConfig.ARCHITECTURE, VenitarConfig.from_dict, build_venitar, replace=True)
