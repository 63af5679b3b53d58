"""The Nelovik decoder, composed from parts.

    x = embed[token]
    each layer:  x += mixer(n1(x)) + ffn(n2(x))            (ParallelBlock with a norm for each sublayer, both of the same x)
        mixer: the gated delta rule (`delta`, `delta_2`), or
               1/2 ( rmsnorm(attention(h)) * w_l + rmsnorm(state_space(h)) * w_r )      (`parallel`: NormedPairMixer)
        ffn:   down( xielu(up h) )
    logits = head . rmsnorm(x)

Tensor names: embed, head, final.norm and, for layer i, l<i>.norm1, l<i>.norm2, l<i>.mlp.{up,down,act} and
  delta rule:  l<i>.mix.{q,k,v,g,b,a,o}, {q,k,v}.conv, A_log, dt_bias, norm
  parallel:    l<i>.mix.left.{q,k,v,o}, {q,k,v}.b, {q,k}.norm, sink;  l<i>.mix.right.{in,conv,conv.b,dt_bias,A_log,D,norm,o};
               l<i>.mix.left.out, l<i>.mix.right.out
The delta rule and the state space keep a 32-bit state slot and the last inputs of their convolutions; the attention
keeps pages of the keys and values inside its window and pages of the means of the blocks behind it.
"""
from __future__ import annotations

import torch

from ..config.nelovik_config import NelovikConfig
from ..config.registry import register_architecture
from ..parts.attention import PooledWindowAttention
from ..parts.base import Runtime
from ..parts.block import ParallelBlock
from ..parts.delta_rule import GatedDeltaRule
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.mlp import DenseFeedForward
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEmbedding
from ..parts.side_by_side import NormedPairMixer
from ..parts.state_space import SelectiveStateSpace
from .decoder import DecoderModel, LayerCall

PAIR_SCALE = 0.5            # the two mixers of a `parallel` layer count half each


def build_nelovik(cfg: NelovikConfig, rt: Runtime) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    embedding = TokenEmbedding(rt, "embed", cfg.vocab, W)
    blocks = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        if l.delta is not None:
            s = l.delta
            mixer = GatedDeltaRule(rt, f"{p}.mix", W, s.heads, s.kv_heads, s.dim, s.vdim, s.conv, eps)
        else:
            a, r = l.left, l.right
            rotary = RotaryEmbedding(rt, a.dim, a.rot_base, a.rot_dims) if a.rot_dims > 0 else None
            left = PooledWindowAttention(rt, f"{p}.mix.left", W, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.softcap, rotary,
                                         a.window, a.pool, eps)
            right = SelectiveStateSpace(rt, f"{p}.mix.right", W, r.heads, r.vdim, r.state, r.groups, r.norm_groups, r.conv, eps)
            mixer = NormedPairMixer(rt, W, left, right, f"{p}.mix.left.out", f"{p}.mix.right.out", PAIR_SCALE, PAIR_SCALE, eps)
        ffn = ffn_norm = None
        if l.ff is not None:
            ffn = DenseFeedForward(rt, f"{p}.mlp.up", f"{p}.mlp.down", W, l.ff, act="xielu", act_name=f"{p}.mlp.act", out_dtype=torch.float32)
            ffn_norm = RMSNorm(rt, f"{p}.norm2", W, eps)
        blocks.append(ParallelBlock(mixer, ffn, RMSNorm(rt, f"{p}.norm1", W, eps), rt.act_dtype, ffn_norm=ffn_norm))
    calls = [LayerCall(i, i) for i in range(len(blocks))]
    final_norm = RMSNorm(rt, "final.norm", W, eps)
    head = OutputHead(rt, "head", cfg.vocab, W, None)
    unused = [f"l{i}.norm2" for i, l in enumerate(cfg.layers) if l.ff is None]       # the norm of a feed-forward that is not there
    return DecoderModel(rt, embedding, blocks, calls, final_norm, head, cfg.vocab, 0, cfg.eos_token_ids, ignored_names=unused)


register_architecture(NelovikConfig.ARCHITECTURE, NelovikConfig.from_dict, build_nelovik, replace=True)
