"""The plain Nelovik implementation against hand-made values and against itself (whole, portions, token by token), the
configuration reader, and the cache manager's page groups with one entry for every block of tokens (CPU)."""
import math

import pytest
import torch

import nelovik_util as nz
import plain_nelovik as plain

F = torch.float64


def test_xielu_by_hand():
    sp = lambda x: math.log1p(math.exp(x))
    z = torch.tensor([2.0, -1.0, 0.0], dtype=F)
    got = plain.xielu(z, 0.3, -0.7)
    assert math.isclose(got[0].item(), sp(0.3) * 4 + 1.0)
    assert math.isclose(got[1].item(), (0.5 + sp(-0.7)) * (math.exp(-1) - 1 + 1) - 0.5)
    assert got[2].item() == 0.0


def test_short_conv_by_hand():
    # two channels, three taps; the last column weighs the current token
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 2.0]], dtype=F)
    x = torch.tensor([[1.0, 1.0], [2.0, 1.0], [3.0, 1.0]], dtype=F)
    y, past = plain.short_conv(x, w, torch.tensor([0.5, 0.0], dtype=F), None)
    assert y.tolist() == [[100.5, 2.0], [210.5, 2.0], [321.5, 2.0]]
    assert past.tolist() == [[2.0, 1.0], [3.0, 1.0]]
    y2, _ = plain.short_conv(torch.tensor([[4.0, 1.0]], dtype=F), w, None, past)
    assert y2.tolist() == [[432.0, 2.0]]
    # one tap: no past at all
    y1, p1 = plain.short_conv(x, w[:, 2:], None, None)
    assert y1.tolist() == [[100.0, 2.0], [200.0, 2.0], [300.0, 2.0]] and p1.shape[0] == 0


def test_delta_rule_by_hand():
    """One head, one channel: q and k become +1 (unit vectors of one entry, q times dim^-1/2 = 1), so with g and w known the
    state follows S <- g S + w (v - g S) by hand."""
    one = torch.ones(1, 1, dtype=F)
    big = 40.0                                          # silu(40) = 40, and 40 / sqrt(1600 + 1e-6) = 1
    w = {"q": one, "k": one, "v": one, "q.conv": one, "k.conv": one, "v.conv": one, "b": torch.zeros(1, 1, dtype=F),
         "a": torch.zeros(1, 1, dtype=F), "A_log": torch.zeros(1, dtype=F), "dt_bias": torch.zeros(1, dtype=F),
         "g": one * 0.0 + 1.0, "norm": torch.ones(1, dtype=F), "o": one}
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "conv": 1}
    h = torch.full((3, 1), big, dtype=F)
    out, (_, _, _, S) = plain.gated_delta_rule(h, w, m, 0.0, None)
    g, beta, v = math.exp(-math.log(2.0)), 0.5, big     # softplus(0) = ln 2, sigmoid(0) = 1/2
    s = 0.0
    for _ in range(3):
        s = g * s
        s = s + beta * (v - s)
    assert math.isclose(S.item(), s, rel_tol=1e-9)
    # the norm leaves the sign; the gate is silu(40) = 40
    assert torch.allclose(out.flatten(), torch.full((3,), big, dtype=F))


def test_pooled_window_by_hand():
    """One head, a scale of zero: every visible key weighs the same, so the output is the mean of what is visible with the
    sink as one more, valueless entry.  Window 2, blocks of 2: position 5 sees tokens 4 and 5 and the blocks (0, 1), (2, 3);
    position 4 sees tokens 3, 4 and block (0, 1) only, token 2 is seen by nobody."""
    d = 2
    eye = torch.eye(d, dtype=F)
    w = {"q": eye, "k": eye, "v": eye, "q.b": torch.zeros(d, dtype=F), "k.b": torch.zeros(d, dtype=F), "v.b": torch.zeros(d, dtype=F),
         "q.norm": torch.ones(d, dtype=F), "k.norm": torch.ones(d, dtype=F), "sink": torch.zeros(1, dtype=F), "o": eye}
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "scale": 0.0, "softcap": 7.0, "rot": {"dims": 0, "base": 10.0},
         "mask": {"size": 2, "pool": 2}}
    h = torch.zeros(6, d, dtype=F)
    h[:, 0] = torch.tensor([1.0, 3.0, 10.0, 30.0, 100.0, 300.0])
    out, _ = plain.pooled_window_attention(h, w, m, 0.0, None)
    assert math.isclose(out[5, 0].item(), (100 + 300 + 2 + 20) / 5)          # two tokens, two blocks, the sink
    assert math.isclose(out[4, 0].item(), (30 + 100 + 2) / 4)
    assert math.isclose(out[1, 0].item(), (1 + 3) / 3)
    # in portions the cache hands the same keys on
    a, past = plain.pooled_window_attention(h[:3], w, m, 0.0, None)
    b, _ = plain.pooled_window_attention(h[3:], w, m, 0.0, past)
    assert torch.allclose(torch.cat([a, b]), out)


def test_state_space_by_hand():
    """One head, one channel, N = 1, one tap with weight 1: x, B, C = silu(40) = 40 each; S <- e^(-dt) S + dt B x, y = C S + D x."""
    inner = 1
    w = {"in": torch.tensor([[0.0], [1.0], [1.0], [1.0], [0.0]], dtype=F), "conv": torch.ones(3, 1, dtype=F), "conv.b": torch.zeros(3, dtype=F),
         "dt_bias": torch.zeros(1, dtype=F), "A_log": torch.zeros(1, dtype=F), "D": torch.tensor([2.0], dtype=F),
         "norm": torch.ones(1, dtype=F), "o": torch.ones(1, 1, dtype=F)}
    m = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "norm_groups": 1, "conv": 1}
    h = torch.full((2, 1), 40.0, dtype=F)
    _, (_, S) = plain.mamba2(h, w, m, 0.0, None)
    dt = math.log(2.0)
    s = dt * 1600.0
    s = math.exp(-dt) * s + dt * 1600.0
    assert math.isclose(S.item(), s, rel_tol=1e-9)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_plain_whole_against_portions_and_single_tokens(name):
    cfg = nz.CONFIGS[name]
    w = nz.make_weights(cfg, 5)
    ids = nz.tokens(cfg, 61, salt=2)
    model = plain.PlainNelovik(cfg, w)
    whole = model.forward(ids)
    for sizes in ((7, 2, 13, 3, 2, 31, 1, 2), (1,) * 61):
        past, rows, at = None, [], 0
        for n in sizes:
            if at >= len(ids):
                break
            got, past = model.run(ids[at:at + n], past)
            rows.append(got)
            at += n
        assert (torch.cat(rows) - whole[:at]).abs().max() <= 1e-9 * whole.abs().max()


def test_sharpened_weights_make_single_keys_and_blocks_matter():
    """Replacing the token just inside the window, or one token of the block that has just become visible, changes the
    last logits; replacing a token that has left the window and whose block is not yet complete does not."""
    cfg = nz._config(50, 32, 1e-6, [nz._pair(nz._left(2, 1, 16, 16, 0.25, 30.0, 8, 100.0, 8, 2), nz._right(1, 8, 4, 1, 1, 2), None)])
    w = nz.make_weights(cfg, 3, sharp=6.0)
    for k in list(w):
        if ".right." in k and (k.endswith(".o") or k.endswith(".in")):
            w[k] = torch.zeros_like(w[k])                   # only the attention speaks
    ids = nz.tokens(cfg, 23, salt=1)                        # last position 22: window 15..22, blocks b with 2 b + 1 <= 14: 0 .. 6
    base = plain.PlainNelovik(cfg, w).forward(ids)[-1]

    def changed(at):
        other = list(ids)
        other[at] = (ids[at] + 7) % 50
        return (plain.PlainNelovik(cfg, w).forward(other)[-1] - base).abs().max().item() / base.abs().max().item()
    assert changed(15) > 1e-2 and changed(13) > 1e-4 and changed(0) > 1e-3          # window's edge, last block seen, first block
    assert changed(14) == 0.0                                                       # out of the window, and block 7 ends at 15 > 14


# ---- configuration ----------------------------------------------------------------------------------------------------
def test_config_reads_every_key_and_round_trips():
    from lucciola_b200.config.nelovik_config import NelovikConfig
    from lucciola_b200.config.registry import resolve_architecture
    for cfg in nz.CONFIGS.values():
        c = NelovikConfig.from_dict(cfg)
        assert c.to_dict() == cfg
        assert resolve_architecture(cfg).name == "Nelovik"
    c = NelovikConfig.from_dict(nz.CONFIGS["A"])
    assert c.layers[1].left.pool == 5 and c.layers[1].left.window == 24 and c.layers[1].right.norm_groups == 3
    assert c.layers[2].type == "delta_2" and c.layers[2].ff is None and c.layers[0].delta.conv == 3


@pytest.mark.parametrize("path,value", [(("layers", 0, "type"), "gamma"), (("layers", 1, "mixer", "left", "mask", "pool"), None),
                                        (("layers", 1, "mixer", "left", "rot", "dims"), 11), (("layers", 0, "mixer", "kv_heads"), 2),
                                        (("layers", 1, "mixer", "right", "norm_groups"), 7), (("layers", 0, "mlp", "kind"), "moe"),
                                        (("norm", "eps"), None), (("layers", 1, "mixer", "left", "softcap"), 0.0)])
def test_config_refuses_what_it_does_not_know(path, value):
    import copy

    from lucciola_b200.config.model_config import ConfigError
    from lucciola_b200.config.nelovik_config import NelovikConfig
    cfg = copy.deepcopy(nz.CONFIGS["A"])
    d = cfg
    for k in path[:-1]:
        d = d[k]
    if value is None:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    with pytest.raises(ConfigError):
        NelovikConfig.from_dict(cfg)


def test_model_asks_for_the_tensors_the_weights_hold():
    from lucciola_b200.config.registry import resolve_architecture
    from lucciola_b200.parts.base import KVPages, Runtime, StateSlot
    for name, cfg in nz.CONFIGS.items():
        arch = resolve_architecture(cfg)
        model = arch.build(arch.config_from_dict(cfg), Runtime("cpu", torch.float32))
        specs = {s.name: tuple(s.shape) for s in model.all_param_specs()}
        w = nz.make_weights(cfg, 1)
        extra = set(model.ignored_names())
        assert set(specs) == set(w) - extra, name
        assert all(tuple(w[n].shape) == s for n, s in specs.items()), name
    cfg = nz.CONFIGS["A"]
    arch = resolve_architecture(cfg)
    reqs = arch.build(arch.config_from_dict(cfg), Runtime("cpu", torch.float32)).cache_requests()
    assert reqs[0] == (StateSlot((2, 2 * 20 + 36), torch.float32), StateSlot((3, 20, 12), torch.float32))
    near, far, conv, state = reqs[1]
    assert near == KVPages(2, 24, 24, v_head_dim=16) and far == KVPages(2, 24, 0, v_head_dim=16, every=5)
    assert reqs[3][0].window == 9                         # blocks longer than the window: a block's tokens stay until it is complete


# ---- pages with one entry for every block of tokens --------------------------------------------------------------------
def test_page_groups_with_an_entry_a_block():
    from lucciola_b200.cache.manager import CacheManager, plan_groups
    from lucciola_b200.parts.base import KVPages
    groups, _ = plan_groups([(KVPages(2, 8, 12), KVPages(2, 8, 0, every=5))])
    assert [g.every for g in groups] == [1, 5]
    m = CacheManager(groups, 4, [10, 3], 2)
    m.admit("a")
    assert m.pages_needed("a", 19) == [5, 1]              # 19 tokens: 5 pages of tokens, 3 whole blocks in one page
    assert m.extend("a", 19)
    assert m.pages_needed("a", 20) == [0, 0] and m.pages_needed("a", 25) == [2, 1]        # the fifth block opens a second page
    assert m.extend_by_one(["a"]) == [19]
    assert not m.extend("a", 45)                          # twelve pages of tokens, the pool has ten
    assert m.extend("a", 40) and len(m.block_table("a", 1)) == 2
    assert m.max_extension("a", 1000) == 40               # the tokens' pages run out first
    freed = m.release_behind_window("a")                  # the window group gives pages back, the blocks' group never does
    assert freed == 7 and all(p >= 0 for p in m.block_table("a", 1))
    assert m.max_extension("a", 1000) == 64               # now the blocks' pages: three pages hold twelve blocks, the 13th starts at 60, ends at 64
    m.check_invariants()
    m.release("a")
    assert [p.num_free for p in m.pools] == [10, 3]
