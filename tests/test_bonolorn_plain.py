"""The plain Bonolorn implementation against hand-made values and against itself (whole, portions, token by token), and
the configuration reader (CPU)."""
import math

import pytest
import torch

import bonolorn_util as bz
import plain_bonolorn as plain


def test_sinusoid_by_hand():
    p = plain.sinusoid_positions(torch.tensor([0, 3]), 4, base=100.0)
    assert torch.allclose(p[0], torch.tensor([0.0, 1.0, 0.0, 1.0], dtype=torch.float64))
    assert torch.allclose(p[1], torch.tensor([math.sin(3.0), math.cos(3.0), math.sin(0.3), math.cos(0.3)], dtype=torch.float64))


def test_layer_norm_and_activations_by_hand():
    x = torch.tensor([[1.0, 3.0]], dtype=torch.float64)
    y = plain.layer_norm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    assert torch.allclose(y, torch.tensor([[-2.0, 0.5]], dtype=torch.float64))
    assert math.isclose(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64)).item(),
                        0.5 * (1 + math.tanh(math.sqrt(2 / math.pi) * 1.044715)))
    # the clamp comes before everything else: g = min(3, 1) = 1, u = clamp(-5) = -1, so (u + 1) = 0
    one = torch.ones(1, 1, dtype=torch.float64)
    assert plain.clamped_expert(one, 3 * one, -5 * one, one, 1.0).item() == 0.0
    got = plain.clamped_expert(one, -2 * one, 0.5 * one, 2 * one, 1.0).item()
    assert math.isclose(got, 2 * (-2 / (1 + math.exp(1.702 * 2))) * 1.5)


def test_slopes_and_window_by_hand():
    assert plain.distance_slopes(4).tolist() == [0.25, 0.0625, 0.015625, 0.00390625]
    # one head, keys and queries all equal, values the positions: with a window of 2 a query sees itself and one before
    T, d = 5, 4
    eye = torch.eye(d, dtype=torch.float64)
    w = {"q": eye, "k": eye, "v": eye, "q.norm": torch.ones(d, dtype=torch.float64), "k.norm": torch.ones(d, dtype=torch.float64),
         "g": torch.zeros(1, d, dtype=torch.float64), "o": eye}
    h = torch.ones(T, d, dtype=torch.float64)
    h[:, 0] = torch.arange(T, dtype=torch.float64)
    # give every token the same key by norming: the rows differ, so use a zero scale instead (scores = minus the bias alone)
    out, k, v = plain.window_attention(h, w, 1, 1, d, d, 0.0, 2, 1e-6)
    slope = 2.0 ** -8
    a = 1 / (1 + math.exp(-slope))                 # weight of the token itself against the one before
    want = [0.0] + [0.5 * (a * t + (1 - a) * (t - 1)) for t in range(1, T)]      # the gate is sigmoid(0) = 1/2
    assert torch.allclose(out[:, 0], torch.tensor(want, dtype=torch.float64))


def test_decay_attention_by_hand():
    # one head, one channel each: S_t = d S + k v, o = S q; the norm leaves the sign, the gate is 1/2
    big = 50.0                                      # silu(50) = 50
    w = {n: torch.tensor([[1.0]], dtype=torch.float64) for n in ("q", "k", "v", "o")}
    w["g"], w["norm"] = torch.zeros(1, 1, dtype=torch.float64), torch.ones(1, dtype=torch.float64)
    out, S = plain.decay_attention(torch.full((3, 1), big, dtype=torch.float64), w, 1, 1, 1, [0.5], 0.0)
    assert math.isclose(S.item(), big * big * (1 + 0.5 + 0.25), rel_tol=1e-12)
    assert torch.allclose(out.flatten(), torch.full((3,), 0.5, dtype=torch.float64))


def test_router_by_hand():
    # six experts in three groups; the corrections push group 0 down, so the best pair is groups 1 and 2
    z = torch.tensor([[4.0, 3.0, 0.0, 1.0, 0.5, -1.0]], dtype=torch.float64)
    corr = torch.tensor([-2.0, -2.0, 0.0, 0.0, 0.0, 0.0], dtype=torch.float64)
    chosen, weights = plain.route(z, torch.eye(6, dtype=torch.float64), corr, 2, 3, 2, 1.5)
    s = torch.sigmoid(z[0])
    assert chosen[0].tolist() == [3, 4]
    assert torch.allclose(weights[0], s[[3, 4]] / (s[3] + s[4]) * 1.5)          # the weights are the plain scores
    # negative choice scores: an expert of a dropped group must not come back because the kept ones are below zero
    corr = torch.tensor([0.0, 0.0, -3.0, -3.0, -9.0, -9.0], dtype=torch.float64)
    chosen, _ = plain.route(z, torch.eye(6, dtype=torch.float64), corr, 3, 3, 2, 1.0)
    assert sorted(chosen[0].tolist()) == [0, 1, 3]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_portions_and_single_tokens_agree(name):
    cfg = bz.CONFIGS[name]
    w = bz.make_weights(cfg, 11)
    ids = bz.tokens(cfg, 70, salt=1)
    model = plain.PlainBonolorn(cfg, w)
    whole = model.forward(ids)
    for sizes in ([70], [1] * 70, [7, 2, 13, 3, 2, 31, 1, 11]):
        st, rows, at = model.new_state(), [], 0
        for n in sizes:
            rows.append(model.step(ids[at:at + n], st))
            at += n
        assert at == 70 and (torch.cat(rows) - whole).abs().max() <= 1e-9 * whole.abs().max()


def test_a_key_behind_the_window_does_not_matter_and_the_state_does():
    cfg = bz.CONFIGS["A"]
    w = bz.make_weights(cfg, 12)
    model = plain.PlainBonolorn(cfg, w)
    ids = bz.tokens(cfg, 90, salt=2)
    other = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]
    a, b = model.forward(ids)[-1], model.forward(other)[-1]
    assert (a - b).abs().max() > 1e-9            # the first token is far behind every window, but the slow decays carry it
    only_left = {k: (v * 0 if ".mix.right.o" in k else v) for k, v in w.items()}
    m2 = plain.PlainBonolorn(cfg, only_left)
    # without the recurrent half nothing reaches the last token from beyond the windows stacked over the layers
    assert (m2.forward(ids)[-1] - m2.forward(other)[-1]).abs().max() == 0.0


def test_configuration_reader():
    from lucciola_b200.config import ConfigError, resolve_architecture
    from lucciola_b200.config.bonolorn_config import BonolornConfig
    for cfg in bz.CONFIGS.values():
        arch = resolve_architecture(cfg)
        c = arch.config_from_dict(cfg)
        assert isinstance(c, BonolornConfig) and c.to_dict() == cfg
    for seed in range(20):
        cfg = bz.random_config(seed)
        assert BonolornConfig.from_dict(cfg).to_dict() == cfg
    bad = {**bz.CONFIGS["B"], "layers": [{**bz.CONFIGS["B"]["layers"][0], "type": "serial"}]}
    with pytest.raises(ConfigError):
        BonolornConfig.from_dict(bad)
    no_mult = {k: v for k, v in bz.CONFIGS["B"].items() if k != "residual_mult"}
    with pytest.raises(ConfigError):
        BonolornConfig.from_dict(no_mult)
    import copy
    wrong = copy.deepcopy(bz.CONFIGS["A"])
    wrong["layers"][1]["mlp"]["router"]["top"] = 5           # more than the kept groups hold
    with pytest.raises(ConfigError):
        BonolornConfig.from_dict(wrong)
    wrong = copy.deepcopy(bz.CONFIGS["A"])
    wrong["layers"][0]["mixer"]["right"]["decay"] = [0.5]
    with pytest.raises(ConfigError):
        BonolornConfig.from_dict(wrong)


def test_model_names_every_tensor_of_its_checkpoint():
    from lucciola_b200.config import resolve_architecture
    from lucciola_b200.parts.base import Runtime
    for name, cfg in bz.CONFIGS.items():
        arch = resolve_architecture(cfg)
        model = arch.build(arch.config_from_dict(cfg), Runtime("cpu", torch.float32))
        specs = {s.name: tuple(s.shape) for s in model.all_param_specs()}
        w = bz.make_weights(cfg, 1)
        assert specs == {k: tuple(v.shape) for k, v in w.items()}, name
        requests = model.cache_requests()
        assert all(isinstance(r, tuple) and len(r) == 2 for r in requests)


def test_the_measurement_configurations_are_valid():
    """What `bench.py --design ...` builds at its sizes parses as Bonolorn, Riruzen, Qwen3, Nelovik and Venitar configurations."""
    import sys

    from conftest import ROOT
    sys.path.insert(0, str(ROOT))
    import bench
    from lucciola_b200.config import resolve_architecture
    for size in bench.DESIGN_SIZES.values():
        cfgs = bench.design_configs(size, 4, 4096)
        assert set(cfgs) == {"bonolorn", "riruzen", "qwen3", "nelovik", "venitar"}
        for name, cfg in cfgs.items():
            arch = resolve_architecture(cfg)
            arch.config_from_dict(cfg)
            cost = bench.design_costs(name, cfg)
            assert cost["weight_bytes"] > 0 and cost["flops_per_token"] > 0 and cost["attn_flops"](64) > 0
