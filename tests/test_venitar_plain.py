"""The plain Venitar implementation against hand-made values and against itself (whole, portions, token by token), the
configuration reader, the order of layer runs, and the frequencies of the scaled rotation (CPU)."""
import json
import math

import pytest
import torch

import plain_venitar as plain
import venitar_util as vz

F = torch.float64


def test_retention_by_hand():
    """One head, one channel, no rotation: S follows d S + k v with k = x / sqrt(1) and the read-out is S q; the norm of a
    single entry leaves its sign, the gate is silu."""
    one = torch.ones(1, 1, dtype=F)
    w = {"q": one, "k": one * 2, "v": one * 3, "g": one, "o": one}
    m = {"heads": 1, "dim": 1, "vdim": 1, "decay": [0.5], "rot": {"dims": 0, "base": 10.0}}
    h = torch.tensor([[1.0], [2.0]], dtype=F)
    out, (n, S) = plain.retention(h, w, m, 0.0, None)
    s1 = 2.0 * 3.0                       # k v at token 0
    s2 = 0.5 * s1 + 4.0 * 6.0            # decayed, plus k v at token 1
    assert n == 2 and math.isclose(S.item(), s2)
    assert torch.allclose(out.flatten(), torch.tensor([plain.silu(torch.tensor(1.0, dtype=F)), plain.silu(torch.tensor(2.0, dtype=F))]))


def test_the_sink_and_the_chunks_by_hand():
    """A scale of zero: every visible key weighs 1 and the sink 1 more, so position i of a chunk of 3 returns the sum of
    the chunk's values so far over (count + 1).  The values are the keys' projection itself."""
    D = 2
    w = {"q": torch.eye(D, dtype=F), "k": torch.eye(D, dtype=F), "q.norm": torch.ones(D, dtype=F), "k.norm": torch.ones(D, dtype=F),
         "o": torch.eye(D, dtype=F)}
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": D, "scale": 0.0, "rot": {"dims": 2, "base": 100.0}, "mask": {"size": 3}}
    h = torch.arange(1, 11, dtype=F).reshape(5, 2)
    out, _ = plain.chunked_attention(h, w, m, 1e-6, None)
    for i in range(5):
        lo = (i // 3) * 3
        assert torch.allclose(out[i], h[lo:i + 1].sum(0) / (i - lo + 2))


def test_window_attention_by_hand():
    """A scale of zero and a window of 2: the mean of the last two values (with their bias), times the sigmoid gate."""
    D = 2
    z = torch.zeros(D, dtype=F)
    w = {"q": torch.eye(D, dtype=F), "k": torch.eye(D, dtype=F), "v": torch.eye(D, dtype=F), "q.b": z, "k.b": z, "v.b": z + 1.0,
         "g": torch.zeros(D, D, dtype=F), "o": torch.eye(D, dtype=F)}
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": D, "scale": 0.0, "rot": {"dims": 0, "base": 100.0}, "mask": {"size": 2}}
    h = torch.arange(1, 9, dtype=F).reshape(4, 2)
    out, _ = plain.window_attention(h, w, m, None)
    for i in range(4):
        assert torch.allclose(out[i], 0.5 * ((h[max(0, i - 1):i + 1] + 1.0).mean(0)))


def test_channel_decays_by_hand():
    """One head, two key channels with decays of their own: with beta = 1/2 and unit q, k the state's rows follow
    S_r <- g_r S_r; u = (v - sum_r S_r k_r) / 2; S_r += k_r u."""
    one = torch.ones(1, 1, dtype=F)
    w = {"q": torch.ones(2, 1, dtype=F), "k": torch.ones(2, 1, dtype=F), "v": one, "q.conv": torch.ones(2, 1, dtype=F),
         "k.conv": torch.ones(2, 1, dtype=F), "v.conv": one, "b": torch.zeros(1, 1, dtype=F), "a1": one * 0.0, "a2": torch.zeros(2, 1, dtype=F),
         "A_log": torch.zeros(1, dtype=F), "dt_bias": torch.tensor([0.0, 3.0], dtype=F), "g1": one * 0.0, "g2": torch.zeros(1, 1, dtype=F),
         "norm": torch.ones(1, dtype=F), "o": one}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "conv": 1}
    big = 40.0                                           # silu(40) = 40; (40, 40) / |(40, 40)| = (1, 1) / sqrt 2
    h = torch.full((3, 1), big, dtype=F)
    _, (_, _, _, S) = plain.channel_delta_rule(h, w, m, 0.0, None)
    g = [math.exp(-math.log1p(math.exp(0.0))), math.exp(-math.log1p(math.exp(3.0)))]
    k = 1 / math.sqrt(2.0 + 1e-6 / 1600.0)
    s = [0.0, 0.0]
    for _ in range(3):
        s = [g[0] * s[0], g[1] * s[1]]
        u = 0.5 * (big - (s[0] + s[1]) * k)
        s = [s[0] + k * u, s[1] + k * u]
    assert torch.allclose(S.flatten(), torch.tensor(s, dtype=F), rtol=1e-9)


def test_scaled_rotation_by_hand():
    """Pairs that make more than `fast` turns in the original context keep their frequency, those below `slow` are
    divided by the factor, and both sines and cosines grow by 0.1 ln(factor) + 1."""
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, mag = plain.rotary_frequencies(rot)
    base = 100.0 ** (-2.0 * torch.arange(4, dtype=F) / 8)
    turns = 64 * base / (2 * math.pi)
    assert math.isclose(mag, 0.1 * math.log(4.0) + 1.0)
    assert torch.all(f[turns > 8.0 * 1.5] == base[turns > 8.0 * 1.5]) and torch.all(f <= base) and torch.all(f >= base / 4.0 - 1e-15)
    assert math.isclose(f[-1].item(), base[-1].item() / 4.0)              # the slowest pair turns less than once
    x = torch.randn(3, 2, 10, dtype=F)
    y = plain.rotate_half(x, torch.tensor([0, 5, 9]), rot)
    assert torch.allclose(y[..., 8:], x[..., 8:]) and torch.allclose(y[0, :, :8], x[0, :, :8] * mag)
    # the package's table is the same numbers, rounded to 32-bit
    from lucciola_b200.parts.rope import yarn_frequencies
    got, got_mag = yarn_frequencies(8, 100.0, 4.0, 64, 8.0, 1.0)
    assert got_mag == mag and torch.equal(got, f.to(torch.float32))


def test_the_order_of_layer_runs():
    cfg = {"layers": [0, 1, 2, 3], "loop": {"start": 1, "stop": 3, "times": 3}}
    assert plain.layer_runs(cfg) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert plain.layer_runs({"layers": [0, 1], "loop": {"start": 2, "stop": 2, "times": 4}}) == [(0, False), (1, False)]
    assert plain.layer_runs({"layers": [0, 1], "loop": {"start": 0, "stop": 2, "times": 1}}) == [(0, False), (1, False)]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_and_single_tokens_equal_the_whole(name):
    """The plain model with its explicit past: a sequence in portions, down to single tokens, gives the logits of the
    sequence run whole."""
    cfg = vz.CONFIGS[name]
    w = vz.make_weights(cfg, 11)
    ids = vz.tokens(cfg, 50, salt=3)
    model = plain.PlainVenitar(cfg, w)
    whole = model.forward(ids)
    past, got, at = None, [], 0
    for n in (1, 7, 2, 1, 1, 19, 3, 16):
        logits, past = model.run(ids[at:at + n], past)
        got.append(logits)
        at += n
    assert at == 50
    assert (torch.cat(got) - whole).abs().max() <= 1e-9 * whole.abs().max()


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_configuration_reader_and_tensor_list(name):
    """config.json -> typed configuration -> config.json again; the model the registry composes asks for exactly the
    tensors a checkpoint of this design has, in their shapes; ranks come from the tensors where config.json is silent."""
    from lucciola_b200.config.registry import resolve_architecture
    from lucciola_b200.parts.base import Runtime
    cfg = vz.CONFIGS[name]
    arch = resolve_architecture(cfg)
    typed = arch.config_from_dict(cfg)
    assert typed.to_dict() == json.loads(json.dumps(cfg))
    w = vz.make_weights(cfg, 5)
    model = arch.build(typed, Runtime("cpu", torch.float32))
    specs = {s.name: tuple(s.shape) for s in model.all_param_specs()}
    assert specs == {k: tuple(v.shape) for k, v in w.items()}
    runs = plain.layer_runs(cfg)
    assert [(c.block, c.add_embedding) for c in model.calls] == runs and [c.cache for c in model.calls] == list(range(len(runs)))
    silent = json.loads(json.dumps(cfg))
    for layer in silent["layers"]:
        if layer["type"] == "parallel":
            del layer["mixer"]["right"]["decay_rank"], layer["mixer"]["right"]["gate_rank"]
    bare = arch.config_from_dict(silent)
    from lucciola_b200.config.model_config import ConfigError
    if any(l["type"] == "parallel" for l in cfg["layers"]):
        with pytest.raises(ConfigError):
            arch.build(bare, Runtime("cpu", torch.float32))
    assert bare.with_tensor_shapes(lambda n: tuple(w[n].shape) if n in w else None) == typed


def test_configurations_that_are_refused():
    from lucciola_b200.config.model_config import ConfigError
    from lucciola_b200.config.venitar_config import VenitarConfig
    good = vz.CONFIGS["A"]
    def broken(change):
        d = json.loads(json.dumps(good))
        change(d)
        with pytest.raises(ConfigError):
            VenitarConfig.from_dict(d)
    broken(lambda d: d["layers"][0].update(type="hyena"))
    broken(lambda d: d["layers"][0]["mlp"].update(kind="experts"))
    broken(lambda d: d["loop"].update(stop=9))
    broken(lambda d: d["layers"][1]["mixer"].update(decay=[0.5]))
    broken(lambda d: d["layers"][2]["mixer"].update(vdim=7))
    broken(lambda d: d["layers"][2]["mixer"]["rot"].update(dims=5))
    broken(lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3))
    broken(lambda d: d.pop("norm"))


@pytest.mark.parametrize("seed", range(6))
def test_configurations_drawn_at_random_build(seed):
    from lucciola_b200.config.registry import resolve_architecture
    from lucciola_b200.parts.base import Runtime
    cfg = vz.random_config(seed)
    arch = resolve_architecture(cfg)
    model = arch.build(arch.config_from_dict(cfg), Runtime("cpu", torch.float32))
    w = vz.make_weights(cfg, seed)
    assert {s.name: tuple(s.shape) for s in model.all_param_specs()} == {k: tuple(v.shape) for k, v in w.items()}
    ids = vz.tokens(cfg, 12, salt=seed)
    assert torch.isfinite(plain.PlainVenitar(cfg, w).forward(ids)).all()
