"""Venitar in the engine against the plain implementation: every mechanism alone, then the whole model under every
way of cutting the work, with pages and state slots that are freed and used again, and generation through the entry
point (GPU)."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_venitar as plain
import replay_util as ru
import venitar_util as vz

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"
F = torch.float64


def stream():
    return torch.cuda.current_stream().cuda_stream


def batch_of(q_lens, slots, starts=None):
    """What the kernels read of a step: token -> sequence map, first token of each sequence, slots, positions."""
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    seq = [i for i, n in enumerate(q_lens) for _ in range(n)]
    starts = starts or [0] * len(q_lens)
    pos = [s + j for s, n in zip(starts, q_lens) for j in range(n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(num_tokens=cu[-1], num_seqs=len(q_lens), token_seq=i32(seq), cu_tokens=i32(cu), state_slots=i32(slots),
                           positions=i32(pos), context_lens=i32([s + n for s, n in zip(starts, q_lens)]), q_lens=list(q_lens),
                           start_positions=list(starts), max_q_len=max(q_lens),
                           max_context_len=max(s + n for s, n in zip(starts, q_lens)), span_hint=0, plans={}, block_tables=[])


def runtime(dtype=torch.float32):
    from lucciola_b200.parts.base import Runtime
    rt = Runtime(DEV, dtype)
    rt.stream = stream()
    return rt


def in_portions(forward, xs, slots, schedule):
    """Run sequences through `forward(rows, step)` in unequal portions that share steps; returns each sequence's rows."""
    got, at = [[] for _ in xs], [0] * len(xs)
    for sizes in schedule:
        live = [i for i in range(len(xs)) if at[i] < xs[i].shape[0] and sizes[i]]
        if not live:
            continue
        lens = [min(sizes[i], xs[i].shape[0] - at[i]) for i in live]
        rows = torch.cat([xs[i][at[i]:at[i] + n] for i, n in zip(live, lens)])
        out = forward(rows.contiguous(), batch_of(lens, [slots[i] for i in live], [at[i] for i in live]))
        o = 0
        for i, n in zip(live, lens):
            got[i].append(out[o:o + n].double().cpu())
            o += n
            at[i] += n
    assert all(a == x.shape[0] for a, x in zip(at, xs))
    return [torch.cat(g) for g in got]


SCHEDULE = ([1, 2], [1, 1], [17, 1], [3, 1], [16, 1], [2, 0], [1, 0], [40, 0])      # [1, 1], [1, 0]: steps of single tokens


def _bind(part, w):
    part.bind_all(lambda name: w[name].to(DEV))


# ---- each mechanism alone --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("heads,dim,dims,yarn", [(3, 20, 8, None), (1, 16, 16, (4.0, 64, 8.0, 1.0)), (4, 64, 0, None), (2, 130, 64, (1.0, 16, 4.0, 2.0))])
def test_rotation_in_place_of_32_bit_rows(heads, dim, dims, yarn):
    from lucciola_b200 import ops
    from lucciola_b200.parts.rope import RotaryEmbedding
    T, n = 9, heads * dim
    rot = vz._rot(dims, 1000.0, yarn)
    enc = RotaryEmbedding(runtime(), dim, 1000.0, dims, yarn=yarn) if dims else None
    x = torch.randn(T, 3 + 2 * n + 5, device=DEV)
    before = x.double().cpu()
    pos = torch.tensor([0, 1, 2, 700, 5, 31, 64, 1023, 40000], dtype=torch.int32, device=DEV)
    table = enc.rotary_table() if enc is not None else (None, 0)
    ops.rotate_rows(x[:, 3:], pos, table[0], dim, table[1], [(0, heads, 1.0), (n, heads, dim ** -0.5)], stream(),
                    rot_scale=enc.magnitude if enc is not None else 1.0)
    got = x.double().cpu()
    q = plain.rotate_half(before[:, 3:3 + n].reshape(T, heads, dim), pos.cpu(), rot).reshape(T, n)
    k = plain.rotate_half(before[:, 3 + n:3 + 2 * n].reshape(T, heads, dim), pos.cpu(), rot).reshape(T, n) * dim ** -0.5
    # the angle is a 32-bit product: at position p it is off by up to p * 2^-24 of a turn's radian
    assert (got[:, 3:3 + n] - q).abs().max() <= 5e-3 and (got[:6, 3:3 + n] - q[:6]).abs().max() <= 2e-4
    assert (got[:6, 3 + n:3 + 2 * n] - k[:6]).abs().max() <= 2e-4
    assert torch.equal(got[:, :3], before[:, :3]) and torch.equal(got[:, 3 + 2 * n:], before[:, 3 + 2 * n:])


@pytest.mark.parametrize("heads,dim,vdim,dims", [(3, 20, 12, 8), (1, 16, 24, 0), (4, 64, 64, 64), (2, 256, 40, 128), (2, 33, 70, 2), (5, 128, 128, 64)])
def test_retention_alone(heads, dim, vdim, dims):
    """Two sequences in unequal portions (single tokens, a few, many) through the part in 32-bit, against the plain
    recurrence; a state row that belongs to another request stays as it is."""
    from lucciola_b200.parts.base import StateCacheView
    from lucciola_b200.parts.decay_attention import DecayLinearAttention
    from lucciola_b200.parts.rope import RotaryEmbedding
    width = 48
    decay = [0.5, 0.9, 0.99, 0.999, 0.9999][:heads]
    layer = vz._retention(heads, dim, vdim, decay, vz._rot(dims, 10000.0), None)
    cfg = vz._config(10, width, 1e-5, 1.0, (0, 0, 1), [layer])
    w = {k[len("l0."):]: v.float() for k, v in vz.make_weights(cfg, heads * 100 + dim).items() if k.startswith("l0.mix.")}
    rt = runtime()
    part = DecayLinearAttention(rt, "mix", width, heads, dim, vdim, decay, 1e-5, act=None,
                                position_encoding=RotaryEmbedding(rt, dim, 10000.0, dims) if dims else None, k_scale=dim ** -0.5,
                                head_norm=True, norm_weight=False, gate_act="silu", out_dtype=torch.float32)
    _bind(part, w)
    cache = StateCacheView(torch.zeros(5, *part.cache_request().shape, device=DEV))
    cache.state[2] = float("nan")
    xs = [torch.randn(n, width, device=DEV) for n in (79, 5)]
    got = in_portions(lambda rows, step: part.forward(rows, step, cache), xs, [1, 3], SCHEDULE)
    sub = {k[len("mix."):]: v.double() for k, v in w.items()}
    for x, g in zip(xs, got):
        want, _ = plain.retention(x.double().cpu(), sub, layer["mixer"], 1e-5, None)
        assert (g - want).abs().max() <= 2e-5 * want.abs().max(), (g - want).abs().max() / want.abs().max()
    assert torch.isnan(cache.state[2]).all() and torch.isfinite(cache.state[[1, 3]]).all()


@pytest.mark.parametrize("heads,dim,vdim,split", [(2, 64, 64, 1), (3, 128, 40, 2), (1, 20, 33, 1), (2, 256, 64, 4)])
def test_decay_recurrence_without_activation_side_by_side_form(heads, dim, vdim, split):
    """The kernel that forms the outputs of 16 tokens side by side (long steps of the bfloat16 engine), on q, k, v as they
    come: its planes' sum through the head-wise gated norm against the token-by-token recurrence."""
    from lucciola_b200 import ops
    n = heads * dim
    lens = [70, 3, 33]
    T = sum(lens)
    pre = torch.randn(T, 2 * n + 2 * heads * vdim + 2, device=DEV)[:, 2:] * 0.5
    decay = torch.tensor([0.9, 0.99, 0.999][:heads], device=DEV)
    state = torch.randn(4, heads, dim, vdim, device=DEV)
    s0 = state.double().cpu()
    step = batch_of(lens, [2, 0, 1])
    o = torch.empty(split, T, heads * vdim, device=DEV)
    ops.decay_recurrence(pre, 0, n, 2 * n, decay, state, o, step, heads, dim, vdim, stream(), max_tokens_a_seq=70, row_split=split, act=False)
    out = torch.empty(T, heads * vdim, device=DEV)
    gate = pre[:, 2 * n + heads * vdim:]
    ops.gated_group_norm(out, o, gate, None, heads, 1e-5, stream(), act="silu", scale=0.5)
    p = pre.double().cpu()
    t0 = 0
    for length, slot in zip(lens, (2, 0, 1)):
        S = s0[slot].clone()
        for t in range(t0, t0 + length):
            q, k, v = p[t, :n].reshape(heads, dim), p[t, n:2 * n].reshape(heads, dim), p[t, 2 * n:2 * n + heads * vdim].reshape(heads, vdim)
            S = decay.double().cpu()[:, None, None] * S + k[:, :, None] * v[:, None, :]
            want = 0.5 * plain.rms_norm(torch.einsum("hdv,hd->hv", S, q), None, 1e-5).reshape(-1) * plain.silu(p[t, 2 * n + heads * vdim:])
            assert (out[t].double().cpu() - want).abs().max() <= 3e-5 * max(want.abs().max().item(), 1.0), t
        assert (state[slot].double().cpu() - S).abs().max() <= 2e-5 * S.abs().max()
        t0 += length
    assert torch.equal(state[3].double().cpu(), s0[3])


@pytest.mark.parametrize("heads,kv,dim,vdim,taps,ra,rg", [(3, 1, 20, 12, 3, 5, 7), (1, 1, 40, 40, 1, 1, 1), (4, 2, 128, 64, 4, 16, 8), (2, 2, 33, 70, 2, 3, 2),
                                                          (2, 1, 200, 48, 4, 8, 24), (6, 3, 8, 8, 5, 24, 24), (1, 1, 256, 33, 2, 4, 4), (5, 5, 32, 48, 3, 8, 16)])
def test_delta_rule_with_channel_decays_alone(heads, kv, dim, vdim, taps, ra, rg):
    from lucciola_b200.parts.base import StateCacheView
    from lucciola_b200.parts.delta_rule import GatedDeltaRule
    width = 48
    right = vz._right(heads, kv, dim, vdim, taps, ra, rg)
    cfg = vz._config(10, width, 1e-5, 1.0, (0, 0, 1), [vz._pair(vz._left(1, 1, 8, 8, 0.3, vz._rot(0, 10.0), 4), right, 1.0, 1.0, None)])
    w = {k[len("l0.mix."):]: v.float() for k, v in vz.make_weights(cfg, heads * 100 + dim).items() if k.startswith("l0.mix.right.")}
    part = GatedDeltaRule(runtime(), "right", width, heads, kv, dim, vdim, taps, 1e-5, decay_rank=ra, gate_rank=rg, gate_act="sigmoid")
    _bind(part, w)
    caches = tuple(StateCacheView(torch.zeros(5, *r.shape, device=DEV)) for r in part.cache_request())
    caches[-1].state[2] = float("nan")
    xs = [torch.randn(n, width, device=DEV) for n in (79, 5)]
    got = in_portions(lambda rows, step: part.forward(rows, step, caches), xs, [1, 3], SCHEDULE)
    sub = {k[len("right."):]: v.double() for k, v in w.items()}
    for x, g in zip(xs, got):
        want, _ = plain.channel_delta_rule(x.double().cpu(), sub, right, 1e-5, None)
        assert (g - want).abs().max() <= 2e-5 * want.abs().max(), (g - want).abs().max() / want.abs().max()
    assert torch.isnan(caches[-1].state[2]).all() and torch.isfinite(caches[-1].state[[1, 3]]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels(dtype):
    """relu squared; the rounded copy of a column range; the scaled embedding and its second copy; the gated norm without a
    weight over planes."""
    from lucciola_b200 import ops
    x = (torch.randn(9, 130, device=DEV) * 3).to(dtype)
    out = torch.empty_like(x)
    ops.activation(out, x, "relu2", stream())
    want = torch.relu(x.double()).pow(2)
    assert (out.double() - want).abs().max() <= (3e-6 if dtype == torch.float32 else 1e-2) * want.abs().max()
    wide = torch.randn(7, 50, device=DEV)
    r = torch.empty(7, 11, dtype=dtype, device=DEV)
    ops.round_cols(r, wide[:, 30:41], stream())
    assert torch.equal(r, wide[:, 30:41].to(dtype))
    table = torch.randn(20, 36, device=DEV).to(dtype)
    ids = torch.tensor([3, 19, 0, 3], dtype=torch.int32, device=DEV)
    a, b = torch.empty(4, 36, device=DEV), torch.full((4, 36), float("nan"), device=DEV)
    ops.embedding(a, ids, table, stream(), scale=0.37, copy=b)
    assert torch.equal(a, b) and torch.equal(a, table[ids.long()].float() * 0.37)
    y, gate = torch.randn(3, 6, 40, device=DEV), torch.randn(6, 42, device=DEV)[:, 2:]
    o = torch.empty(6, 40, dtype=dtype, device=DEV)
    ops.gated_group_norm(o, y, gate, None, 5, 1e-5, stream(), act="sigmoid", scale=2.0)
    want = 2.0 * plain.rms_norm(y.double().sum(0).reshape(6, 5, 8), None, 1e-5).reshape(6, 40) * torch.sigmoid(gate.double())
    assert (o.double() - want).abs().max() <= (3e-6 if dtype == torch.float32 else 1e-2) * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,page,size", [(3, 1, 20, 8, 24), (4, 2, 64, 16, 40), (8, 2, 128, 16, 33), (1, 1, 16, 8, 1), (2, 1, 24, 16, 6),
                                                    (8, 8, 96, 32, 70), (16, 1, 32, 8, 12), (4, 4, 128, 16, 64)])
@pytest.mark.parametrize("mask", ["chunk", "window"])
def test_a_query_finds_its_one_key_at_every_edge(dtype, heads, kv, dim, page, size, mask):
    """Keys and values of a long sequence in pages that lie in a scrambled order; what the mask can no longer reach is
    overwritten with NaN.  One key far above all others stands in turn at the first place the last query sees, at the
    place before it, at the last query's own place, far back, and at a page's first and last slot; the query is the last
    token alone (a decoded token) or the last of a portion that crosses the edge.  Chunks come with the sink of score 0,
    the window without.  The kernels must agree with a plain softmax over exactly the visible keys."""
    from lucciola_b200 import ops
    n = 5 * size + 2 * page + 7
    g = torch.Generator(device=DEV).manual_seed(n + heads)
    last = n - 1
    first_seen = (last // size) * size if mask == "chunk" else max(0, last - size + 1)
    spots = {first_seen, max(0, first_seen - 1), last, 0, (first_seen // page) * page, min(last, (first_seen // page) * page + page - 1), max(0, last - 1)}
    sinks = torch.zeros(heads, device=DEV) if mask == "chunk" else None
    scale = 0.3
    pages = -(-n // page)
    table = torch.arange(pages, dtype=torch.int32, device=DEV).flip(0).reshape(1, pages).contiguous()
    kw = dict(sinks=sinks, chunk=size) if mask == "chunk" else {}
    window = 0 if mask == "chunk" else size
    for spot in sorted(spots):
        K = torch.randn(n, kv, dim, device=DEV, generator=g)
        V = torch.randn(n, kv, dim, device=DEV, generator=g)
        q = torch.randn(3, heads, dim, device=DEV, generator=g)
        K[spot] = 4.0 * q[-1].reshape(kv, heads // kv, dim)[:, 0] / scale / dim ** 0.5
        kc = torch.zeros(pages, kv, page, dim, dtype=dtype, device=DEV)
        vc = torch.zeros(pages, kv, page, dim, dtype=dtype, device=DEV)
        pos = torch.arange(n, device=DEV)
        kc[table[0, pos // page].long(), :, pos % page] = K.to(dtype)
        vc[table[0, pos // page].long(), :, pos % page] = V.to(dtype)
        longest = min(37, n - 1)
        lo_of = (lambda i: (i // size) * size) if mask == "chunk" else (lambda i: max(0, i - size + 1))
        keep_from = lo_of(n - longest)
        gone = torch.arange(0, keep_from, device=DEV)
        gone = gone[(gone // page) < (keep_from // page)]                                                 # whole pages only
        if gone.numel():
            kc[table[0, gone // page].long(), :, gone % page] = float("nan")
            vc[table[0, gone // page].long(), :, gone % page] = float("nan")
        Kc, Vc = K.to(dtype).double(), V.to(dtype).double()
        q = torch.cat([torch.randn(longest - 3, heads, dim, device=DEV, generator=g), q])
        fast = dtype == torch.bfloat16 and ops.attention_flash_ok(q.to(dtype), heads, kv, dim)
        for qs, starts in (([1], [last]), ([3], [n - 3]), ([longest], [n - longest]), ([1, longest], [last, n - longest]), ([2, 1, 5], [n - 2, last, n - 5])):
            step = batch_of(qs, [0] * len(qs), starts)
            tb = table.repeat(len(qs), 1).contiguous()
            qq = torch.cat([q[longest - (n - st): longest - (n - st) + c] for c, st in zip(qs, starts)]).to(dtype).contiguous()
            outs = []
            out = torch.empty(sum(qs), heads, dim, dtype=dtype, device=DEV)
            ops.attention_plain(qq, out, kc, vc, step.positions, step.token_seq, tb, heads, kv, dim, page, window, scale, stream(), **kw)
            outs.append(("plain", out))
            if fast:
                from lucciola_b200.parts.attention import plan_tiles
                from lucciola_b200.parts.base import BatchShape, PlanView
                made = plan_tiles(BatchShape(list(qs), list(starts), max(qs), n, n), heads // kv)
                view = PlanView({k: torch.from_numpy(a).to(DEV) for k, a in made.arrays.items()}, made.host)
                step.block_tables = [tb]
                out = torch.full((sum(qs), heads, dim), float("nan"), dtype=dtype, device=DEV)
                ops.attention(qq, out, kc, vc, step, 0, heads, kv, dim, page, window, scale, stream(), plan=view, **kw)
                outs.append(("tensor cores", out))
                if mask == "chunk":
                    rows = min(made.host["rows"]["all"], 64)
                    for splits, ws in ((2, False), (3, True)):
                        out = torch.full((sum(qs), heads, dim), float("nan"), dtype=dtype, device=DEV)
                        ops.attention_flash(qq, out, kc, vc, step.positions, tb, view.arrays["all"], rows, heads, kv, dim, page, window, scale,
                                            splits, stream(), force_workspace=ws, **kw)
                        outs.append((f"tensor cores, {splits} key ranges", out))
            r = 0
            for c, st in zip(qs, starts):
                for i in range(st, st + c):
                    lo = lo_of(i)
                    for h in range(heads):
                        gk = h // (heads // kv)
                        sc = Kc[lo:i + 1, gk] @ qq[r, h].double() * scale
                        mx = sc.max().clamp(min=0.0) if mask == "chunk" else sc.max()
                        e = torch.exp(sc - mx)
                        want = (e[:, None] * Vc[lo:i + 1, gk]).sum(0) / (e.sum() + (torch.exp(-mx) if mask == "chunk" else 0.0))
                        for which, out in outs:
                            err = (out[r, h].double() - want).abs().max().item()
                            assert err <= (1e-5 if dtype == torch.float32 else 3e-2) * max(want.abs().max().item(), 0.3), (which, spot, qs, i, h, err)
                    r += 1


# ---- the whole model -------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, weights, folder).  Beside A and C: "Asharp" / "Csharp", whose attentions pick out single keys."""
    out = {}
    for name, cfg in vz.CONFIGS.items():
        w = vz.make_weights(cfg, 100 + len(out))
        out[name] = (cfg, w, vz.write_model(tmp_path_factory.mktemp(f"venitar_{name}"), cfg, w, name_ranks=name != "A"))
    for base in ("A", "C"):
        cfg = vz.CONFIGS[base]
        w = vz.make_weights(cfg, 200 + len(out), sharp=4.0)
        out[base + "sharp"] = (cfg, w, vz.write_model(tmp_path_factory.mktemp(f"venitar_{base}sharp"), cfg, w))
    return out


def make_runner(models, name, dtype, num_pages, graphs=False, slots=4, **kw):
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    page = vz.PAGE[name[0]]
    return build_runner(models[name][2], EngineOptions(dtype=dtype, block_size=page, max_blocks=num_pages, max_num_seqs=slots,
                                                       use_cuda_graph=graphs, graph_after=1, max_shape_graphs=1000, **kw),
                        num_pages=num_pages)


TOL_SHARP = {"float32": 1e-4, "bfloat16": 0.12}


def check(models, name, dtype, steps, reqs, graphs=False, poison=True, tol=None, slots=4):
    page = vz.PAGE[name[0]]
    cfg, w, _ = models[name]
    if tol is None:
        tol = vz.bound(dtype, cfg, w, reqs, TOL_SHARP[dtype] if "sharp" in name else None)
    runner = make_runner(models, name, dtype, max(ru.max_live_tokens(steps) // page, 1), graphs=graphs, slots=slots)
    got = ru.replay(runner, steps, poison=poison)
    worst = vz.compare(got, name, cfg, w, reqs, dtype, tol)
    assert runner.manager.num_requests() == 0 and all(p.num_free == p.num_pages for p in runner.manager.pools)
    return runner, got, worst


LENGTHS = {"A": [1, 2, 15, 16, 17, 47, 130], "B": [1, 7, 8, 9, 64, 120], "C": [3, 31, 32, 33, 129, 300], "D": [1, 16, 65, 140, 400]}


def requests_for(models, name):
    cfg = models[name][0]
    return {f"{name}{n}": vz.tokens(cfg, n, salt=len(name)) for n in LENGTHS[name[0]]}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "Asharp", "Csharp"])
@pytest.mark.parametrize("cut", ["whole", "tail_decoded", "portions"])
def test_each_request_alone(models, name, dtype, cut):
    """Whole prompts (lengths at and beside page borders, windows and chunks), prompt then token-by-token decoding, and
    portions of 1 to 31 tokens, each request by itself."""
    reqs = requests_for(models, name)
    check(models, name, dtype, getattr(ru, cut)(reqs), reqs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "Csharp"])
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_batches_with_reused_pages_and_slots(models, name, dtype, seed):
    """Up to four live requests of unequal length, portions beside single tokens; nine requests through four state
    slots and fewer pages than they need together; what a freed page or slot held is overwritten with NaN."""
    cfg = models[name][0]
    reqs = {f"m{i}": vz.tokens(cfg, n, salt=seed + 3) for i, n in enumerate((70, 9, 120, 33, 101, 2, 64, 47, 90))}
    steps = ru.mixed(reqs, seed=seed)
    assert ru.max_live_tokens(steps) < sum(ru.ceil64(len(v)) for v in reqs.values())
    check(models, name, dtype, steps, reqs, slots=4)
    assert max(len(s["entries"]) for s in steps) >= 3


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("cut", ["tail_decoded", "portions", "mixed_decodes_first"])
def test_every_cutting_through_recorded_graphs(models, name, cut):
    """bfloat16 with recordings on: the trace runs twice through one runner; the second pass replays the CUDA graphs
    the first recorded, with other pages and slots under the same requests."""
    cfg, w, _ = models[name]
    if cut.startswith("mixed"):
        reqs = {f"m{i}": vz.tokens(cfg, n, salt=5) for i, n in enumerate((70, 9, 120, 33, 101, 2, 64, 47, 90))}
        steps = ru.mixed(reqs, seed=4, decodes_first=True)
    else:
        reqs = requests_for(models, name)
        steps = getattr(ru, cut)(reqs)
    page = vz.PAGE[name[0]]
    runner = make_runner(models, name, "bfloat16", max(ru.max_live_tokens(steps) // page, 1), graphs=True)
    assert runner._can_record
    tol = vz.bound("bfloat16", cfg, w, reqs)
    first = ru.replay(runner, steps, poison=True)
    vz.compare(first, name, cfg, w, reqs, "bfloat16", tol)
    recorded, replays = len(runner._graphs), runner.graph_replays
    assert recorded > 0
    second = ru.replay(runner, steps, poison=True)
    vz.compare(second, name, cfg, w, reqs, "bfloat16", tol)
    assert len(runner._graphs) == recorded and runner.graph_replays - replays == sum(1 for s in steps if s["entries"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_cutting_does_not_change_float32_results_at_all(models, name, dtype):
    """In 32-bit every sum's order is fixed by the model's sizes alone, so whole prompts, portions, single tokens and
    mixed batches agree to the last bit; in bfloat16 within rounding."""
    reqs = requests_for(models, name)
    runs = []
    for steps in (ru.whole(reqs), ru.portions(reqs), ru.mixed(reqs, seed=3), ru.tail_decoded(reqs, tail=40)):
        runner = make_runner(models, name, dtype, 200)
        runs.append(ru.replay(runner, steps))
    common = set(runs[0]) & set(runs[1]) & set(runs[2])
    assert len(common) > 50
    for key in common:
        for other in runs[1:]:
            if key not in other:
                continue
            if dtype == "float32":
                assert torch.equal(runs[0][key], other[key]), key
            else:
                assert (runs[0][key] - other[key]).abs().max() <= 2 * vz.TOL[dtype] * runs[0][key].abs().max(), key


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Asharp", "Csharp", "D"])
def test_long_decoding_past_windows_and_chunks_with_old_state(models, name, dtype):
    """A short prompt, then hundreds of tokens decoded one by one: every window and chunk passes over decoded tokens
    (pages are given back as it does), and the slow decays still carry what entered the states at the start."""
    cfg = models[name][0]
    ids = vz.tokens(cfg, 390, salt=9)
    steps = ru.tail_decoded({"long": ids}, tail=387)
    _, got, _ = check(models, name, dtype, steps, {"long": ids})
    assert len(got) == 388


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Asharp", "Csharp"])
def test_the_edges_of_windows_and_chunks_really_matter(models, name, dtype):
    """The sharpened model must be one in which single keys matter: replacing the token that stands just inside the
    window of the last query, or the first token of its chunk, changes the last logits by far more than the 32-bit
    tolerance.  Then the engine, the prompt in portions that end at, before and behind the borders of pages, windows
    and chunks, against the plain implementation."""
    cfg, w, _ = models[name]
    window = next(l for l in cfg["layers"] if l["type"] == "parallel")["mixer"]["left"]["mask"]["size"]
    chunk = next(l for l in cfg["layers"] if l["type"] == "attention")["mixer"]["mask"]["size"]
    ids = vz.tokens(cfg, 200, salt=21)
    a = vz.plain_logits(name, cfg, w, ids)
    for spot in (199 - (window - 1), (199 // chunk) * chunk):
        other = list(ids)
        other[spot] = (ids[spot] + 1) % cfg["vocab"]
        b = vz.plain_logits(name, cfg, w, other)
        assert (a[-1] - b[-1]).abs().max() > 20 * TOL_SHARP["float32"] * a.abs().max()
    page = vz.PAGE[name[0]]
    steps = ru.portions({"edge": ids}, sizes=(page - 1, 2, page, page + 1, chunk, chunk - 1 or 1, 2, window + 1, 2 * page - 2, 3, 5 * page, 1, 1, 2))
    check(models, name, dtype, steps, {"edge": ids})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(models, name, dtype):
    """Positions 0 to 5: a single key, fewer tokens than a window or chunk holds, a page with one token, empty states,
    convolutions that reach before the start."""
    cfg = models[name][0]
    for n in (1, 2, 3, 6):
        ids = vz.tokens(cfg, n, salt=n)
        for steps in (ru.whole({"f": ids}), ru.tail_decoded({"f": ids}, tail=n - 1) if n > 1 else ru.whole({"f": ids})):
            check(models, name, dtype, steps, {"f": ids})


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_against_each_alone(models, dtype):
    """Five unequal prompts in one step, then their next tokens in one step: every row equals the request run alone."""
    name = "C"
    cfg = models[name][0]
    reqs = {f"b{n}": vz.tokens(cfg, n, salt=31) for n in (2, 40, 17, 128, 65)}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids[:-1], "want": [len(ids) - 2]} for r, ids in reqs.items()], "end": []},
             {"step": 1, "entries": [{"id": r, "tokens": ids[-1:], "want": [0]} for r, ids in reqs.items()], "end": list(reqs)}]
    _, together, _ = check(models, name, dtype, steps, reqs, slots=8)
    for r, ids in reqs.items():
        _, alone, _ = check(models, name, dtype, ru.whole({r: ids}), {r: ids})
        for p in (len(ids) - 2, len(ids) - 1):
            if dtype == "float32":
                assert torch.equal(together[(r, p)], alone[(r, p)]), (r, p)


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Every size drawn at random: the 32-bit engine must agree with the plain implementation to 32-bit rounding under
    every cutting; the bfloat16 engine within its bound."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    cfg = vz.random_config(seed)
    reqs = {f"q{i}": vz.tokens(cfg, n, salt=seed) for i, n in enumerate((1, 23, 97, 200, 64))}
    w = vz.make_weights(cfg, 300 + seed)
    folder = vz.write_model(tmp_path / "model", cfg, w, name_ranks=seed % 2 == 0)
    for dtype in DTYPES:
        for cut in ("whole", "portions", "mixed", "tail_decoded"):
            steps = getattr(ru, cut)(reqs)
            pages = max(ru.max_live_tokens(steps) // 16, 1)
            runner = build_runner(folder, EngineOptions(dtype=dtype, block_size=16, max_blocks=pages, max_num_seqs=4,
                                                        use_cuda_graph=(cut == "mixed"), graph_after=1), num_pages=pages)
            got = ru.replay(runner, steps, poison=True)
            vz.compare(got, ("drawn", seed), cfg, w, reqs, dtype, tol=5e-5 if dtype == "float32" else vz.bound(dtype, cfg, w, reqs, 5e-2))


# ---- through the entry point -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 0.3)])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(models, name, dtype, slack):
    """Engine.generate with the scheduler's own batching: prompts longer than a step's budget (so they are read in
    portions beside decoding requests), more requests than state slots.  Every generated token must be the plain
    implementation's choice for the same prefix, or lose to it by a near-tie."""
    from lucciola_b200 import Engine, EngineOptions, SamplingParams
    cfg, w, folder = models[name]
    eng = Engine(folder, options=EngineOptions(dtype=dtype, block_size=vz.PAGE[name[0]], max_blocks=64, max_tokens_per_step=48, max_num_seqs=3))
    prompts = [vz.tokens(cfg, n, salt=41) for n in (5, 70, 33, 1, 100)]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert all(len(o) == 6 for o in outs)
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for k, tok in enumerate(out):
            row = vz.plain_logits(name, cfg, w, ids)[-1]
            assert row.max() - row[tok] <= slack * row.abs().max().clamp(min=1.0), f"token {k}: chose {tok}, plain chooses {int(row.argmax())}"
            ids.append(tok)
    assert eng.runner.manager.num_requests() == 0 and all(p.num_free == p.num_pages for p in eng.runner.manager.pools)


def test_generation_under_page_pressure_recomputes_the_state(models):
    """Fewer pages than the requests need together: a request is preempted, gives its pages and its slot back and is
    recomputed later from its prompt and what it had generated; the output is the same as with pages to spare."""
    from lucciola_b200 import Engine, EngineOptions, SamplingParams
    cfg, w, folder = models["D"]                # its window and chunk are longer than the sequences: pages are kept
    prompts = [vz.tokens(cfg, n, salt=51) for n in (60, 50, 40, 30)]
    params = SamplingParams(max_new_tokens=40, ignore_eos=True)
    roomy = Engine(folder, options=EngineOptions(dtype="float32", block_size=16, max_blocks=64, max_tokens_per_step=64, max_num_seqs=4))
    want = roomy.generate(prompts, params)
    tight = Engine(folder, options=EngineOptions(dtype="float32", block_size=16, max_blocks=16, max_tokens_per_step=64, max_num_seqs=4))
    got = tight.generate(prompts, params)
    assert got == want
    assert tight.stats()["preemptions"] > 0 and roomy.stats()["preemptions"] == 0


# ---- the programs ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_trace_run_program(models, tmp_path, dtype, graphs):
    """bin/trace_run as a user runs it on a Venitar folder whose config.json does not name the ranks: the model is chosen by
    config.json, steps come on standard input, <step>.f32 files go out; six requests through its four state slots."""
    import json
    import subprocess
    import sys

    import numpy as np

    from conftest import ROOT
    name = "A"
    cfg, w, folder = models[name]
    reqs = {f"t{i}": vz.tokens(cfg, n, salt=61) for i, n in enumerate((70, 33, 90, 5, 64, 41))}
    steps = ru.mixed(reqs, seed=5, max_live=4)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(ru.max_live_tokens(steps))] + (["--cuda-graph"] if graphs else []),
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got, held = {}, {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        f = out / f"{s['step']}.f32"
        assert f.exists() == (wanted > 0)
        rows = np.fromfile(f, dtype="<f4").reshape(wanted, cfg["vocab"]) if wanted else None
        r = 0
        for e in s["entries"]:
            start = held.get(e["id"], 0)
            for k in e["want"]:
                got[(e["id"], start + k)] = torch.from_numpy(rows[r].astype(np.float64)); r += 1
            held[e["id"]] = start + len(e["tokens"])
    vz.compare(got, name, cfg, w, reqs, dtype, vz.bound(dtype, cfg, w, reqs))


def test_chat_program_and_random_model_program(tmp_path):
    """bin/lucciola_random_model writes a Venitar folder from a config.json; bin/lucciola_chat generates from it, and
    its greedy tokens are the plain implementation's."""
    import json
    import subprocess
    import sys

    from conftest import ROOT
    from lucciola_b200.weights.safetensors_io import SafetensorsFile
    cfg = vz.CONFIGS["B"]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "lucciola_random_model"), "--config", str(tmp_path / "config.json"), "--seed", "3",
                        "--out", str(folder), "--std", "0.3", "--norm-std", "0.1"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    prompt = vz.tokens(cfg, 19, salt=71)
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "lucciola_chat"), "--model", str(folder), "--dtype", "float32", "--max-blocks", "32",
                        "--block-size", "8", "--max-new-tokens", "5", "--ignore-eos", "--prompt-ids", " ".join(map(str, prompt))],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(x) for x in p.stdout.split()[-5:]]
    f = SafetensorsFile(folder / "model.safetensors")
    w = {n: f.get(n).clone() for n in f.names()}
    ids = list(prompt)
    for tok in out:
        row = plain.PlainVenitar(cfg, w).forward(ids)[-1]
        assert row.max() - row[tok] <= 1e-4 * row.abs().max(), (tok, int(row.argmax()))
        ids.append(tok)
