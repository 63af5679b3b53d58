"""Nelovik in the engine against the plain implementation: every mechanism alone, then the whole model under every
way of cutting the work, with pages and state slots that are freed and used again, and generation through the entry
point (GPU)."""
import math
from types import SimpleNamespace

import pytest
import torch

import nelovik_util as nz
import plain_nelovik as plain
import replay_util as ru

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


# ---- each mechanism alone --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("channels,taps,bias,act", [(7, 1, False, True), (40, 2, True, True), (129, 4, False, False), (300, 5, True, True)])
def test_short_convolution_alone(channels, taps, bias, act):
    from lucciola_b200 import ops
    w = torch.randn(channels, taps, device=DEV)
    b = torch.randn(channels, device=DEV) if bias else None
    xs = [torch.randn(n, channels + 3, device=DEV)[:, 3:] for n in (41, 5)]                  # column ranges of wider matrices
    state = torch.zeros(5, max(taps - 1, 1), channels, device=DEV)
    state[2] = float("nan")                                                                  # another request's slot
    wt = w.t().contiguous()

    def forward(rows, step):
        wide = torch.zeros(rows.shape[0], channels + 5, device=DEV)
        wide[:, 5:] = rows
        x = wide[:, 5:]
        out = torch.empty(rows.shape[0], channels, device=DEV)
        ops.short_conv(out, x, wt, b, state if taps > 1 else None, step, stream(), act=act)
        if taps > 1:
            ops.short_conv_state(state, x, taps, step, stream())
        return out
    got = in_portions(forward, xs, [1, 3], SCHEDULE)
    for x, g in zip(xs, got):
        want, _ = plain.short_conv(x.double().cpu(), w.double().cpu(), b.double().cpu() if bias else None, None)
        want = plain.silu(want) if act else want
        assert (g - want).abs().max() <= 3e-6 * max(want.abs().max().item(), 1.0)
    assert torch.isnan(state[2]).all() and torch.isfinite(state[[0, 1, 3]]).all()


def _bind(part, w):
    part.bind_all(lambda name: w[name].to(DEV))


@pytest.mark.parametrize("heads,kv,dim,vdim,taps", [(3, 1, 20, 12, 3), (1, 1, 40, 40, 1), (4, 2, 128, 64, 4), (2, 2, 33, 70, 2), (2, 1, 200, 48, 4),
                                                    (6, 3, 8, 8, 5), (1, 1, 256, 33, 2), (4, 4, 64, 32, 4)])
def test_gated_delta_rule_alone(heads, kv, dim, vdim, taps):
    """Two sequences in unequal portions (single tokens, a few, many) through the part in 32-bit, against the plain
    recurrence; a state row that belongs to another request stays as it is."""
    from lucciola_b200.parts.base import StateCacheView
    from lucciola_b200.parts.delta_rule import GatedDeltaRule
    width = 48
    cfg = nz._config(10, width, 1e-5, [nz._delta(heads, kv, dim, vdim, taps, None)])
    w = {k[len("l0."):]: v.float() for k, v in nz.make_weights(cfg, heads * 100 + dim).items() if k.startswith("l0.mix.")}
    part = GatedDeltaRule(runtime(), "mix", width, heads, kv, dim, vdim, taps, 1e-5)
    _bind(part, w)
    reqs = part.cache_request()
    caches = tuple(StateCacheView(torch.zeros(5, *r.shape, device=DEV)) for r in reqs)
    caches[-1].state[2] = float("nan")
    xs = [torch.randn(n, width, device=DEV) for n in (79, 5)]
    got = in_portions(lambda rows, step: part.forward(rows, step, caches), xs, [1, 3], SCHEDULE)
    sub = {k[len("mix."):]: v.double() for k, v in w.items()}
    for x, g in zip(xs, got):
        want, _ = plain.gated_delta_rule(x.double().cpu(), sub, cfg["layers"][0]["mixer"], 1e-5, None)
        assert (g - want).abs().max() <= 2e-5 * want.abs().max(), (g - want).abs().max() / want.abs().max()
    assert torch.isnan(caches[-1].state[2]).all() and torch.isfinite(caches[-1].state[[1, 3]]).all()


@pytest.mark.parametrize("heads,vdim,state,groups,norm_groups,taps", [(3, 20, 12, 1, 3, 2), (1, 24, 8, 1, 1, 1), (4, 64, 128, 2, 4, 4), (4, 40, 200, 4, 1, 4),
                                                                     (2, 33, 16, 1, 2, 3), (8, 32, 64, 1, 2, 5)])
def test_state_space_alone(heads, vdim, state, groups, norm_groups, taps):
    from lucciola_b200.parts.base import StateCacheView
    from lucciola_b200.parts.state_space import SelectiveStateSpace
    width = 56
    right = nz._right(heads, vdim, state, groups, norm_groups, taps)
    cfg = nz._config(10, width, 1e-6, [nz._pair(nz._left(1, 1, 8, 8, 0.3, 10.0, 0, 10.0, 4, 2), right, None)])
    w = {k[len("l0.mix.right."):]: v.float() for k, v in nz.make_weights(cfg, heads + state).items() if k.startswith("l0.mix.right.")}
    del w["out"]
    part = SelectiveStateSpace(runtime(), "r", width, heads, vdim, state, groups, norm_groups, taps, 1e-6)
    _bind(part, {"r." + k: v for k, v in w.items()})
    caches = tuple(StateCacheView(torch.zeros(5, *r.shape, device=DEV)) for r in part.cache_request())
    xs = [torch.randn(n, width, device=DEV) for n in (79, 5)]
    got = in_portions(lambda rows, step: part.forward(rows, step, caches), xs, [0, 4], SCHEDULE)
    for x, g in zip(xs, got):
        want, _ = plain.mamba2(x.double().cpu(), {k: v.double() for k, v in w.items()}, right, 1e-6, None)
        assert (g - want).abs().max() <= 2e-5 * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,groups,shared", [(36, 3, True), (40, 1, False), (512, 4, False), (96, 8, True), (33, 1, True)])
def test_gated_norm_in_parts_both_orders(dtype, n, groups, shared):
    from lucciola_b200 import ops
    T = 7
    y, gate = torch.randn(T, n, device=DEV) * 3, torch.randn(T, n + 2, device=DEV)[:, 2:]
    w = 1 + 0.3 * torch.randn(n // groups if shared else n, device=DEV)
    wd = w.double().cpu().repeat(groups) if shared else w.double().cpu()
    yd, gd = y.double().cpu(), gate.double().cpu()
    parts = lambda v: plain.rms_norm(v.reshape(T, groups, n // groups), None, 1e-5).reshape(T, n)
    for first in (False, True):
        out = torch.empty(T, n, dtype=dtype, device=DEV)
        ops.gated_group_norm(out, y, gate, w, groups, 1e-5, stream(), gate_first=first, act="silu", scale=0.5)
        want = 0.5 * (parts(yd * plain.silu(gd)) * wd if first else parts(yd) * wd * plain.silu(gd))
        assert (out.double().cpu() - want).abs().max() <= (3e-6 if dtype == torch.float32 else 1e-2) * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_xielu_and_the_other_plain_activations(dtype):
    from lucciola_b200 import ops
    x = (torch.randn(9, 130, device=DEV) * 3).to(dtype)
    x[0, :4] = torch.tensor([0.0, -0.0, 30.0, -30.0], device=DEV).to(dtype)
    p, q = 0.7, -1.3
    sp = lambda v: math.log1p(math.exp(v))
    out = torch.empty_like(x)
    ops.activation(out, x, "xielu", stream(), sp(p), 0.5 + sp(q))
    want = plain.xielu(x.double().cpu(), p, q)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()
    ops.activation(out, x, "silu", stream())
    assert (out.double().cpu() - plain.silu(x.double().cpu())).abs().max() <= tol * 90


@pytest.mark.parametrize("hidden", [40, 72, 256, 1000, 4096])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_norms_of_one_stream_and_the_sum_of_two_normed_rows(hidden, dtype):
    from lucciola_b200 import ops
    T = 6
    r = torch.randn(T, hidden, device=DEV) * 3
    a, b = (torch.randn(T, hidden, device=DEV) for _ in range(2))
    w1, w2 = (1 + 0.3 * torch.randn(hidden, device=DEV) for _ in range(2))
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    for deltas in ((), (a,), (a, b)):
        res = r.clone()
        o1, o2 = (torch.empty(T, hidden, dtype=dtype, device=DEV) for _ in range(2))
        ops.add_rmsnorm_pair(o1, o2, res, deltas, w1, w2, 1e-5, stream())
        x = r.double().cpu() + sum(d.double().cpu() for d in deltas)
        assert (res.double().cpu() - x).abs().max() <= 3e-6 * x.abs().max()
        for o, w in ((o1, w1), (o2, w2)):
            want = plain.rms_norm(x, w.double().cpu(), 1e-5)
            assert (o.double().cpu() - want).abs().max() <= tol * want.abs().max()
    out = torch.empty(T, hidden, device=DEV)
    ops.rmsnorm_mix2(out, a, b, w1, w2, 0.5, 0.25, 1e-5, stream())
    want = 0.5 * plain.rms_norm(a.double().cpu(), w1.double().cpu(), 1e-5) + 0.25 * plain.rms_norm(b.double().cpu(), w2.double().cpu(), 1e-5)
    assert (out.double().cpu() - want).abs().max() <= 3e-6 * want.abs().max()


def test_bias_and_norm_over_whole_projections():
    from lucciola_b200 import ops
    T, nq, nk, nv = 5, 96, 40, 24
    pre = torch.randn(T, nq + nk + nv + 3, device=DEV)
    before = pre.double().cpu()
    bq, bk, bv = (torch.randn(n, device=DEV) for n in (nq, nk, nv))
    wq, wk = (1 + 0.3 * torch.randn(n, device=DEV) for n in (nq, nk))
    ops.bias_rmsnorm_cols(pre, [(0, nq, bq, wq), (nq, nk, bk, wk), (nq + nk, nv, bv, None)], 1e-6, stream())
    got = pre.double().cpu()
    assert (got[:, :nq] - plain.rms_norm(before[:, :nq] + bq.double().cpu(), wq.double().cpu(), 1e-6)).abs().max() <= 3e-6 * 5
    assert (got[:, nq:nq + nk] - plain.rms_norm(before[:, nq:nq + nk] + bk.double().cpu(), wk.double().cpu(), 1e-6)).abs().max() <= 3e-6 * 5
    assert (got[:, nq + nk:nq + nk + nv] - (before[:, nq + nk:nq + nk + nv] + bv.double().cpu())).abs().max() <= 1e-6 * 5
    assert torch.equal(got[:, -3:], before[:, -3:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,page,window,pool", [(3, 1, 20, 12, 8, 24, 5), (4, 2, 64, 64, 16, 40, 16), (2, 2, 32, 80, 4, 7, 3),
                                                               (8, 2, 128, 128, 16, 33, 32), (1, 1, 16, 16, 8, 1, 1), (2, 1, 24, 24, 16, 6, 9),
                                                               (4, 1, 64, 64, 16, 24, 1), (8, 8, 96, 96, 32, 70, 2), (16, 1, 32, 32, 8, 12, 4)])
def test_a_query_finds_its_one_key_or_block_at_every_edge(dtype, heads, kv, dim, vdim, page, window, pool):
    """Keys and values of a long sequence in pages; what has left the window AND been pooled is overwritten with NaN.
    One key far above all others stands in turn just inside the window, just outside it (in a block not yet complete or
    a block already pooled), in the last block a query sees, in the first block, in the block that is not yet seen; the
    query is the last token of the sequence alone (a decoded token) or the last of a portion.  The kernel must agree with a
    plain softmax over the window's keys, the visible blocks' means (as the cache holds them) and the sink."""
    from lucciola_b200 import ops
    n = 5 * max(window, pool) + 3 * pool + 7
    g = torch.Generator(device=DEV).manual_seed(n + heads)
    last = n - 1
    nb_last = max(0, (last - window + 1) // pool)
    spots = {last - window + 1, max(0, last - window), max(0, nb_last * pool - 1), 0, min(last, nb_last * pool), last, max(0, last - pool)}
    sinks = torch.randn(heads, device=DEV, generator=g)
    scale, cap = 0.3, 12.0
    pages = -(-n // page)
    table = torch.arange(pages, dtype=torch.int32, device=DEV).flip(0).reshape(1, pages).contiguous()        # pages in a scrambled order
    far_pages = -(-(n // pool) // page) + 1
    far_table = torch.arange(far_pages, dtype=torch.int32, device=DEV).flip(0).reshape(1, far_pages).contiguous()
    for spot in sorted(spots):
        K = torch.randn(n, kv, dim, device=DEV, generator=g)
        V = torch.randn(n, kv, vdim, device=DEV, generator=g)
        q = torch.randn(3, heads, dim, device=DEV, generator=g)                                          # queries at the last three positions
        K[spot] = 4.0 * q[-1].reshape(kv, heads // kv, dim)[:, 0] / scale / dim ** 0.5                    # stands out for the first head of each group
        kc = torch.zeros(pages, kv, page, dim, dtype=dtype, device=DEV)
        vc = torch.zeros(pages, kv, page, vdim, dtype=dtype, device=DEV)
        pos = torch.arange(n, device=DEV)
        kc[table[0, pos // page].long(), :, pos % page] = K.to(dtype)
        vc[table[0, pos // page].long(), :, pos % page] = V.to(dtype)
        fk = torch.full((far_pages, kv, page, dim), float("nan"), dtype=dtype, device=DEV)
        fv = torch.full((far_pages, kv, page, vdim), float("nan"), dtype=dtype, device=DEV)
        # the blocks are pooled as the steps that complete them would: a long prompt, a portion, single tokens
        for start, count in ((0, n - 9), (n - 9, 6), (n - 3, 1), (n - 2, 1), (n - 1, 1)):
            step = batch_of([count], [0], [start])
            ops.pool_kv(kc, vc, table, fk, fv, far_table, step, kv, dim, vdim, page, pool, stream())
        longest = min(37, n - 1)
        keep_from = (n - longest) - max(window, pool) + 1                                                   # what the window group still holds
        if keep_from > 0:
            gone = torch.arange(0, keep_from, device=DEV)
            gone = gone[(gone // page) < (keep_from // page)]                                                 # whole pages only
            kc[table[0, gone // page].long(), :, gone % page] = float("nan")
            vc[table[0, gone // page].long(), :, gone % page] = float("nan")
        Kc, Vc = K.to(dtype).double(), V.to(dtype).double()
        q = torch.cat([torch.randn(longest - 3, heads, dim, device=DEV, generator=g), q])                    # the queries of the last `longest` positions
        two = table.repeat(2, 1).contiguous(), far_table.repeat(2, 1).contiguous()                           # two requests that read the same pages
        fast = dtype == torch.bfloat16 and dim == vdim and ops.attention_flash_ok(q.to(dtype), heads, kv, dim)
        for qs, starts in (([1], [last]), ([3], [n - 3]), ([longest], [n - longest]), ([1, longest], [last, n - longest]), ([2, 1, 5], [n - 2, last, n - 5])):
            step = batch_of(qs, [0] * len(qs), starts)
            tb, ftb = (table, far_table) if len(qs) == 1 else (two[0][:1].repeat(len(qs), 1).contiguous(), two[1][:1].repeat(len(qs), 1).contiguous())
            qq = torch.cat([q[longest - (n - st): longest - (n - st) + c] for c, st in zip(qs, starts)]).to(dtype).contiguous()
            outs = []
            out = torch.empty(sum(qs), heads, vdim, dtype=dtype, device=DEV)
            ops.attention_plain(qq, out, kc, vc, step.positions, step.token_seq, tb, heads, kv, dim, page, window, scale, stream(),
                                v_dim=vdim, softcap=cap, sinks=sinks, pool=pool, pool_k=fk, pool_v=fv, pool_table=ftb)
            outs.append(("plain", out))
            if fast:
                # the tensor-core kernel: as the engine calls it, and with its keys cut into ranges both ways of combining them
                from lucciola_b200.parts.attention import plan_tiles
                from lucciola_b200.parts.base import BatchShape, PlanView
                made = plan_tiles(BatchShape(list(qs), list(starts), max(qs), n, n), heads // kv)
                view = PlanView({k: torch.from_numpy(a).to(DEV) for k, a in made.arrays.items()}, made.host)
                step.block_tables = [tb, ftb]
                out = torch.full((sum(qs), heads, vdim), float("nan"), dtype=dtype, device=DEV)
                ops.attention(qq, out, kc, vc, step, 0, heads, kv, dim, page, window, scale, stream(), plan=view, softcap=cap, sinks=sinks,
                              pool=pool, pool_k=fk, pool_v=fv, pool_group=1)
                outs.append(("tensor cores", out))
                rows = min(made.host["rows"]["all"], 64)
                for splits, ws in ((2, False), (3, True), (4, False), (5, True)):
                    out = torch.full((sum(qs), heads, vdim), float("nan"), dtype=dtype, device=DEV)
                    ops.attention_flash(qq, out, kc, vc, step.positions, tb, view.arrays["all"], rows, heads, kv, dim, page, window, scale,
                                        splits, stream(), force_workspace=ws, softcap=cap, sinks=sinks, pool=pool, pool_k=fk, pool_v=fv,
                                        pool_table=ftb)
                    outs.append((f"tensor cores, {splits} key ranges", out))
            r = 0
            for c, st in zip(qs, starts):
                for i in range(st, st + c):
                    nb, lo = max(0, (i - window + 1) // pool), max(0, i - window + 1)
                    for h in range(heads):
                        gk = h // (heads // kv)
                        mk = Kc[:nb * pool, gk].reshape(nb, pool, dim).mean(1).to(dtype).double()
                        mv = Vc[:nb * pool, gk].reshape(nb, pool, vdim).mean(1).to(dtype).double()
                        keys, vals = torch.cat([mk, Kc[lo:i + 1, gk]]), torch.cat([mv, Vc[lo:i + 1, gk]])
                        sc = cap * torch.tanh(keys @ qq[r, h].double() * scale / cap)
                        e = torch.exp(sc - sc.max())
                        want = (e[:, None] * vals).sum(0) / (e.sum() + torch.exp(sinks[h].double() - sc.max()))
                        for which, out in outs:
                            err = (out[r, h].double() - want).abs().max().item()
                            assert err <= (1e-5 if dtype == torch.float32 else 3e-2) * max(want.abs().max().item(), 0.3), (which, spot, qs, i, h, err)
                    r += 1


# ---- the whole model -------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, weights, folder).  Beside A and C: "Asharp" / "Csharp", whose attention picks out single keys and blocks."""
    out = {}
    for name, cfg in nz.CONFIGS.items():
        w = nz.make_weights(cfg, 100 + len(out))
        out[name] = (cfg, w, nz.write_model(tmp_path_factory.mktemp(f"nelovik_{name}"), cfg, w))
    for base in ("A", "C"):
        cfg = nz.CONFIGS[base]
        w = nz.make_weights(cfg, 200 + len(out), sharp=4.0)
        out[base + "sharp"] = (cfg, w, nz.write_model(tmp_path_factory.mktemp(f"nelovik_{base}sharp"), cfg, w))
    return out


def make_runner(models, name, dtype, num_pages, graphs=False, slots=4, **kw):
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    page = nz.PAGE[name[0]]
    return build_runner(models[name][2], EngineOptions(dtype=dtype, block_size=page, max_blocks=num_pages, max_num_seqs=slots,
                                                       use_cuda_graph=graphs, graph_after=1, max_shape_graphs=1000, **kw),
                        num_pages=num_pages)


TOL_SHARP = {"float32": 1e-4, "bfloat16": 0.12}


def check(models, name, dtype, steps, reqs, graphs=False, poison=True, tol=None, slots=4):
    page = nz.PAGE[name[0]]
    cfg, w, _ = models[name]
    if tol is None:
        tol = nz.bound(dtype, cfg, w, reqs, TOL_SHARP[dtype] if "sharp" in name else None)
    runner = make_runner(models, name, dtype, max(ru.max_live_tokens(steps) // page, 1), graphs=graphs, slots=slots)
    got = ru.replay(runner, steps, poison=poison)
    worst = nz.compare(got, name, cfg, w, reqs, dtype, tol)
    assert runner.manager.num_requests() == 0 and all(p.num_free == p.num_pages for p in runner.manager.pools)
    return runner, got, worst


LENGTHS = {"A": [1, 2, 15, 16, 17, 47, 130], "B": [1, 7, 8, 9, 64, 120], "C": [3, 31, 32, 33, 129, 300], "D": [1, 16, 65, 140, 400]}


def requests_for(models, name):
    cfg = models[name][0]
    return {f"{name}{n}": nz.tokens(cfg, n, salt=len(name)) for n in LENGTHS[name[0]]}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "Asharp", "Csharp"])
@pytest.mark.parametrize("cut", ["whole", "tail_decoded", "portions"])
def test_each_request_alone(models, name, dtype, cut):
    """Whole prompts (lengths at and beside page borders, windows and blocks), prompt then token-by-token decoding, and
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
    reqs = {f"m{i}": nz.tokens(cfg, n, salt=seed + 3) for i, n in enumerate((70, 9, 120, 33, 101, 2, 64, 47, 90))}
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
        reqs = {f"m{i}": nz.tokens(cfg, n, salt=5) for i, n in enumerate((70, 9, 120, 33, 101, 2, 64, 47, 90))}
        steps = ru.mixed(reqs, seed=4, decodes_first=True)
    else:
        reqs = requests_for(models, name)
        steps = getattr(ru, cut)(reqs)
    page = nz.PAGE[name[0]]
    runner = make_runner(models, name, "bfloat16", max(ru.max_live_tokens(steps) // page, 1), graphs=True)
    assert runner._can_record
    tol = nz.bound("bfloat16", cfg, w, reqs)
    first = ru.replay(runner, steps, poison=True)
    nz.compare(first, name, cfg, w, reqs, "bfloat16", tol)
    recorded, replays = len(runner._graphs), runner.graph_replays
    assert recorded > 0
    second = ru.replay(runner, steps, poison=True)
    nz.compare(second, name, cfg, w, reqs, "bfloat16", tol)
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
                assert (runs[0][key] - other[key]).abs().max() <= 2 * nz.TOL[dtype] * runs[0][key].abs().max(), key


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Asharp", "Csharp", "D"])
def test_long_decoding_past_windows_and_blocks_with_old_state(models, name, dtype):
    """A short prompt, then hundreds of tokens decoded one by one: every window passes over decoded tokens (pages are
    given back as it does), blocks are completed by decoded tokens, and the slow decays still carry what entered the
    states at the start."""
    cfg = models[name][0]
    ids = nz.tokens(cfg, 390, salt=9)
    steps = ru.tail_decoded({"long": ids}, tail=387)
    _, got, _ = check(models, name, dtype, steps, {"long": ids})
    assert len(got) == 388


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Asharp", "Csharp"])
def test_the_edges_of_windows_and_blocks_really_matter(models, name, dtype):
    """The sharpened model must be one in which single keys matter: replacing the token that stands just inside the
    attention layer's window of the last query changes the last logits by far more than the 32-bit tolerance.  Then the
    engine, the prompt in portions that end at, before and behind the borders of pages and blocks, against the plain
    implementation."""
    cfg, w, _ = models[name]
    left = next(l for l in cfg["layers"] if l["type"] == "parallel")["mixer"]["left"]
    window, pool = left["mask"]["size"], left["mask"]["pool"]
    ids = nz.tokens(cfg, 200, salt=21)
    other = list(ids)
    other[199 - (window - 1)] = (ids[199 - (window - 1)] + 1) % cfg["vocab"]
    a, b = nz.plain_logits(name, cfg, w, ids), nz.plain_logits(name, cfg, w, other)
    assert (a[-1] - b[-1]).abs().max() > 20 * TOL_SHARP["float32"] * a.abs().max()
    page = nz.PAGE[name[0]]
    steps = ru.portions({"edge": ids}, sizes=(page - 1, 2, page, page + 1, pool, pool - 1 or 1, 2, pool + 1, 2 * page - 2, 3, 5 * page, 1, 1, 2))
    check(models, name, dtype, steps, {"edge": ids})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(models, name, dtype):
    """Positions 0 to 5: a single key, fewer tokens than a window holds, no block yet, a page with one token, empty
    states, convolutions that reach before the start."""
    cfg = models[name][0]
    for n in (1, 2, 3, 6):
        ids = nz.tokens(cfg, n, salt=n)
        for steps in (ru.whole({"f": ids}), ru.tail_decoded({"f": ids}, tail=n - 1) if n > 1 else ru.whole({"f": ids})):
            check(models, name, dtype, steps, {"f": ids})


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_against_each_alone(models, dtype):
    """Five unequal prompts in one step, then their next tokens in one step: every row equals the request run alone."""
    name = "C"
    cfg = models[name][0]
    reqs = {f"b{n}": nz.tokens(cfg, n, salt=31) for n in (2, 40, 17, 128, 65)}
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
    cfg = nz.random_config(seed)
    reqs = {f"q{i}": nz.tokens(cfg, n, salt=seed) for i, n in enumerate((1, 23, 97, 200, 64))}
    w = nz.make_weights(cfg, 300 + seed)
    folder = nz.write_model(tmp_path / "model", cfg, w)
    for dtype in DTYPES:
        for cut in ("whole", "portions", "mixed", "tail_decoded"):
            steps = getattr(ru, cut)(reqs)
            pages = max(ru.max_live_tokens(steps) // 16, 1)
            runner = build_runner(folder, EngineOptions(dtype=dtype, block_size=16, max_blocks=pages, max_num_seqs=4,
                                                        use_cuda_graph=(cut == "mixed"), graph_after=1), num_pages=pages)
            got = ru.replay(runner, steps, poison=True)
            nz.compare(got, ("drawn", seed), cfg, w, reqs, dtype, tol=5e-5 if dtype == "float32" else nz.bound(dtype, cfg, w, reqs, 5e-2))


# ---- through the entry point -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 0.3)])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(models, name, dtype, slack):
    """Engine.generate with the scheduler's own batching: prompts longer than a step's budget (so they are read in
    portions beside decoding requests), more requests than state slots.  Every generated token must be the plain
    implementation's choice for the same prefix, or lose to it by a near-tie."""
    from lucciola_b200 import Engine, EngineOptions, SamplingParams
    cfg, w, folder = models[name]
    eng = Engine(folder, options=EngineOptions(dtype=dtype, block_size=nz.PAGE[name[0]], max_blocks=64, max_tokens_per_step=48, max_num_seqs=3))
    prompts = [nz.tokens(cfg, n, salt=41) for n in (5, 70, 33, 1, 100)]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert all(len(o) == 6 for o in outs)
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for k, tok in enumerate(out):
            row = nz.plain_logits(name, cfg, w, ids)[-1]
            assert row.max() - row[tok] <= slack * row.abs().max().clamp(min=1.0), f"token {k}: chose {tok}, plain chooses {int(row.argmax())}"
            ids.append(tok)
    assert eng.runner.manager.num_requests() == 0 and all(p.num_free == p.num_pages for p in eng.runner.manager.pools)


def test_generation_under_page_pressure_recomputes_the_state(models):
    """Fewer pages than the requests need together: a request is preempted, gives its pages and its slot back and is
    recomputed later from its prompt and what it had generated; the output is the same as with pages to spare."""
    from lucciola_b200 import Engine, EngineOptions, SamplingParams
    cfg, w, folder = models["D"]                # its first layer's window is longer than the sequences: pages are kept
    prompts = [nz.tokens(cfg, n, salt=51) for n in (60, 50, 40, 30)]
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
    """bin/trace_run as a user runs it on a Nelovik folder: the model is chosen by config.json, steps come on standard
    input, <step>.f32 files go out; six requests through its four state slots."""
    import json
    import subprocess
    import sys

    import numpy as np

    from conftest import ROOT
    name = "A"
    cfg, w, folder = models[name]
    reqs = {f"t{i}": nz.tokens(cfg, n, salt=61) for i, n in enumerate((70, 33, 90, 5, 64, 41))}
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
    nz.compare(got, name, cfg, w, reqs, dtype, nz.bound(dtype, cfg, w, reqs))


def test_chat_program_and_random_model_program(tmp_path):
    """bin/lucciola_random_model writes a Nelovik folder from a config.json; bin/lucciola_chat generates from it, and
    its greedy tokens are the plain implementation's."""
    import json
    import subprocess
    import sys

    from conftest import ROOT
    from lucciola_b200.weights.safetensors_io import SafetensorsFile
    cfg = nz.CONFIGS["B"]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "lucciola_random_model"), "--config", str(tmp_path / "config.json"), "--seed", "3",
                        "--out", str(folder), "--std", "0.3", "--norm-std", "0.1"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    prompt = nz.tokens(cfg, 19, salt=71)
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "lucciola_chat"), "--model", str(folder), "--dtype", "float32", "--max-blocks", "32",
                        "--block-size", "8", "--max-new-tokens", "5", "--ignore-eos", "--prompt-ids", " ".join(map(str, prompt))],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(x) for x in p.stdout.split()[-5:]]
    f = SafetensorsFile(folder / "model.safetensors")
    w = {n: f.get(n).clone() for n in f.names()}
    ids = list(prompt)
    for tok in out:
        row = plain.PlainNelovik(cfg, w).forward(ids)[-1]
        assert row.max() - row[tok] <= 1e-4 * row.abs().max(), (tok, int(row.argmax()))
        ids.append(tok)
