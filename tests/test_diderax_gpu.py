"""Diderax on the GPU: every new kernel form alone against its reference at sizes other than any
model's, with inputs made so that a fault shows (a key far back that carries all the weight, a sink
that takes it away, NaN in pages and slots that belong to nobody, choice scores that are all negative);
the whole model in float32 and bfloat16 against the plain implementation under every cut of the work;
slots and pages used again; long decoding; greedy generation through ``LLM`` with recorded decode
steps; the command line; and ``bin/trace_run`` as a subprocess."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import kernel_refs as refs
import plain_diderax as plain
import replay_cases as cases
from diderax_cases import CONFIGS, CONFIG_D, assert_rows_close, oracle as plain_oracle, random_config, write_model
from fegilix_cases import FakeStep, run_steps
from guzovik_cases import FakeCtx
from tiny_configs import random_prompt

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DTYPES = [torch.float32, torch.bfloat16]


def _rand(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()


def _tol(dtype):
    return {"atol": 2e-5, "rtol": 2e-5} if dtype == torch.float32 else {"atol": 2e-2, "rtol": 2e-2}


class Arena:
    def take(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device="cuda")


class Ctx(FakeCtx):
    def __init__(self, query_lens, context_lens):
        super().__init__(query_lens, context_lens, device="cuda")
        self.arena = Arena()


def _tables(lens, page, seed):
    """Block tables over shuffled pages (two spare pages stay NaN), as a device tensor and lists."""
    need = [-(-n // page) for n in lens]
    order = torch.randperm(sum(need) + 2, generator=torch.Generator().manual_seed(seed)).tolist()
    tables, at = [], 0
    for n in need:
        tables.append(order[at: at + n])
        at += n
    width = max(need)
    dev = torch.tensor([t + [0] * (width - len(t)) for t in tables], dtype=torch.int32, device="cuda")
    return tables, dev, sum(need) + 2


# ------------------------------------------------------------ kernels one by one
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, groups, d, rotary", [(4, 2, 32, 8), (1, 1, 48, 2), (6, 3, 64, 64), (2, 1, 128, 32), (3, 3, 24, 0),
                                                      (5, 1, 17, 4)])
def test_norm_over_the_whole_projection_kernel(dtype, heads, groups, d, rotary) -> None:
    """q and k normed over all their heads at once with a weight per element, the values the raw keys; q, k and
    the gate are column slices of one wider product."""
    from tinyserve_b200.kernels import ops

    t, page = 21, 4
    wide = _rand(t, (heads + groups) * d + 5, seed=1, scale=2.0, dtype=dtype)
    q, k = wide[:, : heads * d], wide[:, heads * d: (heads + groups) * d]
    qw, kw = (1 + _rand(heads * d, seed=2, scale=0.3)).to(dtype), (1 + _rand(groups * d, seed=3, scale=0.3)).to(dtype)
    pos = torch.arange(100, 100 + t, dtype=torch.float64)
    cos = sin = None
    if rotary:
        ang = pos[:, None] * (1e4 ** (-torch.arange(0, rotary, 2, dtype=torch.float64) / rotary) / 6.0)[None, :]
        cos, sin = ang.cos().float().cuda(), ang.sin().float().cuda()
    slots = torch.randperm(8 * page, generator=torch.Generator().manual_seed(4))[:t].int().cuda()
    res = []
    for impl in (ops, refs):
        kc = torch.full((8, groups, page, d), float("nan"), dtype=dtype, device="cuda")
        vc = torch.full((8, groups, page, d), float("nan"), dtype=dtype, device="cuda")
        qo = torch.empty(t, heads, d, dtype=dtype, device="cuda")
        impl.qkv_prepare(q, k, k, qw, kw, 1e-6, cos, sin, rotary, slots, kc, vc, page, heads, groups, d, d, qo, norm_whole=True)
        res.append((qo.float(), kc.float(), vc.float()))
    for got, want in zip(*res):
        torch.testing.assert_close(got, want, equal_nan=True, **_tol(dtype))
    sl = slots.long()
    assert torch.equal(res[0][2][sl // page, :, sl % page], k.float().view(t, groups, d)), "the values are the keys as projected"
    per_head = torch.empty(t, heads, d, dtype=dtype, device="cuda")
    ops.qkv_prepare(q, None, None, qw[:d].contiguous(), None, 1e-6, cos, sin, rotary, None, None, None, page, heads, groups, d, d, per_head)
    if heads > 1:
        assert (per_head.float() - res[0][0]).abs().max() > 1e-2, "the norm over all heads equals the norm head by head"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, width, pad", [(1, 8, 0), (33, 80, 160), (7, 515, 3), (300, 128, 8), (5, 1536, 64)])
def test_norm_of_a_column_slice_kernel(dtype, rows, width, pad) -> None:
    from tinyserve_b200.kernels import ops

    wide = _rand(rows, width + pad, seed=1, scale=3.0, dtype=dtype)
    w = (1 + _rand(width, seed=2, scale=0.3)).to(dtype)
    got, want = torch.empty(rows, width, dtype=dtype, device="cuda"), torch.empty(rows, width, dtype=dtype, device="cuda")
    ops.rms_norm_rows(wide[:, :width], w, 1e-6, got)
    refs.rms_norm_rows(wide[:, :width], w, 1e-6, want)
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, hidden", [(1, 48), (37, 256), (5, 37), (300, 1024)])
def test_layer_scale_pending_kernel(dtype, rows, hidden) -> None:
    from tinyserve_b200.kernels import ops

    x, y = _rand(rows, hidden, seed=1, scale=2.0), _rand(rows, hidden, seed=2, scale=3.0, dtype=dtype)
    ls, w = (1 + _rand(hidden, seed=3, scale=0.3)).to(dtype), (1 + _rand(hidden, seed=4, scale=0.3)).to(dtype)
    bias = _rand(hidden, seed=5, dtype=dtype)
    for b in (None, bias):              # the sub-layer's output bias rides along with the pending output
        got_x, want_x = x.clone(), x.clone()
        got, want = torch.empty(rows, hidden, dtype=dtype, device="cuda"), torch.empty(rows, hidden, dtype=dtype, device="cuda")
        ops.post_norm_add_rms_norm(got_x, y, None, ls, 0.0, False, w, False, 1e-6, got, delta_bias=b)
        refs.post_norm_add_rms_norm(want_x, y, None, ls, 0.0, False, w, False, 1e-6, want, delta_bias=b)
        torch.testing.assert_close(got_x, want_x, atol=1e-5, rtol=1e-5)
        added = y.float() if b is None else y.float() + b.float()
        torch.testing.assert_close(got_x, x + ls.float() * added, atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))


def _sink_case(dtype, heads, rank, rot, page, lens, news, sinks, far=None):
    """The kernels and the references on the same cached rows: the new tokens of every request attend to all
    its rows. ``far``: the last query of request 0 points strongly at the key at that position."""
    from tinyserve_b200.kernels import ops

    tables, table, pages = _tables(lens, page, 7)
    d = rank + rot
    store = torch.full((pages * page, d), float("nan"), dtype=dtype, device="cuda")
    for b, n in enumerate(lens):
        rows = _rand(n, d, seed=40 + b, scale=0.5, dtype=dtype)
        if far is not None and b == 0:
            rows[far] = 0
            rows[far, 0] = 8.0
        idx = torch.tensor([tables[b][p // page] * page + p % page for p in range(n)], device="cuda")
        store[idx] = rows
    t = sum(news)
    q = _rand(t, heads, d, seed=3, scale=0.5, dtype=dtype)
    if far is not None:
        q[news[0] - 1] = 0
        q[news[0] - 1, :, 0] = 8.0
    ctx = Ctx(news, lens)
    res = []
    for impl in (ops, refs):
        out = torch.empty(t, heads, rank, dtype=dtype, device="cuda")
        impl.latent_attention(q, store, page, table, ctx, rank, 1.0, 0, out, sinks=sinks)
        res.append(out.float())
    return res[0], res[1], store, tables


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, rank, rot, page", [(3, 20, 8, 4), (8, 64, 32, 16), (1, 12, 2, 8), (10, 128, 32, 16), (4, 32, 16, 32)])
def test_latent_attention_with_sinks_kernels(dtype, heads, rank, rot, page) -> None:
    """Prompt portions and single tokens (those of long requests are cut into key ranges on the tensor cores and
    merged: the sink must count once, not once per range)."""
    sinks = _rand(heads, seed=9, scale=2.0)
    for lens, news in (([page * 3 + 1, 170, 33, 1, 400], [1, 17, 33, 1, 130]), ([700, 650, 900, 1], [1, 1, 1, 1])):
        got, want, *_ = _sink_case(dtype, heads, rank, rot, page, lens, news, sinks)
        assert not got.isnan().any()
        torch.testing.assert_close(got, want, **_tol(dtype))
        none, *_ = _sink_case(dtype, heads, rank, rot, page, lens, news, None)
        assert (none - got).abs().max() > 1e-2, "the sink changes nothing"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("new", [1, 2, 70])
@pytest.mark.parametrize("rank, rot, page", [(16, 8, 16), (64, 32, 16), (24, 2, 4)])
def test_a_far_key_and_a_sink_that_takes_its_weight(dtype, new, rank, rot, page) -> None:
    """One key among hundreds carries all the weight, at the first position, at page borders and just before the
    query: the output is its latent. A sink far above its score leaves nothing."""
    heads, total = 4, 600
    for far in (0, 1, page - 1, page, 5 * page, 333, total - new - 1, total - 2, total - 1):
        quiet = torch.full((heads,), -30.0, device="cuda")
        got, want, store, tables = _sink_case(dtype, heads, rank, rot, page, [total, 40], [new, 1], quiet, far=far)
        torch.testing.assert_close(got, want, **_tol(dtype))
        latent = store[tables[0][far // page] * page + far % page, :rank].float()
        for h in range(heads):
            torch.testing.assert_close(got[new - 1, h], latent, atol=3e-2, rtol=3e-2)
        loud = torch.full((heads,), 90.0, device="cuda")
        got, want, *_ = _sink_case(dtype, heads, rank, rot, page, [total, 40], [new, 1], loud, far=far)
        assert got[new - 1].abs().max() < 1e-3 and want[new - 1].abs().max() < 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, d, dv, tau", [(2, 16, 24, 4.0), (1, 40, 16, 16.0), (3, 8, 8, 0.5), (2, 64, 64, 16.0), (1, 128, 40, 1.0),
                                               (1, 256, 32, 8.0)])
def test_gated_linear_scan_kernel(dtype, heads, d, dv, tau) -> None:
    """Prompt portions, single tokens and a portion long enough to run in segments, from and to state slots that
    are not in order; q, k, v are column slices of one product. The pad slot and foreign slots stay as they are."""
    from tinyserve_b200.kernels import ops

    for lens in ([5, 1, 33, 1, 2], [1, 1, 1], [300, 7, 1], [16, 17]):
        t = sum(lens)
        wide = _rand(t, 2 * heads * d + heads * dv + 3, seed=1, scale=0.5, dtype=dtype)
        q, k, v = wide[:, : heads * d], wide[:, heads * d: 2 * heads * d], wide[:, 2 * heads * d: 2 * heads * d + heads * dv]
        z, bias = _rand(t, heads * d, seed=2, scale=2.0), _rand(heads * d, seed=3)
        slots = torch.randperm(len(lens) + 2, generator=torch.Generator().manual_seed(5))[: len(lens)].tolist()
        start = _rand(len(lens) + 3, heads * d * dv, seed=4, scale=0.3)
        res = []
        for impl in (ops, refs):
            state = start.clone()
            ctx = FakeStep(lens, slots, device="cuda")
            ctx.arena = Arena()
            out = torch.full((t, heads, dv), float("nan"), device="cuda")
            impl.linear_scan_gated(q, k, v, z, bias, tau, d ** -0.5, state, ctx, heads, d, dv, out)
            res.append((out, state))
        scale = max(1.0, float(res[1][0].abs().max()))
        tol = 2e-5 * scale if dtype == torch.float32 else 2e-2 * scale
        torch.testing.assert_close(res[0][0], res[1][0], atol=tol, rtol=tol)
        torch.testing.assert_close(res[0][1], res[1][1], atol=tol, rtol=tol)
        untouched = [s for s in range(len(lens) + 3) if s not in slots]
        assert torch.equal(res[0][1][untouched], start[untouched])


def test_gated_linear_scan_in_segments_of_several_lengths() -> None:
    from tinyserve_b200.kernels import ops

    heads, d, dv, lens = 2, 32, 48, [700, 257, 1, 64]
    t = sum(lens)
    q, k, v = (_rand(t, heads * n, seed=s, scale=0.5) for s, n in ((1, d), (2, d), (3, dv)))
    z, bias = _rand(t, heads * d, seed=4, scale=2.0) + 2.0, _rand(heads * d, seed=5)
    want_state = torch.zeros(5, heads * d * dv, device="cuda")
    want = torch.empty(t, heads, dv, device="cuda")
    ctx = FakeStep(lens, [3, 0, 1, 2], device="cuda")
    refs.linear_scan_gated(q, k, v, z, bias, 4.0, d ** -0.5, want_state, ctx, heads, d, dv, want)
    saved = ops.LINEAR_SCAN_SEGMENT_TOKENS
    try:
        for seg in (None, 16, 64, 100, 512):
            ops.LINEAR_SCAN_SEGMENT_TOKENS = seg
            state = torch.zeros(5, heads * d * dv, device="cuda")
            out = torch.empty(t, heads, dv, device="cuda")
            ctx = FakeStep(lens, [3, 0, 1, 2], device="cuda")
            ctx.arena = Arena()
            ops.linear_scan_gated(q, k, v, z, bias, 4.0, d ** -0.5, state, ctx, heads, d, dv, out)
            tol = 2e-5 * float(want.abs().max())
            torch.testing.assert_close(out, want, atol=tol, rtol=2e-5)
            torch.testing.assert_close(state, want_state, atol=tol, rtol=2e-5)
    finally:
        ops.LINEAR_SCAN_SEGMENT_TOKENS = saved


@pytest.mark.parametrize("tokens", [1, 9, 64, 65, 700])
@pytest.mark.parametrize("outputs, identity, top, groups, keep, scale", [(8, 2, 3, 4, 2, 2.0), (6, 3, 3, 2, 1, 1.0), (2, 1, 1, 1, 1, 1.5),
                                                                         (12, 0, 4, 3, 2, 0.5), (24, 6, 5, 3, 1, 1.75), (5, 0, 2, 1, 1, 1.0),
                                                                         (96, 32, 8, 32, 5, 2.5), (40, 0, 32, 1, 1, 1.0)])
def test_scored_routing_kernel(tokens, outputs, identity, top, groups, keep, scale) -> None:
    """Picks, weights and the sorted order against the reference; the router's outputs are the first columns of
    a wider product; the correction makes every choice score negative for some tokens."""
    from tinyserve_b200.kernels import ops

    wide = _rand(tokens, outputs + 1, seed=1, scale=3.0)
    corr = _rand(outputs, seed=2, scale=0.3) - 0.4
    rule = ops.RouteRule(scored=True, groups=groups, keep=keep, scale=scale, identity=identity, correction=corr)
    real = outputs - identity
    counts = torch.zeros(real, dtype=torch.int32, device="cuda")
    plan = ops.moe_route(wide, top, counts, Arena(), rule=rule, outputs=outputs)
    want = refs.moe_route(wide, top, None, rule=rule, outputs=outputs)
    assert torch.equal(plan["ids"], want["ids"])
    torch.testing.assert_close(plan["weights"], want["weights"], atol=1e-6, rtol=1e-5)
    assert torch.equal(plan["offsets"], want["offsets"]) and int(counts.abs().sum()) == 0
    ids, rows = plan["ids"].long(), plan["row_of"].long()
    assert torch.equal(rows < 0, ids >= real), "identity picks take no row, all others one"
    queued = rows[rows >= 0]
    assert sorted(queued.tolist()) == list(range(len(queued))), "every sorted row belongs to one pick"
    offsets = plan["offsets"].long()
    pick = torch.nonzero(rows >= 0).reshape(-1)
    assert bool(((rows[pick] >= offsets[ids[pick]]) & (rows[pick] < offsets[ids[pick] + 1])).all())
    assert torch.equal(plan["token_of"].long()[rows[pick]], pick // top)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, top, hidden", [(1, 1, 48), (37, 3, 256), (5, 4, 37), (130, 8, 1024)])
def test_combine_with_identity_picks_and_a_gated_shared_expert_kernel(dtype, tokens, top, hidden) -> None:
    from tinyserve_b200.kernels import ops

    picks = tokens * top
    g = torch.Generator().manual_seed(3)
    rows = torch.randperm(picks, generator=g).int()
    rows[torch.rand(picks, generator=g) < 0.4] = -1
    plan = {"top": top, "picks": picks, "row_of": rows.cuda(), "weights": _rand(picks, seed=4).abs(), "identity": 1}
    y, x, shared = _rand(picks, hidden, seed=5, dtype=dtype), _rand(tokens, hidden, seed=6, dtype=dtype), _rand(tokens, hidden, seed=7, dtype=dtype)
    unused = sorted(set(range(picks)) - set(rows[rows >= 0].tolist()))
    y[unused] = float("nan")                # an identity pick reads the token's input, never a row of y
    gate = _rand(tokens, 5, seed=8, scale=2.0)[:, 4]
    for sh, gt in ((shared, gate), (shared, None), (None, None)):
        got, want = torch.empty(tokens, hidden, dtype=dtype, device="cuda"), torch.empty(tokens, hidden, dtype=dtype, device="cuda")
        ops.moe_combine(y, plan, sh, got, x=x, shared_gate=gt)
        refs.moe_combine(y, plan, sh, want, x=x, shared_gate=gt)
        torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, experts, identity, top, hidden, ff", [(9, 4, 2, 3, 64, 24), (300, 6, 2, 3, 128, 64), (700, 8, 4, 3, 256, 256),
                                                                        (1500, 4, 12, 4, 512, 256)])
def test_experts_with_identity_picks_from_routing_to_combine(dtype, tokens, experts, identity, top, hidden, ff) -> None:
    """The whole mixture against the references, at sizes that take each form of the experts' products (the largest
    ones sort and gather the rows for tiles of 128): rows of the sorted order that no pick owns are never looked up."""
    from tinyserve_b200.kernels import ops

    outputs = experts + identity
    x = _rand(tokens, hidden, seed=1, dtype=dtype)
    w_router = _rand(outputs + 1, hidden, seed=2, scale=0.3, dtype=dtype)
    w_gu, w_down = _rand(experts, 2 * ff, hidden, seed=3, scale=0.1, dtype=dtype), _rand(experts, hidden, ff, seed=4, scale=0.1, dtype=dtype)
    shared = _rand(tokens, hidden, seed=5, dtype=dtype)
    rule = ops.RouteRule(scored=True, groups=2, keep=1, scale=1.5, identity=identity, correction=_rand(outputs, seed=6, scale=0.05))
    res = []
    for impl in (ops, refs):
        arena = Arena()
        counts = torch.zeros(experts, dtype=torch.int32, device="cuda")
        tile_rows = impl.moe_tile_rows(tokens, top, experts, dtype, (hidden, ff))
        plan = impl.moe_route_from(x, w_router, top, counts, arena, tile_rows, rule, outputs)
        act = torch.full((tokens * top, ff), float("nan"), dtype=dtype, device="cuda")
        impl.moe_gemm(x, w_gu, act, plan, gated=True, gather=True, arena=arena)
        y = torch.full((tokens * top, hidden), float("nan"), dtype=dtype, device="cuda")
        impl.moe_gemm(act, w_down, y, plan, gated=False, gather=False, arena=arena)
        out = torch.empty(tokens, hidden, dtype=dtype, device="cuda")
        impl.moe_combine(y, plan, shared, out, x=x, shared_gate=plan["logits"][:, outputs])
        res.append((out.float(), plan))
    (got, plan), (want, ref_plan) = res
    assert not got.isnan().any()
    if dtype == torch.float32:
        assert torch.equal(plan["ids"], ref_plan["ids"])
        torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)
    else:
        same = (plan["ids"].view(tokens, top) == ref_plan["ids"].view(tokens, top)).all(-1)      # rounding may flip a close call
        assert float(same.float().mean()) > 0.97
        torch.testing.assert_close(got[same], want[same], atol=2e-2 * float(want.abs().max()), rtol=6e-2)     # bfloat16 steps at the outputs' size
    assert bool((plan["ids"] >= experts).any()) and bool((plan["ids"] < experts).any())


# ------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {k: write_model(tmp_path_factory.mktemp("diderax" + k), k) for k in CONFIGS}


LENGTHS = {"A": [1, 2, 9, 37, 70, 131], "B": [3, 33, 64, 97, 150], "C": [5, 18, 40, 120], "D": [2, 47, 160, 230]}


@pytest.fixture(scope="module")
def oracle(folders):
    out = {}
    for which in CONFIGS:
        vocab = plain.read_config(folders[which])["vocab"]
        reqs = {f"r{i}": random_prompt(n, vocab, 200 + 7 * i) for i, n in enumerate(LENGTHS[which])}
        out[which] = (reqs, {rid: plain_oracle(folders[which], toks) for rid, toks in reqs.items()})
    return out


def _check(got, reqs, want, dtype, what) -> None:
    assert all(sorted(got[rid]) == list(range(len(reqs[rid]))) for rid in got)
    rows = torch.cat([torch.stack([got[rid][p] for p in range(len(reqs[rid]))]) for rid in got])
    assert_rows_close(rows, torch.cat([want[rid][0] for rid in got]), torch.cat([want[rid][1] for rid in got]), dtype, what)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which, page", [("A", 4), ("A", 16), ("B", 8), ("B", 16), ("C", 16), ("C", 32), ("D", 16), ("D", 8)])
def test_model_under_every_cut(folders, oracle, dtype, which, page) -> None:
    from tinyserve_b200.model import DecoderModel

    reqs, want = oracle[which]
    model = DecoderModel.from_folder(folders[which], dtype, "cuda")
    plans = [cases.mixed(reqs, 3), cases.mixed(reqs, 4, max_live=2)]
    for rid, toks in reqs.items():
        plans += [cases.whole(rid, toks), cases.tail_decoded(rid, toks, 32), cases.portions(rid, toks, 1)]
    for n, steps in enumerate(plans):
        got, _ = run_steps(model, page, steps, cases.max_live_tokens(steps))
        _check(got, reqs, want, dtype, f"{which}, schedule {n}")


@pytest.mark.parametrize("seed", list(range(1, 13)))
def test_configurations_drawn_at_random(seed, tmp_path) -> None:
    """Sizes, head counts, ranks, groups, identity experts, layer order and constants drawn at random; a prompt
    alone, decoded token by token, in portions, and mixed with others, in both types."""
    from tinyserve_b200.model import DecoderModel

    cfg = random_config(seed)
    folder = write_model(tmp_path, cfg, seed)
    reqs = {f"r{i}": random_prompt(n, cfg["vocab"], 300 + seed + 7 * i) for i, n in enumerate([2, 35, 90, 61])}
    want = {rid: plain_oracle(folder, toks) for rid, toks in reqs.items()}
    page = [4, 8, 16, 32][seed % 4]
    plans = [cases.mixed(reqs, seed), cases.whole("r2", reqs["r2"]), cases.tail_decoded("r2", reqs["r2"], 40), cases.portions("r3", reqs["r3"], seed)]
    for dtype in DTYPES:
        model = DecoderModel.from_folder(folder, dtype, "cuda")
        for n, steps in enumerate(plans):
            got, _ = run_steps(model, page, steps, cases.max_live_tokens(steps))
            _check(got, reqs, want, dtype, f"seed {seed}, schedule {n}: {json.dumps(cfg)[:300]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompts(dtype, tmp_path) -> None:
    """Prompts of several hundred tokens: the linear scans of a long portion run in segments, a decoded token's
    latent attention is cut into key ranges. Whole, in long and short portions (one just above the bound),
    decoded at the end, and mixed with a short request."""
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.model import DecoderModel

    folder = write_model(tmp_path, CONFIG_D, 31)
    vocab = CONFIG_D["vocab"]
    reqs = {"long": random_prompt(700, vocab, 41), "mid": random_prompt(300, vocab, 42), "short": random_prompt(9, vocab, 43)}
    assert ops.linear_scan_segments(700, 1, 2, 64, 64)[1] > 1 and ops.linear_scan_segments(257, 3, 2, 64, 64)[1] > 1
    want = {rid: plain_oracle(folder, toks) for rid, toks in reqs.items()}
    model = DecoderModel.from_folder(folder, dtype, "cuda")
    plans = [cases.whole("long", reqs["long"]), cases.tail_decoded("long", reqs["long"], 20),
             cases.portions("long", reqs["long"], 1, sizes=(300, 257, 2, 100)), cases.mixed(reqs, 2)]
    for n, steps in enumerate(plans):
        got, _ = run_steps(model, 16, steps, cases.max_live_tokens(steps))
        _check(got, {rid: reqs[rid] for rid in got}, want, dtype, f"long prompts, schedule {n}")


def test_batch_mates_pages_and_slots_do_not_matter(folders, oracle) -> None:
    """float32: a request's logits alone, beside others, and again on the pages and in the slot that another
    request has just given back, agree to rounding."""
    from tinyserve_b200.engine.replay import Replayer
    from tinyserve_b200.model import DecoderModel

    reqs, _ = oracle["A"]
    model = DecoderModel.from_folder(folders["A"], torch.float32, "cuda")
    toks, other = reqs["r4"], reqs["r5"]
    rep = Replayer(model, 256, page_size=4, max_live=2)
    alone = rep.run_step([("x", toks, [len(toks) - 1])], ["x"]).clone()
    rep.run_step([("y", other[:50], [])], [])
    beside = rep.run_step([("y", other[50:51], []), ("x", toks, [len(toks) - 1])], ["x", "y"]).clone()
    again = rep.run_step([("z", toks[:7], []), ("w", other[:3], [])], [])
    again = rep.run_step([("w", other[3:4], []), ("z", toks[7:], [len(toks) - 8])], ["z", "w"]).clone()
    torch.testing.assert_close(beside, alone, atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(again, alone, atol=2e-5, rtol=2e-5)
    assert rep.cache.state_pool.num_free == 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "D"])
def test_long_decoding(folders, dtype, which) -> None:
    from tinyserve_b200.model import DecoderModel

    vocab = plain.read_config(folders[which])["vocab"]
    toks = random_prompt(150, vocab, 9)
    want = plain_oracle(folders[which], toks)
    model = DecoderModel.from_folder(folders[which], dtype, "cuda")
    got, _ = run_steps(model, 16, cases.tail_decoded("a", toks, 145), 192)
    rows = torch.stack([got["a"][p] for p in range(150)])
    assert_rows_close(rows, *want, dtype, "all tokens")


def test_a_far_token_decides_the_logits(folders) -> None:
    """A model of attention layers alone: changing the second token of a prompt of several hundred changes the
    logits of the last, decoded, token, by what the plain model says."""
    from tinyserve_b200.model import DecoderModel

    cfg = {"architecture": "Diderax", "vocab": 50, "width": 32, "norm": {"eps": 1e-5},
           "layers": [{"type": "attention", "mlp": None, "mixer": CONFIGS["A"][0]["layers"][3]["mixer"]},
                      {"type": "latent_attention", "mlp": None, "mixer": CONFIGS["C"][0]["layers"][4]["mixer"]}]}
    folder = write_model(folders["A"].parent / "attention_only", cfg, 3)
    model = DecoderModel.from_folder(folder, torch.float32, "cuda")
    base = random_prompt(300, 50, 1)
    changed = list(base)
    changed[1] = (base[1] + 1) % 50

    def last_logits(toks):
        got, _ = run_steps(model, 4, cases.tail_decoded("a", toks, 20), 320)
        return got["a"][len(toks) - 1]

    ref, got = last_logits(base), last_logits(changed)
    assert (got - ref).abs().max() > 1e-5, "a token far back no longer reaches the last query"
    want = plain_oracle(folder, changed)
    assert_rows_close(got[None], want[0][299:], want[1][299:], torch.float32, "far token")


def _with_overlap(mask, fn):
    """``fn()`` with the launch-overlap mask of every kind of step set to ``mask``."""
    from tinyserve_b200.kernels import ops

    saved = (ops.PREFILL_PDL_MASK, ops.SMALL_DECODE_PDL_MASK, ops.DEFAULT_PDL_MASK)
    try:
        ops.PREFILL_PDL_MASK = ops.SMALL_DECODE_PDL_MASK = ops.DEFAULT_PDL_MASK = mask
        ops.set_programmatic_launch(mask)
        return fn()
    finally:
        ops.PREFILL_PDL_MASK, ops.SMALL_DECODE_PDL_MASK, ops.DEFAULT_PDL_MASK = saved
        ops.set_programmatic_launch(saved[2])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "D"])
def test_overlapping_launches_change_no_bit(folders, oracle, dtype, which) -> None:
    """A kernel that starts while the kernels before it still run must read their results behind its wait: the
    logits of mixed steps, decoded tokens and portions are equal bit for bit with the overlap on and off."""
    from tinyserve_b200.model import DecoderModel

    reqs, _ = oracle[which]
    model = DecoderModel.from_folder(folders[which], dtype, "cuda")
    long = list(reqs)[-1]
    for steps in (cases.mixed(reqs, 5), cases.tail_decoded(long, reqs[long], 40), cases.portions(long, reqs[long], 3)):
        rows = {}
        for mask in (0, -1):
            got, _ = _with_overlap(mask, lambda: run_steps(model, 16, steps, cases.max_live_tokens(steps)))
            rows[mask] = torch.cat([torch.stack([got[r][p] for p in sorted(got[r])]) for r in sorted(got)])
        assert torch.equal(rows[0], rows[-1])


def test_a_long_prompt_at_a_real_width_with_overlapping_launches() -> None:
    """2,048 tokens at width 1,024 through linear attention and experts with identity experts: the experts' products
    run on sorted, gathered rows in tiles of 128, of which the identity picks own none. Two different prompts one
    after the other on the same scratch, overlap on and off: equal bit for bit, and no row of garbage is looked up."""
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.engine.replay import Replayer
    from tinyserve_b200.model import DecoderModel

    cfg = {"architecture": "Diderax", "vocab": 1000, "width": 1024, "norm": {"eps": 1e-6}, "layers": [
        {"type": "gla", "mixer": {"heads": 8, "dim": 128, "vdim": 128, "tau": 8.0, "decay_rank": 64},
         "mlp": {"kind": "moe", "router": {"experts": 16, "identity": 4, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}},
                 "expert": {"ff": 768}, "shared": {"ff": 768}}}]}
    model = DecoderModel.from_config(config_from_dict(cfg), seed=1, dtype=torch.bfloat16, device="cuda")
    prompts = [random_prompt(2048, 1000, s) for s in (1, 2)]

    def run():
        rep = Replayer(model, 4096, page_size=16, max_live=2)
        return torch.cat([rep.run_step([(f"p{i}", p, [0, 1000, 2047])], [f"p{i}"]).clone() for i, p in enumerate(prompts)])

    plain, overlapped = _with_overlap(0, run), _with_overlap(-1, run)
    assert not plain.isnan().any() and torch.equal(plain, overlapped)


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("which", ["A", "D"])
def test_greedy_generation_through_llm(folders, graphs, which) -> None:
    from tinyserve_b200 import LLM

    cfg, w = plain.read_config(folders[which]), plain.read_weights(folders[which], torch.float64)
    prompts = [random_prompt(n, cfg["vocab"], 40 + n) for n in (3, 11, 26, 50)]
    want = [plain.greedy(cfg, w, p, 8) for p in prompts]
    llm = LLM.from_folder(folders[which], dtype="float32", page_size=8, num_pages=64, max_num_seqs=3, max_batch_tokens=32,
                          chunked_prefill=True, decode_graphs=graphs)
    assert llm.generate(prompts, max_new_tokens=8) == want
    assert (llm.engine.runner.num_graph_steps > 0) == graphs
    assert all(g.allocator.num_used == 0 for g in llm.cache.groups)


def test_command_line(folders) -> None:
    cfg, w = plain.read_config(folders["A"]), plain.read_weights(folders["A"], torch.float64)
    prompt = random_prompt(19, cfg["vocab"], 77)
    want = plain.greedy(cfg, w, prompt, 8)
    cmd = [sys.executable, str(ROOT / "bin" / "generate"), "--model-dir", str(folders["A"]), "--prompt-ids", ",".join(map(str, prompt)),
           "--max-new-tokens", "8", "--dtype", "float32", "--block-size", "8"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert f"new ids:    {want}" in out.stdout


def test_trace_run_subprocess(folders, oracle, tmp_path) -> None:
    reqs, want = oracle["C"]
    steps = cases.mixed(reqs, 6, max_live=3)
    lines = [json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": p} for r, t, p in entries], "end": end})
             for i, (entries, end) in enumerate(steps)]
    out = tmp_path / "out"
    vocab = plain.read_config(folders["C"])["vocab"]
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders["C"]), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", str(cases.max_live_tokens(steps)), "--max-requests", "3"],
                          input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [x for x in proc.stdout.split("\n") if x.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    fed: dict[str, int] = {}
    for i, (entries, _) in enumerate(steps):
        rows = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab))
        at = 0
        for rid, toks, places in entries:
            base = fed.get(rid, 0)
            for p in places:
                w, c = want[rid]
                assert_rows_close(rows[at][None], w[base + p][None], c[base + p][None], torch.float32, f"{rid} at {base + p}")
                at += 1
            fed[rid] = base + len(toks)
