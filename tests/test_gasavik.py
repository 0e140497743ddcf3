"""Gasavik on the host: its configuration and tensor names; the kernels' references against the
plain implementation, one mechanism at a time; and the whole engine (cache manager, step function,
scheduler, sampler) with the references in the kernels' place against the plain model, under
every cut of the work."""

from __future__ import annotations

import copy
import json

import pytest
import torch

import kernel_refs as refs
import plain_gasavik as plain
import replay_cases as cases
from fegilix_cases import FakeStep, run_steps
from gasavik_cases import CONFIGS, CONFIG_A, CONFIG_B, CONFIG_C, assert_rows_close, oracle as plain_oracle, random_config, write_model
from kernel_refs import use_references
from tiny_configs import random_prompt

from tinyserve_b200.cache.allocator import PageAllocator
from tinyserve_b200.cache.block_table import RELEASED, BlockTable
from tinyserve_b200.config import UnsupportedConfigError, config_from_dict
from tinyserve_b200.model import DecoderModel, build_parts
from tinyserve_b200.parts import SplitKVNeed, KVNeed, StateNeed
from tinyserve_b200.weights.loader import checkpoint_names, merge_specs


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {k: write_model(tmp_path_factory.mktemp("gasavik" + k), k) for k in CONFIGS}


def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


# ------------------------------------------------------------------ configuration
def test_config_round_trip_and_names(folders) -> None:
    for which, (cfg, _) in CONFIGS.items():
        c = config_from_dict(cfg)
        assert config_from_dict(c.to_dict()) == c
        assert json.loads((folders[which] / "config.json").read_text())["architecture"] == "Gasavik"
    names = checkpoint_names(merge_specs(build_parts(config_from_dict(CONFIG_A).to_spec()).tensor_specs()))
    assert names["embed"] == (97, 64) and names["pos"] == (160, 64) and names["embed.norm"] == (64,)
    assert names["side.embed"] == (97, 4 * 8) and names["l2.side.gate"] == (8, 64) and names["l2.side.proj"] == (64, 8)
    assert names["l0.mix.mu.w"] == (64,) and names["l0.mix.r"] == (32, 64) and names["l0.mix.w1"] == (8, 64)
    assert names["l0.mix.w2"] == (32, 8) and names["l0.mix.u"] == (2, 16) and names["l0.mix.norm"] == (32,)
    assert names["l1.mix.left.q"] == (128, 64) and names["l1.mix.left.k.b"] == (64,) and names["l1.mix.left.v"] == (32, 64)
    assert names["l1.mix.left.g"] == (4, 64) and names["l1.mix.left.q.norm"] == (32,) and names["l1.mix.left.o"] == (64, 64)
    assert names["l1.mix.right.k"] == (32, 64) and names["l1.mix.right.g"] == (64, 64) and names["l1.mix.right.norm"] == (64,)
    assert names["l1.mlp.up.b"] == (96,) and names["l1.mlp.down.b"] == (64,)
    assert names["l2.mix.q.conv"] == (32, 3) and names["l2.mix.v"] == (96, 64) and names["l2.mix.b"] == (4, 64)
    assert names["l2.mix.A_log"] == (4,) and names["l2.mix.dt_bias"] == (4,) and names["l2.mix.norm"] == (24,)
    assert not any(n.startswith("l2.mlp.") for n in names) and "l0.norm2" not in names
    assert names["final.norm"] == (64,) and names["head"] == (97, 64)
    b = checkpoint_names(merge_specs(build_parts(config_from_dict(CONFIG_B).to_spec()).tensor_specs()))
    assert "side.embed" not in b and not any(".side." in n for n in b)


def test_cache_needs(folders) -> None:
    model = DecoderModel.from_folder(folders["A"], torch.float32, "cpu")
    assert model.cache_needs() == [
        StateNeed((2 * 16 * 16 + 64,), torch.float32), SplitKVNeed(2, 32, 16, 9, 3), StateNeed((2 * 16 * 32,), torch.float32),
        StateNeed((4 * 16 * 24 + 2 * (2 * 2 * 16 + 4 * 24),), torch.float32), SplitKVNeed(1, 16, 32, 21, 18),
        StateNeed((3 * 8 * 16,), torch.float32)]
    b = DecoderModel.from_folder(folders["B"], torch.float32, "cpu").cache_needs()
    assert b[0] == KVNeed(3, 16, 12, 0) and b[4] == KVNeed(1, 32, None, 0)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown mixer type"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "decay constants"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "has no 'scale'"),
    (lambda c: c["layers"][1]["mixer"]["left"]["mask"].update(size=0), "size must be positive"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "only 'dense'"),
    (lambda c: c.pop("max_positions"), "has no 'max_positions'"),
    (lambda c: c["layers"][2]["mixer"].pop("conv"), "has no 'conv'"),
])
def test_config_refusals(change, message) -> None:
    cfg = copy.deepcopy(CONFIG_A)
    change(cfg)
    with pytest.raises(UnsupportedConfigError, match=message):
        config_from_dict(cfg)


# ----------------------------------------------- pages in front of a window that stay
def test_block_table_keeps_the_first_pages() -> None:
    alloc = PageAllocator(32)
    t = BlockTable(alloc, 4, window=6, keep_first=5)          # positions 0..4 lie on pages 0 and 1
    for n in (3, 9, 1, 1, 14, 1):
        t.append(n)
        t.release_passed()
        first_needed = max(0, t.num_tokens - 6 + 1)
        for i, p in enumerate(t.pages):
            needed = i < 2 or (i + 1) * 4 > first_needed
            assert (p != RELEASED) == needed, (t.num_tokens, i)
        assert alloc.num_used == len(t.live_pages())
    t.release()
    assert alloc.num_used == 0


# ------------------------------------------- the references, one mechanism at a time
def _mixer_weights(prefix: str, shapes: dict, seed: int) -> dict:
    return {prefix + n: _rand(*s, seed=seed + i, scale=0.5) for i, (n, s) in enumerate(shapes.items())}


@pytest.mark.parametrize("cuts", [[11], [4, 7], [1, 1, 2, 7], [2] * 5 + [1]])
def test_reference_time_mixing(cuts) -> None:
    heads, d, width, t = 3, 8, 20, 11
    w = _mixer_weights("m.", {"r": (24, width), "k": (24, width), "v": (24, width), "w_pre": (t, 24), "w0": (24,), "u": (heads, d)}, 1)
    h = _rand(t, width, seed=9)
    r, k, v = h @ w["m.r"].T, h @ w["m.k"].T, h @ w["m.v"].T
    want = torch.zeros(t, heads, d, dtype=torch.float64)
    decay = torch.exp(-torch.exp(w["m.w_pre"] + w["m.w0"]))
    for a in range(heads):
        S = torch.zeros(d, d, dtype=torch.float64)
        sl = slice(a * d, (a + 1) * d)
        for i in range(t):
            kv = torch.outer(k[i, sl], v[i, sl])
            want[i, a] = (S + w["m.u"][a][:, None] * kv).T @ r[i, sl]
            S = decay[i, sl][:, None] * S + kv
    state = torch.zeros(3, heads * d * d, dtype=torch.float64)
    got = torch.zeros(t, heads, d, dtype=torch.float64)
    at = 0
    for n in cuts:
        step = FakeStep([n], [1])
        part = torch.zeros(n, heads, d, dtype=torch.float64)
        refs.linear_scan_bonus(r[at: at + n], k[at: at + n], v[at: at + n], w["m.w_pre"][at: at + n], w["m.w0"], w["m.u"].reshape(-1),
                               state, step, heads, d, d, part)
        got[at: at + n] = part
        at += n
    torch.testing.assert_close(got, want)
    assert state[0].abs().sum() == 0 and state[2].abs().sum() == 0


@pytest.mark.parametrize("cuts", [[9], [2, 7], [1] * 9])
def test_reference_decayed_linear_attention_and_token_shift(cuts) -> None:
    heads, d, dv, t = 2, 8, 5, 9
    q, k, v = _rand(t, heads * d, seed=1), _rand(t, heads * d, seed=2), _rand(t, heads * dv, seed=3)
    decay = torch.tensor([0.5, 0.97], dtype=torch.float64)
    want = torch.zeros(t, heads, dv, dtype=torch.float64)
    for a in range(heads):
        S = torch.zeros(d, dv, dtype=torch.float64)
        for i in range(t):
            S = decay[a] * S + torch.outer(plain.silu(k[i, a * d: (a + 1) * d]), plain.silu(v[i, a * dv: (a + 1) * dv]))
            want[i, a] = S.T @ plain.silu(q[i, a * d: (a + 1) * d])
    state, shift = torch.zeros(2, heads * d * dv, dtype=torch.float64), torch.zeros(2, 6, dtype=torch.float64)
    x, mu = _rand(t, 6, seed=4), _rand(3, 6, seed=5)
    before = torch.cat([torch.zeros(1, 6, dtype=torch.float64), x[:-1]])
    want_mix = x[None] + (before - x)[None] * mu[:, None]
    got, got_mix, at = torch.zeros_like(want), torch.zeros_like(want_mix), 0
    for n in cuts:
        part, mix = torch.zeros(n, heads, dv, dtype=torch.float64), torch.zeros(3, n, 6, dtype=torch.float64)
        refs.linear_scan_decay(q[at: at + n], k[at: at + n], v[at: at + n], decay, state, FakeStep([n], [0]), heads, d, dv, part)
        refs.token_shift_mix(x[at: at + n], mu, shift, FakeStep([n], [0]), mix)
        got[at: at + n], got_mix[:, at: at + n] = part, mix
        at += n
    torch.testing.assert_close(got, want)
    torch.testing.assert_close(got_mix, want_mix)


def test_reference_delta_rule_with_one_decay_per_head() -> None:
    heads, groups, d, dv, t = 4, 2, 6, 5, 7
    qkv = _rand(t, 2 * groups * d + heads * dv, seed=1)
    a, beta, dt_bias, a_log = _rand(t, heads, seed=2), _rand(t, heads, seed=3), _rand(heads, seed=4), _rand(heads, seed=5, scale=0.3)
    want = torch.zeros(t, heads, dv, dtype=torch.float64)
    for hd in range(heads):
        g, S = hd // 2, torch.zeros(d, dv, dtype=torch.float64)
        for i in range(t):
            q = plain.unit(qkv[i, g * d: (g + 1) * d]) * d ** -0.5
            k = plain.unit(qkv[i, groups * d + g * d: groups * d + (g + 1) * d])
            v = qkv[i, 2 * groups * d + hd * dv: 2 * groups * d + (hd + 1) * dv]
            S = torch.exp(-torch.exp(a_log[hd]) * plain.softplus(a[i, hd] + dt_bias[hd])) * S
            S = S + torch.outer(k, torch.sigmoid(beta[i, hd]) * (v - S.T @ k))
            want[i, hd] = S.T @ q
    state, got = torch.zeros(1, heads * d * dv, dtype=torch.float64), torch.zeros_like(want)
    for lo, hi in ((0, 3), (3, 4), (4, 7)):
        part = torch.zeros(hi - lo, heads, dv, dtype=torch.float64)
        refs.delta_scan(qkv[lo:hi], 0, groups * d, 2 * groups * d, a[lo:hi], dt_bias, a_log, beta[lo:hi], d ** -0.5, state,
                        FakeStep([hi - lo], [0]), heads, groups, d, dv, part)
        got[lo:hi] = part
    torch.testing.assert_close(got, want)


@pytest.mark.parametrize("window, keep", [(5, 0), (5, 3), (3, 7), (1, 1), (40, 2)])
def test_reference_attention_keeps_the_first_tokens(window, keep) -> None:
    """One key carries all the weight; it is seen exactly when the mask says so."""
    t, d, page = 23, 8, 4
    k_cache, v_cache = torch.zeros(8, 1, page, d, dtype=torch.float64), torch.zeros(8, 1, page, d, dtype=torch.float64)
    table = torch.tensor([[5, 2, 7, 0, 3, 6]], dtype=torch.int32)
    keys, vals = _rand(t, d, seed=1, scale=0.1), _rand(t, d, seed=2)
    for far in range(t):
        kk = keys.clone()
        kk[far] = 0
        kk[far, 0] = 50.0                                      # the query below points at this key alone
        for p in range(t):
            k_cache[table[0, p // page], 0, p % page], v_cache[table[0, p // page], 0, p % page] = kk[p], vals[p]
        for new in (1, 4):
            q = torch.zeros(new, 1, d, dtype=torch.float64)
            q[:, 0, 0] = 1.0
            ctx = FakeStep([new], [0])
            ctx.context_lens_dev = torch.tensor([t], dtype=torch.int32)
            out = torch.zeros(new, d, dtype=torch.float64)
            refs.paged_attention(q, k_cache, v_cache, page, table, ctx, 1.0, window, out, keep_first=keep)
            for r in range(new):
                i = t - new + r
                seen = plain.visible(i, far, window, keep)
                assert torch.allclose(out[r], vals[far], atol=1e-6) == seen, (far, i, seen)


def test_reference_pieces_around_the_stream() -> None:
    t, h = 5, 12
    resid, y1, y2, bias = _rand(t, h, seed=1), _rand(t, h, seed=2), _rand(t, h, seed=3), _rand(h, seed=4)
    want = resid + 0.7 * 0.8 * y1 + 0.7 * y2 + 0.7 * bias
    copy_ = torch.zeros(t, h, dtype=torch.float64)
    refs.stream_sum(resid, [y1, y2], [0.7 * 0.8, 0.7], bias=bias, bias_scale=0.7, copy=copy_)
    torch.testing.assert_close(resid, want, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(copy_, want, atol=1e-5, rtol=1e-5)
    table, pos, nw = _rand(9, h, seed=5), _rand(30, h, seed=6), _rand(h, seed=7)
    toks, places = torch.tensor([3, 8, 0]), torch.tensor([0, 1, 29])
    out = torch.zeros(3, h, dtype=torch.float64)
    refs.embed_pos_norm(toks, places, table, pos, nw, 1e-5, out)
    torch.testing.assert_close(out, plain.rms_norm(table[toks] + pos[places], nw, 1e-5), atol=1e-5, rtol=1e-5)
    side, x = _rand(9, 8, seed=8), _rand(3, 4, seed=9)
    gated = torch.zeros(3, 4, dtype=torch.float64)
    refs.act_mul_gather(x, toks, side, 4, gated, "gelu_tanh")
    torch.testing.assert_close(gated, plain.gelu_tanh(x) * side[toks][:, 4:8], atol=1e-5, rtol=1e-5)


# ----------------------------------------------- the engine on the host, every cut
LENGTHS = {"A": [1, 2, 9, 37, 70], "B": [3, 45, 90], "C": [5, 18, 40], "D": [2, 21, 50]}


@pytest.fixture(scope="module")
def oracle(folders):
    out = {}
    for which in CONFIGS:
        vocab = plain.read_config(folders[which])["vocab"]
        reqs = {f"r{i}": random_prompt(n, vocab, 100 + 7 * i) for i, n in enumerate(LENGTHS[which])}
        out[which] = (reqs, {rid: plain_oracle(folders[which], toks) for rid, toks in reqs.items()})
    return out


@pytest.mark.parametrize("which, page", [("A", 4), ("A", 16), ("B", 8), ("C", 4), ("D", 16)])
def test_engine_on_host_under_every_cut(folders, oracle, which, page) -> None:
    reqs, want = oracle[which]
    model = DecoderModel.from_folder(folders[which], torch.float32, "cpu")
    plans = [cases.mixed(reqs, 3), cases.mixed(reqs, 5, max_live=2)]
    for rid, toks in reqs.items():
        plans += [cases.whole(rid, toks), cases.tail_decoded(rid, toks, 12), cases.portions(rid, toks, 1)]
    with use_references():
        for steps in plans:
            got, _ = run_steps(model, page, steps, cases.max_live_tokens(steps))
            for rid in got:
                rows = torch.stack([got[rid][p] for p in range(len(reqs[rid]))])
                assert_rows_close(rows, *want[rid], torch.float32, f"{which}/{rid}")


@pytest.mark.parametrize("kind", ["parallel", "wkv", "delta"])
def test_each_mixer_alone_on_host(kind, tmp_path) -> None:
    """A model of one layer of one kind, without a feed-forward and without a token input."""
    layer = next(copy.deepcopy(x) for x in CONFIG_A["layers"] + CONFIG_C["layers"] if x["type"] == kind)
    layer["mlp"] = None
    cfg = {"architecture": "Gasavik", "vocab": 53, "width": 40, "max_positions": 64, "norm": {"eps": 1e-5}, "layers": [layer]}
    folder = write_model(tmp_path, cfg, 5)
    toks = random_prompt(33, 53, 8)
    want = plain_oracle(folder, toks)
    model = DecoderModel.from_folder(folder, torch.float32, "cpu")
    with use_references():
        for steps in (cases.whole("a", toks), cases.portions("a", toks, 2), cases.tail_decoded("a", toks, 20)):
            got, _ = run_steps(model, 4, steps, cases.max_live_tokens(steps))
            assert_rows_close(torch.stack([got["a"][p] for p in range(len(toks))]), *want, torch.float32, kind)


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_configurations_drawn_at_random_on_host(seed, tmp_path) -> None:
    cfg = random_config(seed)
    folder = write_model(tmp_path, cfg, seed)
    reqs = {f"r{i}": random_prompt(n, cfg["vocab"], 10 * seed + i) for i, n in enumerate((1, 14, 47))}
    want = {rid: plain_oracle(folder, toks) for rid, toks in reqs.items()}
    model = DecoderModel.from_folder(folder, torch.float32, "cpu")
    with use_references():
        for steps in (cases.mixed(reqs, seed), cases.portions("r2", reqs["r2"], seed)):
            got, _ = run_steps(model, 8, steps, cases.max_live_tokens(steps))
            for rid in got:
                assert_rows_close(torch.stack([got[rid][p] for p in range(len(reqs[rid]))]), *want[rid], torch.float32, f"{seed}/{rid}")


def test_greedy_generation_through_the_engine_on_host(folders) -> None:
    from tinyserve_b200.cache import CacheManager
    from tinyserve_b200.engine import Engine

    cfg, w = plain.read_config(folders["A"]), plain.read_weights(folders["A"], torch.float64)
    prompts = [random_prompt(n, cfg["vocab"], 40 + n) for n in (3, 11, 26)]
    want = [plain.greedy(cfg, w, p, 6) for p in prompts]
    model = DecoderModel.from_folder(folders["A"], torch.float32, "cpu")
    for kw in (dict(num_pages=64), dict(num_pages=64, max_batch_tokens=8, chunked_prefill=True), dict(num_pages=6)):
        pages = kw.pop("num_pages")
        cache = CacheManager(model.cache_needs(), page_size=8, num_pages=pages, max_requests=3, dtype=torch.float32, device="cpu")
        with use_references():
            e = Engine(model, cache, max_num_seqs=3, **kw)
            assert e.generate(prompts, 6) == want
        assert all(g.allocator.num_used == 0 for g in cache.groups)
    assert len({tuple(x) for x in want}) > 1
