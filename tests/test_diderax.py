"""Diderax on the host: its configuration and tensor names; the kernels' references against the
plain implementation, one mechanism at a time, with inputs made so that a fault shows; and the whole
engine (cache manager, step function, scheduler, sampler) with the references in the kernels' place
against the plain model, under every cut of the work."""

from __future__ import annotations

import copy
import json
import math

import pytest
import torch

import kernel_refs as refs
import plain_diderax as plain
import replay_cases as cases
from diderax_cases import CONFIGS, CONFIG_A, CONFIG_B, CONFIG_C, assert_rows_close, oracle as plain_oracle, random_config, write_model
from fegilix_cases import FakeStep, run_steps
from kernel_refs import use_references
from tiny_configs import random_prompt

from tinyserve_b200.config import UnsupportedConfigError, config_from_dict
from tinyserve_b200.kernels.ops import RouteRule
from tinyserve_b200.model import DecoderModel, build_parts
from tinyserve_b200.parts import KVNeed, StateNeed
from tinyserve_b200.parts.base import LatentNeed
from tinyserve_b200.parts.rope import RotaryEncoding
from tinyserve_b200.weights.loader import checkpoint_names, merge_specs


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {k: write_model(tmp_path_factory.mktemp("diderax" + k), k) for k in CONFIGS}


def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


# ------------------------------------------------------------------ configuration
def test_config_round_trip_and_names(folders) -> None:
    for which, (cfg, _) in CONFIGS.items():
        c = config_from_dict(cfg)
        assert config_from_dict(c.to_dict()) == c
        assert json.loads((folders[which] / "config.json").read_text())["architecture"] == "Diderax"
    names = checkpoint_names(merge_specs(build_parts(config_from_dict(CONFIG_A).to_spec()).tensor_specs()))
    assert names["embed"] == (97, 64) and names["final.norm"] == (64,) and names["head"] == (97, 64)
    assert names["l0.norm1"] == (64,) and names["l0.ls1"] == (64,) and names["l0.ls2"] == (64,)
    assert names["l0.mix.q"] == (32, 64) and names["l0.mix.v"] == (48, 64) and names["l0.mix.g"] == (48, 64)
    assert names["l0.mix.a1"] == (6, 64) and names["l0.mix.a2"] == (32, 6) and names["l0.mix.a2.b"] == (32,)
    assert names["l0.mix.norm"] == (24,) and names["l0.mix.o"] == (64, 48)
    assert names["l0.mlp.router"] == (8, 64) and names["l0.mlp.correction"] == (8,) and names["l0.mlp.e5.down"] == (64, 24)
    assert "l0.mlp.e6.gate" not in names, "identity experts have no tensors"
    assert names["l0.mlp.shared.sg"] == (1, 64) and names["l0.mlp.shared.up"] == (40, 64)
    assert names["l1.mix.q"] == (128, 64) and names["l1.mix.k"] == (64, 64) and "l1.mix.v" not in names
    assert names["l1.mix.q.norm"] == (128,) and names["l1.mix.k.norm"] == (64,) and names["l1.mix.g"] == (128, 64)
    assert names["l1.mlp.gate.b"] == (80,) and names["l1.mlp.down.b"] == (64,)
    assert names["l2.mix.dq"] == (20, 64) and names["l2.mix.dq.norm"] == (20,) and names["l2.mix.uq"] == (3 * 24, 20)
    assert names["l2.mix.dkv"] == (40, 64) and names["l2.mix.dkv.norm"] == (32,) and names["l2.mix.uk"] == (48, 32)
    assert names["l2.mix.uv"] == (72, 32) and names["l2.mix.sink"] == (3,) and names["l2.mix.o"] == (64, 72)
    assert not any(n.startswith("l2.mlp.") or n in ("l2.norm2", "l2.ls2") for n in names)
    assert "l3.mlp.shared.sg" not in names and names["l3.mlp.router"] == (5, 64)


def test_cache_needs(folders) -> None:
    model = DecoderModel.from_folder(folders["A"], torch.float32, "cpu")
    assert model.cache_needs() == [StateNeed((2 * 16 * 24,), torch.float32), KVNeed(2, 32, None, 0), LatentNeed(40, None),
                                   KVNeed(1, 16, None, 0)]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown mixer type"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=16), "vdim=16 must equal dim=32"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "has no 'scale'"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "must be even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(scaling={"factor": 0.0}), "must be positive"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "has no 'q_rank'"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0.0), "tau=0.0 must be positive"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "do not fit"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "do not fit"),
    (lambda c: c["layers"][1]["mlp"].update(kind="conv"), "'dense' and 'moe'"),
    (lambda c: c.pop("vocab"), "has no 'vocab'"),
])
def test_config_refusals(change, message) -> None:
    cfg = copy.deepcopy(CONFIG_A)
    change(cfg)
    with pytest.raises(UnsupportedConfigError, match=message):
        config_from_dict(cfg)


def test_rotary_frequencies_divided_by_the_factor() -> None:
    enc = RotaryEncoding(head_dim=32, rotary_dim=8, theta=1e4, pairing="half", scaling={"factor": 4.0})
    want = torch.tensor([1e4 ** (-2.0 * i / 8) / 4.0 for i in range(4)], dtype=torch.float64)
    torch.testing.assert_close(enc._inv_freq_host, want)
    plain_enc = RotaryEncoding(head_dim=32, rotary_dim=8, theta=1e4, pairing="half")
    assert enc.key() != plain_enc.key()


# ------------------------------------------- the references, one mechanism at a time
@pytest.mark.parametrize("cuts", [[11], [4, 7], [1, 1, 2, 7], [2] * 5 + [1]])
def test_reference_gated_linear_attention(cuts) -> None:
    heads, d, dv, width, t, tau = 3, 8, 5, 20, 11, 4.0
    h = _rand(t, width, seed=9)
    w = {"m." + n: _rand(*s, seed=i + 1, scale=0.5) for i, (n, s) in enumerate({
        "q": (24, width), "k": (24, width), "v": (15, width), "g": (15, width), "a1": (4, width), "a2": (24, 4), "a2.b": (24,),
        "norm": (dv,), "o": (width, 15)}.items())}
    q, k, v = h @ w["m.q"].T, h @ w["m.k"].T, h @ w["m.v"].T
    z = (h @ w["m.a1"].T) @ w["m.a2"].T
    state = torch.zeros(3, heads * d * dv, dtype=torch.float64)
    read = torch.zeros(t, heads, dv, dtype=torch.float64)
    at = 0
    for n in cuts:
        part = torch.zeros(n, heads, dv, dtype=torch.float64)
        refs.linear_scan_gated(q[at: at + n], k[at: at + n], v[at: at + n], z[at: at + n], w["m.a2.b"], tau, d ** -0.5, state,
                               FakeStep([n], [1]), heads, d, dv, part)
        read[at: at + n] = part
        at += n
    gated = torch.zeros(t, heads * dv, dtype=torch.float64)
    refs.head_norm_gate(read, w["m.norm"], False, h @ w["m.g"].T, True, 1e-5, gated, gate_silu=True)
    want = plain.gla_mixer(h, w, "m.", {"heads": heads, "dim": d, "vdim": dv, "tau": tau}, 1e-5)
    torch.testing.assert_close(gated @ w["m.o"].T, want, atol=1e-5, rtol=1e-5)      # the gate reference works in 32-bit
    assert state[0].abs().sum() == 0 and state[2].abs().sum() == 0 and state[1].abs().sum() > 0


def test_a_decay_of_one_keeps_and_a_decay_of_zero_forgets() -> None:
    """Pre-activations of +40 and -40 make the decay 1 and (with a small tau) 0: the state then holds every
    token's write, or only the last one's."""
    heads, d, dv, t = 1, 4, 3, 6
    q, k, v = _rand(t, d, seed=1), _rand(t, d, seed=2), _rand(t, dv, seed=3)
    for z0, want_fn in ((40.0, lambda i: sum(torch.outer(k[j], v[j]) for j in range(i + 1))), (-40.0, lambda i: torch.outer(k[i], v[i]))):
        state = torch.zeros(1, d * dv, dtype=torch.float64)
        out = torch.zeros(t, heads, dv, dtype=torch.float64)
        refs.linear_scan_gated(q, k, v, torch.full((t, d), z0, dtype=torch.float64), torch.zeros(d, dtype=torch.float64), 0.5, 1.0,
                               state, FakeStep([t], [0]), heads, d, dv, out)
        for i in range(t):
            torch.testing.assert_close(out[i, 0], want_fn(i).T @ q[i], atol=1e-9, rtol=1e-9)


def _route_case(t, outputs, seed, spread=3.0):
    return _rand(t, outputs, seed=seed, scale=spread).float()


@pytest.mark.parametrize("outputs, identity, top, groups, keep, scale", [(8, 2, 3, 4, 2, 2.0), (6, 3, 3, 2, 1, 1.0), (2, 1, 1, 1, 1, 1.5),
                                                                         (12, 0, 4, 3, 2, 0.5), (24, 6, 5, 3, 1, 1.75), (5, 0, 2, 1, 1, 1.0)])
def test_reference_routing_against_the_plain_rule(outputs, identity, top, groups, keep, scale) -> None:
    t, width = 37, 16
    h = _rand(t, width, seed=1)
    w = {"m.router": _rand(outputs, width, seed=2), "m.correction": _rand(outputs, seed=3, scale=0.2)}
    router = {"experts": outputs - identity, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}
    want = plain.route(h, w, "m.", router)
    rule = RouteRule(scored=True, groups=groups, keep=keep, scale=scale, identity=identity, correction=w["m.correction"].float())
    plan = refs.moe_route((h @ w["m.router"].T).float(), top, None, rule=rule)
    ids, weights = plan["ids"].view(t, top).tolist(), plan["weights"].view(t, top).tolist()
    for n in range(t):
        assert ids[n] == [e for e, _ in want[n]], n
        assert weights[n] == pytest.approx([x for _, x in want[n]], rel=1e-5)
    rows = plan["row_of"].view(t, top)
    assert ((rows < 0) == (plan["ids"].view(t, top) >= outputs - identity)).all(), "identity picks take no row"
    assert int(plan["offsets"][-1]) == int((rows >= 0).sum())


def test_groups_that_are_left_out_count_as_minus_infinity() -> None:
    """Every choice score is negative (a large negative correction): a group that is left out must not win with
    a zero in the place of its scores. And the weights come from the scores without the correction."""
    outputs, top = 6, 2
    logits = torch.tensor([[2.0, 1.0, 0.0, 3.0, 0.5, 0.1]])
    corr = torch.tensor([-5.0, -5.0, -5.0, -9.0, -9.0, -9.0])
    rule = RouteRule(scored=True, groups=2, keep=1, scale=1.0, identity=0, correction=corr)
    plan = refs.moe_route(logits, top, None, rule=rule)
    assert plan["ids"].tolist() == [0, 1], "the first group wins although output 3 has the largest score"
    s = torch.softmax(logits[0], -1)
    assert plan["weights"].tolist() == pytest.approx([float(s[0] / (s[0] + s[1])), float(s[1] / (s[0] + s[1]))], rel=1e-6)


def test_reference_combine_with_identity_picks_and_a_gate() -> None:
    t, top, h = 5, 3, 8
    x, y, shared = _rand(t, h, seed=1), _rand(t * top, h, seed=2), _rand(t, h, seed=3)
    rows = torch.tensor([0, -1, 1, 2, 3, -1, -1, -1, 4, 5, 6, 7, -1, 8, 9], dtype=torch.int32)
    weights, gate = _rand(t * top, seed=4).abs(), _rand(t, seed=5)
    plan = {"top": top, "row_of": rows, "weights": weights, "picks": t * top, "identity": 2}
    out = torch.zeros(t, h, dtype=torch.float64)
    refs.moe_combine(y, plan, shared, out, x=x, shared_gate=gate)
    for n in range(t):
        want = torch.sigmoid(gate[n]) * shared[n]
        for j in range(top):
            r = int(rows[n * top + j])
            want = want + weights[n * top + j] * (x[n] if r < 0 else y[r])
        torch.testing.assert_close(out[n], want)


def test_reference_norm_over_the_whole_projection_and_values_that_are_the_keys() -> None:
    t, heads, groups, d, page = 7, 4, 2, 8, 4
    q, k = _rand(t, heads * d, seed=1), _rand(t, groups * d, seed=2)
    qw, kw = _rand(heads * d, seed=3), _rand(groups * d, seed=4)
    pos = torch.arange(t, dtype=torch.float64)
    freq = torch.tensor([100.0 ** (-2.0 * i / 4) / 2.0 for i in range(2)], dtype=torch.float64)
    cos, sin = torch.cos(pos[:, None] * freq), torch.sin(pos[:, None] * freq)
    k_cache, v_cache = torch.zeros(3, groups, page, d, dtype=torch.float64), torch.zeros(3, groups, page, d, dtype=torch.float64)
    slots = torch.tensor([8, 9, 10, 11, 0, 1, 2], dtype=torch.int32)
    q_out = torch.zeros(t, heads, d, dtype=torch.float64)
    refs.qkv_prepare(q, k, k, qw, kw, 1e-5, cos, sin, 4, slots, k_cache, v_cache, page, heads, groups, d, d, q_out, norm_whole=True)
    want_q = plain.rotate_half(plain.rms_norm(q, qw, 1e-5).view(t, heads, d), 4, 100.0, 2.0)
    want_k = plain.rotate_half(plain.rms_norm(k, kw, 1e-5).view(t, groups, d), 4, 100.0, 2.0)
    torch.testing.assert_close(q_out, want_q)
    for n in range(t):
        s = int(slots[n])
        torch.testing.assert_close(k_cache[s // page, :, s % page], want_k[n])
        torch.testing.assert_close(v_cache[s // page, :, s % page], k[n].view(groups, d)), "the values are the keys before norm and rotation"


@pytest.mark.parametrize("sink", [-30.0, 0.0, 2.0, 40.0])
def test_reference_latent_attention_with_a_sink(sink) -> None:
    """A sink far below the scores changes nothing, one far above them takes all the weight; in between the
    weights are those of a softmax with one more term."""
    t, heads, rank, rot, page = 9, 2, 6, 2, 4
    rows = _rand(3 * page, rank + rot, seed=1)
    table = torch.tensor([[2, 0, 1]], dtype=torch.int32)
    q = _rand(t, heads, rank + rot, seed=2)
    ctx = FakeStep([t], [0])
    ctx.context_lens_dev = torch.tensor([t], dtype=torch.int32)
    out = torch.zeros(t, heads, rank, dtype=torch.float64)
    refs.latent_attention(q, rows, page, table, ctx, rank, 0.3, 0, out, sinks=torch.tensor([sink, sink]))
    keys = torch.stack([rows[int(table[0, p // page]) * page + p % page] for p in range(t)])
    for i in range(t):
        for a in range(heads):
            p = plain.softmax_with_sink((keys[: i + 1] @ q[i, a]) * 0.3, sink)
            torch.testing.assert_close(out[i, a], p @ keys[: i + 1, :rank], atol=1e-6, rtol=1e-6)
    if sink == 40.0:
        assert out.abs().max() < 1e-6
    if sink == -30.0:
        plain_out = torch.zeros_like(out)
        refs.latent_attention(q, rows, page, table, ctx, rank, 0.3, 0, plain_out)
        torch.testing.assert_close(out, plain_out, atol=1e-6, rtol=1e-6)


def test_reference_layer_scale_pending_on_the_stream() -> None:
    t, h = 5, 12
    resid, y, ls, w = _rand(t, h, seed=1).float(), _rand(t, h, seed=2).float(), _rand(h, seed=3).float(), _rand(h, seed=4).float()
    out = torch.zeros(t, h)
    want_x = resid + ls * y
    refs.post_norm_add_rms_norm(resid, y, None, ls, 0.0, False, w, False, 1e-5, out)
    torch.testing.assert_close(resid, want_x)
    torch.testing.assert_close(out, plain.rms_norm(want_x, w, 1e-5), atol=1e-5, rtol=1e-5)


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


@pytest.mark.parametrize("kind", ["attention", "latent_attention", "gla"])
@pytest.mark.parametrize("ff", [None, "dense", "moe"])
def test_each_mixer_and_each_feed_forward_alone_on_host(kind, ff, tmp_path) -> None:
    """A model of one layer: one mixer, and no feed-forward, a dense one or routed experts."""
    layer = next(copy.deepcopy(x) for x in CONFIG_B["layers"] + CONFIG_A["layers"] if x["type"] == kind)
    layer["mlp"] = None if ff is None else next(copy.deepcopy(x["mlp"]) for x in CONFIG_A["layers"] + CONFIG_B["layers"]
                                               if x["mlp"] is not None and x["mlp"]["kind"] == ff)
    cfg = {"architecture": "Diderax", "vocab": 53, "width": 40, "norm": {"eps": 1e-5}, "layers": [layer]}
    folder = write_model(tmp_path, cfg, 5)
    toks = random_prompt(33, 53, 8)
    want = plain_oracle(folder, toks)
    model = DecoderModel.from_folder(folder, torch.float32, "cpu")
    with use_references():
        for steps in (cases.whole("a", toks), cases.portions("a", toks, 2), cases.tail_decoded("a", toks, 20)):
            got, _ = run_steps(model, 4, steps, cases.max_live_tokens(steps))
            assert_rows_close(torch.stack([got["a"][p] for p in range(len(toks))]), *want, torch.float32, f"{kind}/{ff}")


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
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


def test_a_far_token_decides_the_logits_and_the_sink_matters(tmp_path) -> None:
    """A model of attention layers alone: changing the second token of a long prompt changes the last logits
    (every position stays visible), as the plain model says; and the latent layer's sink weights reach them."""
    cfg = {"architecture": "Diderax", "vocab": 50, "width": 32, "norm": {"eps": 1e-5},
           "layers": [{"type": "attention", "mlp": None, "mixer": CONFIG_A["layers"][3]["mixer"]},
                      {"type": "latent_attention", "mlp": None, "mixer": CONFIG_C["layers"][4]["mixer"]}]}
    folder = write_model(tmp_path, cfg, 3)
    model = DecoderModel.from_folder(folder, torch.float32, "cpu")
    base = random_prompt(70, 50, 1)
    changed = list(base)
    changed[1] = (base[1] + 1) % 50

    def last_logits(m, toks):
        with use_references():
            got, _ = run_steps(m, 4, cases.tail_decoded("a", toks, 20), 128)
        return got["a"][len(toks) - 1]

    ref = last_logits(model, base)
    got = last_logits(model, changed)
    assert (got - ref).abs().max() > 1e-4, "a token far back no longer reaches the last query"
    want = plain_oracle(folder, changed)
    assert_rows_close(got[None], want[0][69:], want[1][69:], torch.float32, "far token")
    model.tensors["l1.mix.sink"].add_(3.0)
    model.parts.bind(model.tensors)
    assert (last_logits(model, base) - ref).abs().max() > 1e-4, "the sink does not reach the logits"


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
    assert math.isfinite(sum(sum(x) for x in want))
