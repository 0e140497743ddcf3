"""Gasavik on the GPU: every new kernel alone against its reference at sizes other than any model's,
with inputs made so that a fault shows (a key that carries all the weight just inside and just
outside the window and the kept first tokens, NaN in pages and slots that belong to nobody); the
whole model in float32 and bfloat16 against the plain implementation under every cut of the work;
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
import plain_gasavik as plain
import replay_cases as cases
from fegilix_cases import FakeStep, run_steps
from gasavik_cases import CONFIGS, assert_rows_close, oracle as plain_oracle, random_config, row_errors, write_model
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


# ------------------------------------------------------------ kernels one by one
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, hidden", [(1, 48), (37, 256), (5, 37), (130, 1024)])
def test_stream_kernels(dtype, tokens, hidden) -> None:
    from tinyserve_b200.kernels import ops

    vocab, places = 23, 50
    table, pos, nw = _rand(vocab, hidden, seed=1, dtype=dtype), _rand(places, hidden, seed=2, dtype=dtype), _rand(hidden, seed=3, dtype=dtype)
    toks = torch.randint(0, vocab, (tokens,), generator=torch.Generator().manual_seed(4)).int().cuda()
    at = torch.randint(0, places, (tokens,), generator=torch.Generator().manual_seed(5)).int().cuda()
    for norm_w in (nw, None):
        got, want = torch.empty(tokens, hidden, device="cuda"), torch.empty(tokens, hidden, device="cuda")
        ops.embed_pos_norm(toks, at, table, pos, norm_w, 1e-5, got, 1.5)
        refs.embed_pos_norm(toks, at, table, pos, norm_w, 1e-5, want, 1.5)
        torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    bad = toks.clone()
    bad[0] = vocab
    ops.embed_pos_norm(bad, at, table, pos, nw, 1e-5, got)
    assert got[0].isnan().all() and not got[1:].isnan().any()
    terms = [_rand(tokens, hidden, seed=10 + i, dtype=dtype) for i in range(4)]
    bias = _rand(hidden, seed=20, dtype=dtype)
    for n in (1, 2, 3, 4):
        for b, with_copy in ((None, False), (bias, True)):
            a, c = _rand(tokens, hidden, seed=30), _rand(tokens, hidden, seed=30)
            ca = torch.empty(tokens, hidden, dtype=dtype, device="cuda") if with_copy else None
            cc = torch.empty(tokens, hidden, dtype=dtype, device="cuda") if with_copy else None
            scales = [0.7, -1.25, 0.5, 2.0][:n]
            ops.stream_sum(a, terms[:n], scales, bias=b, bias_scale=0.3, copy=ca)
            refs.stream_sum(c, terms[:n], scales, bias=b, bias_scale=0.3, copy=cc)
            torch.testing.assert_close(a, c, atol=1e-5, rtol=1e-5)
            if with_copy:
                torch.testing.assert_close(ca.float(), cc.float(), **_tol(dtype))
    y, z = _rand(tokens, hidden, seed=40, dtype=dtype), _rand(tokens, hidden, seed=40, dtype=dtype)
    ops.add_bias(y, bias)
    refs.add_bias(z, bias)
    torch.testing.assert_close(y.float(), z.float(), **_tol(dtype))
    ops.tanh_(y)
    refs.tanh_(z)
    torch.testing.assert_close(y.float(), z.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_kernels(dtype) -> None:
    from tinyserve_b200.kernels import ops

    t, n, vocab = 19, 12, 31
    wide = _rand(t, 40, seed=1, scale=2.0, dtype=dtype)
    table = _rand(vocab, 5 * n, seed=2, dtype=dtype)
    rows = torch.randint(0, vocab, (t,), generator=torch.Generator().manual_seed(3)).int().cuda()
    for act in ("gelu_tanh", "silu"):
        a, b = torch.empty(t, n, dtype=dtype, device="cuda"), torch.empty(t, n, dtype=dtype, device="cuda")
        ops.act_mul_gather(wide[:, 7: 7 + n], rows, table, 3 * n, a, act)
        refs.act_mul_gather(wide[:, 7: 7 + n], rows, table, 3 * n, b, act)
        torch.testing.assert_close(a.float(), b.float(), **_tol(dtype))
        gu, bias = _rand(t, 2 * 36, seed=4, scale=2.0, dtype=dtype), _rand(2 * 36, seed=5, dtype=dtype)
        a, b = torch.empty(t, 36, dtype=dtype, device="cuda"), torch.empty(t, 36, dtype=dtype, device="cuda")
        ops.act_mul(gu, a, act, bias=bias)
        refs.act_mul(gu, b, act, bias=bias)
        torch.testing.assert_close(a.float(), b.float(), **_tol(dtype))
    x, w, gate = _rand(t, 3, 20, seed=6), _rand(20, seed=7, dtype=dtype), _rand(t, 60, seed=8, dtype=dtype)
    a, b = torch.empty(t, 60, dtype=dtype, device="cuda"), torch.empty(t, 60, dtype=dtype, device="cuda")
    ops.head_norm_gate(x, w, False, gate, True, 1e-5, a, gate_silu=True)
    refs.head_norm_gate(x, w, False, gate, True, 1e-5, b, gate_silu=True)
    torch.testing.assert_close(a.float(), b.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, width, per_head, gate_per_head, f32_in", [(1, 512, False, False, True), (2, 1000, True, False, True),
                                                                           (1, 4096, False, False, True), (3, 515, False, True, False)])
def test_norm_and_gate_of_wide_rows(dtype, heads, width, per_head, gate_per_head, f32_in) -> None:
    """Rows of 512 values or more (all heads normed together) take a CTA each."""
    from tinyserve_b200.kernels import ops

    t = 9
    x = _rand(t, heads, width, seed=1, dtype=torch.float32 if f32_in else dtype)
    weight = (1 + _rand(heads * width if per_head else width, seed=2, scale=0.1)).to(dtype)
    wide = _rand(t, 8 + (heads if gate_per_head else heads * width), seed=3, dtype=dtype)
    a, b = torch.empty(t, heads * width, dtype=dtype, device="cuda"), torch.empty(t, heads * width, dtype=dtype, device="cuda")
    ops.head_norm_gate(x, weight, per_head, wide[:, 8:], True, 1e-5, a, gate_per_head=gate_per_head)
    refs.head_norm_gate(x, weight, per_head, wide[:, 8:], True, 1e-5, b, gate_per_head=gate_per_head)
    torch.testing.assert_close(a.float(), b.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, inter, k", [(1, 64, 128), (3, 48, 96), (8, 512, 256), (16, 1024, 1024), (29, 96, 64), (40, 96, 64),
                                            (300, 1024, 256), (700, 2048, 512), (2048, 3072, 1024), (5, 20, 36), (260, 200, 72)])
def test_feed_forward_product_with_biases(dtype, rows, inter, k) -> None:
    """The three routes (few rows, tensor-core tiles of 128 and of 256 rows, product + activation kernel)."""
    from tinyserve_b200.kernels import ops

    x, w = _rand(rows, k, seed=1, dtype=dtype), _rand(2 * inter, k, seed=2, scale=k ** -0.5, dtype=dtype)
    bias = _rand(2 * inter, seed=3, dtype=dtype)
    a, b = torch.empty(rows, inter, dtype=dtype, device="cuda"), torch.empty(rows, inter, dtype=dtype, device="cuda")
    ops.gemm_biased_swiglu(x, w, bias, a, Arena())
    refs.gemm_biased_swiglu(x, w, bias, b)
    ops.check_device_errors()
    torch.testing.assert_close(a.float(), b.float(), **({"atol": 1e-4, "rtol": 1e-4} if dtype == torch.float32 else {"atol": 3e-2, "rtol": 3e-2}))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, d, dv", [(2, 16, 16), (3, 40, 24), (1, 48, 70), (2, 64, 32), (1, 128, 64), (2, 8, 8)])
def test_linear_scan_kernels(dtype, heads, d, dv) -> None:
    """Both forms over requests of unequal lengths (chunk edges at 16 and 8 tokens), the state in a column range of
    wider slots, slots of other requests and the pad slot full of NaN; then a second step from the state."""
    from tinyserve_b200.kernels import ops

    lens, slots = [1, 17, 16, 33, 8, 2], [4, 0, 6, 2, 5, 1]
    t, width, extra = sum(lens), heads * d * dv, 11
    for mode in ("bonus", "decay"):
        states = []
        for _ in range(2):
            st = torch.full((8, width + extra), float("nan"), device="cuda")
            st[slots] = 0.0
            states.append(st)
        for phase in range(2):
            q, k = _rand(t, heads * d + 8, seed=1 + phase, dtype=dtype), _rand(t, heads * d, seed=3 + phase, dtype=dtype)
            v = _rand(t, heads * dv, seed=5 + phase, dtype=dtype)
            w_pre, w0, u = _rand(t, heads * d, seed=7 + phase), _rand(heads * d, seed=9) - 1.0, _rand(heads * d, seed=10)
            decay = torch.linspace(0.3, 1.0, heads).cuda()
            step = FakeStep(lens, slots, device="cuda")
            outs = []
            for impl, st in zip((ops, refs), states):
                out = torch.full((t, heads, dv), float("nan"), device="cuda")
                if mode == "bonus":
                    impl.linear_scan_bonus(q[:, 8:], k, v, w_pre, w0, u, st[:, extra:], step, heads, d, dv, out)
                else:
                    impl.linear_scan_decay(q[:, 8:], k, v, decay, st[:, extra:], step, heads, d, dv, out)
                outs.append(out)
            assert not outs[0].isnan().any()
            torch.testing.assert_close(outs[0], outs[1], atol=1e-3, rtol=1e-4)
            torch.testing.assert_close(states[0][slots], states[1][slots], atol=1e-3, rtol=1e-4)
            assert states[0][[3, 7]].isnan().all() and (states[0][slots, :extra] == 0).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seg_len, scratch", [(None, None), (2, None), (5, None), (16, None), (64, None), (2, 40_000), (None, 1)])
@pytest.mark.parametrize("heads, d, dv", [(2, 16, 16), (1, 40, 70), (2, 64, 32)])
def test_linear_scan_in_segments(dtype, seg_len, scratch, heads, d, dv, monkeypatch) -> None:
    """Long portions cut into segments that run side by side, beside short ones and single tokens, against the
    token-by-token reference: the segment lengths the kernel chooses itself (portions just below and above the bound
    and a multiple of both lengths), forced short ones (edges everywhere), a scratch bound that lengthens the
    segments, and one that leaves a single segment. A decay close to 1 and one close to 0, so that what the first
    tokens wrote is still seen after the last segment, or gone at once; then a second step from the state."""
    from tinyserve_b200.kernels import ops

    if seg_len is not None:
        monkeypatch.setattr(ops, "LINEAR_SCAN_SEGMENT_TOKENS", seg_len)
        monkeypatch.setattr(ops, "LINEAR_SCAN_SEGMENT_MIN_TOKENS", 2)
    if scratch is not None:
        monkeypatch.setattr(ops, "LINEAR_SCAN_SEGMENT_SCRATCH_BYTES", scratch)
    lens, slots = ([255, 1, 257, 64, 384, 129, 2], [4, 0, 6, 2, 5, 1, 7]) if seg_len is None else ([1, 37, 2, 16, 65, 3], [4, 0, 6, 2, 5, 1])
    t, width, extra = sum(lens), heads * d * dv, 3
    for mode in ("bonus", "decay"):
        states = []
        for _ in range(2):
            st = torch.full((9, width + extra), float("nan"), device="cuda")
            st[slots] = 0.0
            states.append(st)
        for phase in range(2):
            q, k = _rand(t, heads * d, seed=1 + phase, dtype=dtype), _rand(t, heads * d, seed=3 + phase, dtype=dtype)
            v = _rand(t, heads * dv, seed=5 + phase, dtype=dtype)
            w_pre, w0, u = _rand(t, heads * d, seed=7 + phase) - 3.0, _rand(heads * d, seed=9) - 1.0, _rand(heads * d, seed=10)
            w0[: d // 2] = 2.0                                   # channels that forget at once beside ones that keep
            decay = torch.linspace(0.05, 0.9995, heads).cuda() if heads > 1 else torch.tensor([0.999]).cuda()
            step = FakeStep(lens, slots, device="cuda")
            outs = []
            for impl, st in zip((ops, refs), states):
                out = torch.full((t, heads, dv), float("nan"), device="cuda")
                if mode == "bonus":
                    impl.linear_scan_bonus(q, k, v, w_pre, w0, u, st[:, extra:], step, heads, d, dv, out)
                else:
                    impl.linear_scan_decay(q, k, v, decay, st[:, extra:], step, heads, d, dv, out)
                outs.append(out)
            ops.check_device_errors()
            assert not outs[0].isnan().any()
            scale = float(outs[1].abs().max())
            torch.testing.assert_close(outs[0], outs[1], atol=2e-5 * scale, rtol=1e-4)
            torch.testing.assert_close(states[0][slots], states[1][slots], atol=2e-5 * float(states[1][slots].abs().max()), rtol=1e-4)
            assert states[0][[3, 8]].isnan().all() and (states[0][slots, :extra] == 0).all()


def test_linear_scan_segment_choice() -> None:
    from tinyserve_b200.kernels import ops

    assert ops.linear_scan_segments(255, 1, 8, 128, 128) == (0, 1)
    assert ops.linear_scan_segments(2048, 1, 2, 128, 64) == (64, 32)
    assert ops.linear_scan_segments(2048, 8, 64, 64, 64) == (128, 16)
    seg, n = ops.linear_scan_segments(8192, 16, 64, 128, 128)       # 64 MB of states a segment: the bound allows 4
    assert n == 4 and seg % 16 == 0 and seg * n >= 8192


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channels, mixes", [(48, 5), (100, 1), (1024, 3)])
def test_token_shift_kernel(dtype, channels, mixes) -> None:
    from tinyserve_b200.kernels import ops

    lens, slots = [3, 1, 20, 1], [2, 0, 3, 1]
    t = sum(lens)
    mu = _rand(mixes, channels, seed=1, dtype=dtype)
    states = [torch.full((6, 7 + channels), float("nan"), device="cuda") for _ in range(2)]
    for st in states:
        st[slots] = 0.0
    for phase in range(3):
        x = _rand(t, channels, seed=2 + phase, dtype=dtype)
        outs = []
        for impl, st in zip((ops, refs), states):
            out = torch.full((mixes, t, channels), float("nan"), dtype=dtype, device="cuda")
            impl.token_shift_mix(x, mu, st[:, 7:], FakeStep(lens, slots, device="cuda"), out)
            outs.append(out.float())
        torch.testing.assert_close(outs[0], outs[1], **_tol(dtype))
        torch.testing.assert_close(states[0][slots], states[1][slots])
        assert states[0][[4, 5]].isnan().all()


@pytest.mark.parametrize("heads, groups, d, dv", [(4, 2, 16, 24), (2, 2, 40, 16), (1, 1, 48, 40), (6, 3, 64, 32), (2, 1, 128, 64)])
def test_delta_rule_with_one_decay_per_head_kernel(heads, groups, d, dv) -> None:
    from tinyserve_b200.kernels import ops

    lens, slots = [1, 17, 2, 40], [3, 0, 2, 1]
    t, width = sum(lens), heads * d * dv
    states = [torch.zeros(5, width + 9, device="cuda") for _ in range(2)]
    for st in states:
        st[4] = float("nan")
    for phase in range(2):
        qkv = _rand(t, 2 * groups * d + heads * dv, seed=1 + phase)
        both = _rand(t, 2 * heads, seed=3 + phase)                      # beta and step-size pre-activations side by side
        dt_bias, a_log = _rand(heads, seed=5), _rand(heads, seed=6, scale=0.3)
        outs = []
        for impl, st in zip((ops, refs), states):
            out = torch.full((t, heads, dv), float("nan"), device="cuda")
            impl.delta_scan(qkv, 0, groups * d, 2 * groups * d, both[:, heads:], dt_bias, a_log, both[:, :heads], d ** -0.5,
                            st[:, :width], FakeStep(lens, slots, device="cuda"), heads, groups, d, dv, out)
            outs.append(out)
        torch.testing.assert_close(outs[0], outs[1], atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(states[0][:4], states[1][:4], atol=1e-4, rtol=1e-4)


def _tables(lens: list[int], page: int, seed: int):
    need = [-(-n // page) for n in lens]
    order = torch.randperm(sum(need) + 3, generator=torch.Generator().manual_seed(seed)).tolist()
    tables, at = [], 0
    for n in need:
        tables.append(order[at: at + n])
        at += n
    table = torch.zeros(len(lens), max(need), dtype=torch.int32)
    for b, pages in enumerate(tables):
        table[b, : len(pages)] = torch.tensor(pages)
    return tables, table.cuda(), sum(need) + 3


def _kept_case(dtype, heads, groups, d, dv, page, lens, news, window, keep, far=None):
    """Keys and values written through qkv_prepare (with biases), then attention over a window that keeps the first
    tokens, by the kernels and by the references. ``far``: the position of request 0 whose key is made to carry all
    the weight for that request's last query."""
    from tinyserve_b200.kernels import ops

    tables, table, pages = _tables(lens, page, 7)
    caches = [(torch.full((pages, groups, page, d), float("nan"), dtype=dtype, device="cuda"),
               torch.full((pages, groups, page, dv), float("nan"), dtype=dtype, device="cuda")) for _ in range(2)]
    biases = [_rand(heads * d, seed=40, scale=0.1, dtype=dtype), _rand(groups * d, seed=41, scale=0.1, dtype=dtype),
              _rand(groups * dv, seed=42, scale=0.1, dtype=dtype)]
    res = None
    for phase, counts in enumerate(([n - m for n, m in zip(lens, news)], news)):
        starts = [0] * len(lens) if phase == 0 else [n - m for n, m in zip(lens, news)]
        live = [b for b, c in enumerate(counts) if c > 0]
        if not live:
            continue
        pos = torch.cat([torch.arange(starts[b], starts[b] + counts[b]) for b in live])
        t = len(pos)
        slots = torch.cat([torch.tensor([tables[b][p // page] * page + p % page for p in range(starts[b], starts[b] + counts[b])])
                           for b in live]).int().cuda()
        q, k, v = (_rand(t, heads * d, seed=10 + phase, scale=0.3, dtype=dtype), _rand(t, groups * d, seed=20 + phase, scale=0.3, dtype=dtype),
                   _rand(t, groups * dv, seed=30 + phase, dtype=dtype))
        if far is not None and live[0] == 0:
            if starts[0] <= far < starts[0] + counts[0]:
                k[far - starts[0]] = 4.0
            if phase == 1:
                q[counts[0] - 1] = 4.0
        ctx = Ctx([counts[b] for b in live], [starts[b] + counts[b] for b in live])
        tb = table[torch.tensor(live, device="cuda")].contiguous()
        res = []
        for impl, (kc, vc) in zip((ops, refs), caches):
            qo = torch.empty(t, heads, d, dtype=dtype, device="cuda")
            impl.qkv_prepare(q, k, v, None, None, 0.0, None, None, 0, slots, kc, vc, page, heads, groups, d, dv, qo,
                             q_bias=biases[0], k_bias=biases[1], v_bias=biases[2])
            out = torch.empty(t, heads * dv, dtype=dtype, device="cuda")
            impl.paged_attention(qo, kc, vc, page, tb, ctx, 1.0, window, out, keep_first=keep)
            res.append(out.float())
        res += [v, counts, starts, biases[2]]
    return res


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, groups, d, dv, page, window, keep", [
    (4, 2, 32, 16, 4, 7, 3), (8, 1, 48, 48, 16, 96, 20), (4, 2, 64, 64, 16, 40, 17), (2, 2, 24, 40, 8, 19, 30), (6, 3, 96, 48, 16, 33, 1),
    (4, 4, 64, 64, 16, 1, 1), (3, 1, 16, 16, 8, 5, 64), (4, 1, 128, 128, 16, 100, 130), (8, 2, 128, 128, 32, 200, 5),
    (6, 3, 64, 64, 8, 60, 129), (2, 1, 128, 128, 16, 128, 128)])
def test_attention_that_keeps_the_first_tokens_kernels(dtype, heads, groups, d, dv, page, window, keep) -> None:
    lens, news = [page * 3 + 1, 170, page * 2, 33, 1, 400], [1, 17, 1, 33, 1, 130]
    got, want, *_ = _kept_case(dtype, heads, groups, d, dv, page, lens, news, window, keep)
    assert not got.isnan().any()
    torch.testing.assert_close(got, want, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("new", [1, 2, 70])
@pytest.mark.parametrize("window, keep, page, d", [(16, 5, 16, 32), (33, 16, 16, 64), (40, 17, 8, 128), (7, 40, 4, 32), (100, 140, 16, 64)])
def test_edges_of_the_window_and_of_the_kept_tokens(dtype, new, window, keep, page, d) -> None:
    """The last query of a long request points at one key: it takes that key's value exactly when the key is
    inside the window or among the kept first tokens; keys in prompts and among the step's own tokens. Head
    sizes of 64 and 128 in bfloat16 run the prompt's rows on the tensor cores."""
    heads, groups, total = 4, 2, 300
    last = total - 1
    for far in (0, keep - 1, keep, keep + 1, last - window, last - window + 1, last - 1, last):
        if not 0 <= far <= last:
            continue
        got, want, v, counts, starts, v_bias = _kept_case(dtype, heads, groups, d, d, page, [total, 40], [new, 1], window, keep, far=far)
        torch.testing.assert_close(got, want, **_tol(dtype))
        seen = plain.visible(last, far, window, keep)
        out = got[counts[0] - 1].view(heads, d)
        if far >= starts[0]:                                   # the key is among this step's tokens: its value is at hand
            value = (v[far - starts[0]].float() + v_bias.float()).view(groups, d)
            close = all((out[h] - value[h // 2]).abs().max() < 5e-2 for h in range(heads))
            assert close == seen, f"key {far}, query {last}: seen {close}, the mask says {seen}"


# ------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {k: write_model(tmp_path_factory.mktemp("gasavik" + k), k) for k in CONFIGS}


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
    """Sizes, head counts, windows, kept tokens, taps, layer order and constants drawn at random; a prompt alone,
    decoded token by token, in portions, and mixed with others, in both types."""
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
def test_long_prompts_whose_scans_run_in_segments(dtype, tmp_path) -> None:
    """Prompts of several hundred tokens: the linear scans of a long portion run in segments. Whole, in long and
    short portions (one just above the bound), decoded at the end, and mixed with a short request."""
    import copy

    from tinyserve_b200.kernels import ops
    from tinyserve_b200.model import DecoderModel

    cfg = copy.deepcopy(CONFIGS["D"][0])
    cfg["max_positions"] = 720
    folder = write_model(tmp_path, cfg, 31)
    reqs = {"long": random_prompt(700, cfg["vocab"], 41), "mid": random_prompt(300, cfg["vocab"], 42), "short": random_prompt(9, cfg["vocab"], 43)}
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
def test_long_decoding_past_the_windows(folders, dtype, which) -> None:
    from tinyserve_b200.model import DecoderModel

    vocab = plain.read_config(folders[which])["vocab"]
    toks = random_prompt(150, vocab, 9)
    want = plain_oracle(folders[which], toks)
    model = DecoderModel.from_folder(folders[which], dtype, "cuda")
    got, _ = run_steps(model, 16, cases.tail_decoded("a", toks, 145), 192)
    rows = torch.stack([got["a"][p] for p in range(150)])
    assert_rows_close(rows, *want, dtype, "all tokens")


def test_a_far_kept_token_decides_the_logits(folders) -> None:
    """Changing one of the kept first tokens changes the logits far beyond the window; changing the token just
    after the kept ones changes them only through the recurrent layers. A model of attention layers alone shows
    the difference exactly."""
    from tinyserve_b200.model import DecoderModel

    mixer = {"left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 6, "keep_first": 2}},
             "right": {"heads": 1, "dim": 8, "vdim": 8, "decay": [0.0]}, "left_scale": 1.0, "right_scale": 1.0}
    cfg = {"architecture": "Gasavik", "vocab": 50, "width": 32, "max_positions": 64, "norm": {"eps": 1e-5},
           "layers": [{"type": "parallel", "mlp": None, "mixer": mixer}]}
    folder = write_model(folders["A"].parent / "kept_only", cfg, 3)
    model = DecoderModel.from_folder(folder, torch.float32, "cuda")
    base = random_prompt(40, 50, 1)

    def last_logits(toks):
        got, _ = run_steps(model, 4, cases.tail_decoded("a", toks, 20), 64)
        return got["a"][39]

    ref = last_logits(base)
    kept, dropped = list(base), list(base)
    kept[1], dropped[2] = (base[1] + 1) % 50, (base[2] + 1) % 50
    assert (last_logits(kept) - ref).abs().max() > 1e-3, "a kept first token no longer reaches the last query"
    assert (last_logits(dropped) - ref).abs().max() < 1e-6, "a token behind the window and after the kept ones is still seen"
    want = plain_oracle(folder, kept)
    assert_rows_close(last_logits(kept)[None], want[0][39:], want[1][39:], torch.float32, "kept")


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
