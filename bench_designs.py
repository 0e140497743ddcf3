"""``python bench.py --designs [--design fegilix|guzovik|gasavik|diderax] [--design-beside qwen3|guzovik|...]``:
prefill and decode throughput of a design at layer sizes that resemble a real model's (random weights), beside
the dense Qwen3 decoder (or, with ``--design-beside``, another design of the framework), with the same width,
attention heads, (active) feed-forward size and number of layers; and where each design's step time goes, kernel class by kernel class, with the
share of the measured peaks each class reaches. The default workload of ``bench.py`` does not come
through here.

The Fegilix layers follow the pattern mLSTM, mLSTM, attention + feed-forward, delta rule, mLSTM,
attention on the third layer's keys and values + feed-forward, with two hyper-connection lanes.
"""

from __future__ import annotations

import json
import statistics

from bench import PAGE, Bench, peaks

SIZES = {
    # width, attention heads, kv heads, head size, feed-forward, recurrent heads
    "1k": dict(width=1024, heads=16, kv_heads=8, dim=128, ff=3072, rec_heads=8, experts=16),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, rec_heads=32, experts=32),
}
VOCAB = 32768
LAYERS = 6


def fegilix_config(s: dict) -> dict:
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
            "rot": {"dims": s["dim"], "base": 1e6}}
    mlp = {"kind": "dense", "ff": s["ff"]}
    mlstm = {"type": "mlstm", "mlp": None, "mixer": {"heads": s["rec_heads"], "dim": s["dim"], "vdim": s["dim"], "gate_cap": 15.0}}
    delta = {"type": "channel_delta", "mlp": None,
             "mixer": {"heads": s["rec_heads"], "kv_heads": max(1, s["rec_heads"] // 2), "dim": s["dim"], "vdim": s["dim"],
                       "conv": 4, "step_rank": 64, "gate_rank": 64}}
    return {"architecture": "Fegilix", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5}, "streams": 2,
            "logit_softcap": 30.0, "max_positions": 8192,
            "layers": [mlstm, mlstm, {"type": "attention", "mlp": mlp, "mixer": attn}, delta, mlstm,
                       {"type": "attention", "mlp": mlp, "mixer": {**attn, "kv_from": 2}}]}


def qwen3_config(s: dict) -> dict:
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": VOCAB, "hidden_size": s["width"],
            "intermediate_size": s["ff"], "num_hidden_layers": LAYERS, "num_attention_heads": s["heads"],
            "num_key_value_heads": s["kv_heads"], "head_dim": s["dim"], "hidden_act": "silu", "rms_norm_eps": 1e-6,
            "rope_theta": 1e6, "max_position_embeddings": 8192, "tie_word_embeddings": False}


def guzovik_config(s: dict) -> dict:
    """Windowed attention + clamped feed-forward, latent attention + routed experts, windowed attention +
    routed experts, that layer again on the same tensors, a second latent layer, and the shared layer once
    more. Three experts of a third of the dense feed-forward's size are used per token beside a shared one of
    that size, so a token's feed-forward work equals the dense model's; latents of 512 + 64 as in large
    models of this kind."""
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
            "mask": {"size": 512}}
    latent = {"heads": s["heads"], "dim": s["dim"], "rot_dim": 64, "vdim": s["dim"], "kv_rank": 512,
              "scale": (s["dim"] + 64) ** -0.5, "mask": {"size": 1024}, "rot": {"dims": 64, "base": 1e6}}
    ff = s["ff"] // 4
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": 3}, "expert": {"ff": ff}, "shared": {"ff": ff}}
    dense = {"kind": "dense", "ff": s["ff"], "limit": 7.0}
    shared_layer = {"type": "attention", "mlp": moe, "mixer": attn, "weights_of": 2}
    return {"architecture": "Guzovik", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "max_positions": 8192,
            "layers": [{"type": "attention", "mlp": dense, "mixer": attn}, {"type": "latent_attention", "mlp": moe, "mixer": latent},
                       {"type": "attention", "mlp": moe, "mixer": attn}, shared_layer,
                       {"type": "latent_attention", "mlp": moe, "mixer": latent}, dict(shared_layer)]}


def gasavik_config(s: dict) -> dict:
    """Windowed attention that keeps the first tokens beside decayed linear attention, time mixing twice, the
    gated delta rule, the pair again, time mixing; every layer with the dense model's feed-forward beside its
    mixer and a token input of 256 columns behind it. Time mixing with heads of 64 that fill the width."""
    pair = {"left": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
                     "mask": {"size": 512, "keep_first": 16}},
            "right": {"heads": s["rec_heads"], "dim": s["dim"], "vdim": s["dim"],
                      "decay": [1.0 - 2.0 ** -(2 + 6 * i / max(1, s["rec_heads"] - 1)) for i in range(s["rec_heads"])]},
            "left_scale": 0.6, "right_scale": 0.5}
    mlp = {"kind": "dense", "ff": s["ff"]}
    wkv = {"type": "wkv", "mlp": mlp, "mixer": {"heads": s["width"] // 64, "dim": 64, "decay_rank": 64}}
    delta = {"type": "delta", "mlp": mlp, "mixer": {"heads": s["rec_heads"], "kv_heads": max(1, s["rec_heads"] // 2), "dim": s["dim"],
                                                     "vdim": s["dim"], "conv": 4}}
    par = {"type": "parallel", "mlp": mlp, "mixer": pair}
    return {"architecture": "Gasavik", "vocab": VOCAB, "width": s["width"], "max_positions": 8192, "norm": {"eps": 1e-6},
            "residual_mult": 0.5, "token_side": {"dim": 256}, "layers": [par, wkv, wkv, delta, par, wkv]}


def diderax_config(s: dict) -> dict:
    """Attention whose values are the keys + biased feed-forward, gated linear attention + routed experts, gated
    linear attention + feed-forward, latent attention with a query latent + routed experts, attention + feed-forward,
    gated linear attention + routed experts. Three of the router's outputs are used per token (experts of a quarter
    of the dense feed-forward's size, or one of four identity experts) beside a gated shared expert of that size;
    latents of 512 + 64 for keys and values and of three eighths of the width for the queries; linear-attention
    heads of 128 that fill the width."""
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
            "rot": {"dims": s["dim"] // 2, "base": 5e5, "scaling": {"factor": 4.0}}}
    latent = {"heads": s["heads"], "dim": s["dim"], "rot_dim": 64, "vdim": s["dim"], "kv_rank": 512, "q_rank": 3 * s["width"] // 8,
              "scale": (s["dim"] + 64) ** -0.5, "rot": {"dims": 64, "base": 5e5}}
    gla = {"heads": s["rec_heads"], "dim": s["dim"], "vdim": s["dim"], "tau": 8.0, "decay_rank": 64}
    ff = s["ff"] // 4
    moe = {"kind": "moe", "router": {"experts": s["experts"], "identity": 4, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}},
           "expert": {"ff": ff}, "shared": {"ff": ff}}
    dense = {"kind": "dense", "ff": s["ff"]}
    return {"architecture": "Diderax", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-6}, "max_positions": 8192,
            "layers": [{"type": "attention", "mlp": dense, "mixer": attn}, {"type": "gla", "mlp": moe, "mixer": gla},
                       {"type": "gla", "mlp": dense, "mixer": gla}, {"type": "latent_attention", "mlp": moe, "mixer": latent},
                       {"type": "attention", "mlp": dense, "mixer": attn}, {"type": "gla", "mlp": moe, "mixer": gla}]}


DESIGNS = {"fegilix": fegilix_config, "guzovik": guzovik_config, "gasavik": gasavik_config, "diderax": diderax_config}
NEW_OPS = ["post_norm_add_rms_norm", "latent_prepare", "latent_attention", "bmm", "transpose01", "moe_route_from", "moe_route", "moe_gemm",
           "moe_combine", "gemm_gated", "hc_mix_norm", "hc_collapse", "act_mul", "softcap", "head_norm_gate", "mlstm_scan", "delta_scan",
           "causal_conv_silu", "qkv_prepare", "linear_scan_bonus", "linear_scan_decay", "token_shift_mix", "embed_pos_norm",
           "stream_sum", "add_bias", "tanh_", "act_mul_gather", "gemm_biased_swiglu", "linear_scan_gated", "rms_norm_rows"]
OLD_OPS = ["embed", "add_rms_norm", "rope_tables", "silu_mul", "qk_norm_rope_write", "paged_attention",
           "decode_attention_fused", "gemm", "gemm_swiglu", "gemm_to_stream", "gemm_normed", "sample"]


class DesignBench(Bench):
    def __init__(self, cfg_dict: dict, graphs: bool = True) -> None:
        import torch

        from tinyserve_b200.config import config_from_dict
        from tinyserve_b200.model import DecoderModel

        self.torch, self.name = torch, cfg_dict.get("architecture") or cfg_dict["architectures"][0]
        self.cfg = config_from_dict(cfg_dict)
        self.dev = torch.device("cuda:0")
        torch.cuda.set_device(self.dev)
        self.model = DecoderModel.from_config(self.cfg, seed=0, dtype=torch.bfloat16, device=self.dev)
        self.graphs = graphs
        self.gen = torch.Generator().manual_seed(0)
        self.check_rel, self.checks = 0.0, 0

    def kv_bytes_per_token(self) -> int:
        return max(super().kv_bytes_per_token(), 1)

    def prefill_ms(self, tokens: int) -> float:
        from tinyserve_b200.engine.step import StepEntry

        torch = self.torch
        e = self.new_engine(1, tokens + 8)
        toks = self.prompts([tokens])[0]
        times = []
        for it in range(3 + 5):
            req = e.cache.new_request()
            e.cache.append(req, tokens)
            torch.cuda.synchronize()
            s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_.record()
            e.runner.step([StepEntry(req, toks)])
            e_.record()
            torch.cuda.synchronize()
            e.cache.free(req)
            if it >= 3:
                times.append(s_.elapsed_time(e_))
        return statistics.median(times)

    def op_table(self, batch: int, prompt_len: int, pk: dict, prefill_tokens: int = 0) -> dict:
        """Device time of a step by ``ops`` function (event pairs around every call, the step queued
        behind a spin kernel, launch overlap off; median of three steps), with the bytes a call must
        move and its multiply-adds where they are what bounds it."""
        from tinyserve_b200.engine.step import StepEntry
        from tinyserve_b200.kernels import ops

        torch = self.torch
        saved, self.graphs = self.graphs, False
        if prefill_tokens:
            e = self.new_engine(1, prefill_tokens + 8, run_ahead=False)
            prompt, reqs = self.prompts([prefill_tokens])[0], []
        else:
            e = self.prefilled(batch, prompt_len, 16, run_ahead=False)
            reqs = list(e.requests.values())
        self.graphs = saved
        e.runner.tune_launch_overlap = False
        ops.set_programmatic_launch(0)
        records: list = []

        def nbytes(*ts) -> float:
            return float(sum(t.numel() * t.element_size() for t in ts if isinstance(t, torch.Tensor)))

        def seen(ctx, window: int) -> float:
            """(query, key) pairs of a step under a causal mask and a window (0: none)."""
            total = 0.0
            for n, c in zip(ctx.query_lens, ctx.context_lens):
                for p in range(c - n, c):
                    total += min(p + 1, window) if window else p + 1
            return total

        def work(name: str, a: tuple, k: dict) -> tuple[float, float]:
            """(bytes, flops) of one call."""
            if name in ("gemm", "gemm_swiglu", "gemm_to_stream", "gemm_gated"):
                return nbytes(a[0], a[1], a[2]), 2.0 * a[0].shape[0] * a[1].shape[0] * a[1].shape[1]
            if name == "gemm_biased_swiglu":      # x, the gate and up rows, the biases, the result
                return nbytes(a[0], a[1], a[2], a[3]), 2.0 * a[0].shape[0] * a[1].shape[0] * a[1].shape[1]
            if name == "bmm":
                return nbytes(a[0], a[1], a[2]), 2.0 * a[0].shape[0] * a[0].shape[1] * a[0].shape[2] * a[1].shape[2]
            if name == "moe_gemm":            # the matrices of the experts that have rows, the rows in and out
                plan, used = a[3], min(a[3]["experts"], a[3]["picks"])
                return (used * a[1][0].numel() * a[1].element_size() + nbytes(a[2]) + plan["picks"] * a[1].shape[2] * 2.0,
                        2.0 * plan["picks"] * a[1].shape[1] * a[1].shape[2])
            if name == "moe_combine":
                return nbytes(a[0], a[2], a[3]), 0.0
            if name == "moe_route":
                return nbytes(a[0]) * 3.0, 0.0
            if name == "moe_route_from":
                return nbytes(a[0], a[1]), 2.0 * a[0].shape[0] * a[1].shape[0] * a[1].shape[1]
            if name == "post_norm_add_rms_norm":      # the stream read and written, the pending output, the result
                return 2.0 * nbytes(a[0]) + nbytes(a[1], a[9]), 0.0
            if name == "latent_prepare":
                return nbytes(a[1], a[2]) + 2.0 * nbytes(a[15]), 0.0
            if name == "latent_attention":    # every request's visible rows once (all heads share them)
                ctx, rank, window, d = a[4], a[5], a[7], a[0].shape[2]
                rows = sum(min(c, (window or c) + n - 1) for n, c in zip(ctx.query_lens, ctx.context_lens))
                return rows * d * a[1].element_size() + nbytes(a[0], a[8]), 2.0 * a[0].shape[1] * (d + rank) * seen(ctx, window)
            if name == "transpose01":
                return nbytes(a[0], a[1]), 0.0
            if name == "gemm_normed":
                return nbytes(a[0], a[4], a[5]), 2.0 * a[0].shape[0] * a[4].shape[0] * a[4].shape[1]
            if name in ("paged_attention", "decode_attention_fused"):
                kc, vc = (a[1], a[2]) if name == "paged_attention" else (a[7], a[8])
                ctx = a[5] if name == "paged_attention" else a[11]
                heads = a[0].shape[1] if name == "paged_attention" else a[14]
                window = a[7] if name == "paged_attention" else 0
                rows = sum(min(c, (window or c) + n - 1) for n, c in zip(ctx.query_lens, ctx.context_lens))
                return (float(rows) * kc.shape[1] * (kc.shape[3] + vc.shape[3]) * kc.element_size(),
                        2.0 * heads * (kc.shape[3] + vc.shape[3]) * seen(ctx, window))
            if name == "qk_norm_rope_write":
                return 2.0 * nbytes(a[0]), 0.0
            if name == "qkv_prepare":         # q, k and v rows read and written
                return 2.0 * nbytes(a[0], a[1], a[2]), 0.0
            if name == "embed":
                return nbytes(a[0], a[2]) + a[0].numel() * a[1].shape[1] * a[1].element_size(), 0.0
            if name == "mlstm_scan":          # state in and out, the rows read, the read-out written; 6 flops per state element and token
                ctx, heads, d, dv = a[9], a[10], a[11], a[12]
                return (2.0 * ctx.num_seqs * heads * d * dv * 4 + nbytes(a[0], a[4], a[13]), 6.0 * a[0].shape[0] * heads * d * dv)
            if name == "delta_scan":          # 8 flops per state element and token
                ctx, heads, d, dv = a[10], a[11], a[13], a[14]
                return (2.0 * ctx.num_seqs * heads * d * dv * 4 + nbytes(a[0], a[4], a[7], a[15]), 8.0 * a[0].shape[0] * heads * d * dv)
            if name == "causal_conv_silu":
                return nbytes(a[0], a[4]), 0.0
            if name == "linear_scan_bonus":   # state in and out, r, k, v and the decays read, the read-out written; 6 flops per state element and token
                ctx, heads, d, dv = a[7], a[8], a[9], a[10]
                return (2.0 * ctx.num_seqs * heads * d * dv * 4 + nbytes(a[0], a[1], a[2], a[3], a[11]), 6.0 * a[0].shape[0] * heads * d * dv)
            if name == "linear_scan_decay":   # 4 flops per state element and token
                ctx, heads, d, dv = a[5], a[6], a[7], a[8]
                return (2.0 * ctx.num_seqs * heads * d * dv * 4 + nbytes(a[0], a[1], a[2], a[9]), 4.0 * a[0].shape[0] * heads * d * dv)
            if name == "linear_scan_gated":   # state in and out, q, k, v and the decays' pre-activations read, the read-out written; 4 flops per state element and token
                ctx, heads, d, dv = a[8], a[9], a[10], a[11]
                return (2.0 * ctx.num_seqs * heads * d * dv * 4 + nbytes(a[0], a[1], a[2], a[3], a[12]), 4.0 * a[0].shape[0] * heads * d * dv)
            if name == "rms_norm_rows":
                return 2.0 * nbytes(a[3]), 0.0
            if name == "token_shift_mix":
                return nbytes(a[0], a[4]), 0.0
            if name == "stream_sum":          # the stream read and written, every term read, the copy written
                return 2.0 * nbytes(a[0]) + nbytes(*a[1]) + nbytes(k.get("copy")), 0.0
            if name == "embed_pos_norm":
                return nbytes(a[6]) * (1.0 + 2.0 * a[2].element_size() / 4.0), 0.0
            if name == "act_mul_gather":
                return nbytes(a[0], a[4]) * 1.5, 0.0
            if name in ("add_bias", "tanh_"):
                return 2.0 * nbytes(a[0]), 0.0
            if name == "hc_mix_norm":         # the lanes read and written, the pending output, the result
                return 2.0 * nbytes(a[0]) + nbytes(a[2], a[8]), 0.0
            if name == "hc_collapse":
                return nbytes(a[6]) * (a[0].shape[0] + 1), 0.0
            if name == "head_norm_gate":
                return nbytes(a[0], a[6]) * 1.5, 0.0
            if name == "softcap":
                return 2.0 * nbytes(a[0]), 0.0
            return nbytes(*a), 0.0

        names = OLD_OPS + NEW_OPS
        originals = {n: getattr(ops, n) for n in names}
        depth = [0]

        def wrap(name: str):
            fn = originals[name]

            def timed(*a, **k):
                if depth[0]:
                    return fn(*a, **k)
                s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s_.record()
                depth[0] += 1
                try:
                    r = fn(*a, **k)
                finally:
                    depth[0] -= 1
                e_.record()
                records.append((name, s_, e_, *work(name, a, k)))
                return r
            return timed

        for n in names:
            setattr(ops, n, wrap(n))
        out = torch.empty(max(batch, 1), dtype=torch.int32, device=self.dev)
        rounds = []
        try:
            for it in range(5):
                records.clear()
                entries = []
                if prefill_tokens:
                    req = e.cache.new_request()
                    e.cache.append(req, prefill_tokens)
                    entries.append(StepEntry(req, prompt))
                for r in reqs:
                    e.cache.append(r.cache, 1)
                    entries.append(StepEntry(r.cache, [r.output[-1]]))
                torch.cuda._sleep(40_000_000 if not prefill_tokens else 150_000_000)
                ops.sample(e.runner.step(entries), out[: len(entries)])
                torch.cuda.synchronize()
                if prefill_tokens:
                    e.cache.free(req)
                if it >= 2:
                    acc: dict = {}
                    for name, s_, e_, by, fl in records:
                        a = acc.setdefault(name, [0.0, 0.0, 0.0, 0.0])
                        a[0] += s_.elapsed_time(e_)
                        a[1] += by
                        a[2] += 1
                        a[3] += fl
                    rounds.append(acc)
        finally:
            for n in names:
                setattr(ops, n, originals[n])
            ops.set_programmatic_launch(ops.DEFAULT_PDL_MASK)
        for r in reqs:
            e.cache.free(r.cache)
        table = {}
        for name in rounds[0]:
            ms = statistics.median(r[name][0] for r in rounds)
            _, by, calls, fl = rounds[0][name]
            row = {"calls": int(calls), "ms": round(ms, 4), "hbm_frac": round(by / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)}
            if fl:
                row["tflops"] = round(fl / (ms * 1e-3) / 1e12, 2)
            table[name] = row
        return table


def run(args) -> int:
    import torch

    pk, pk_src = peaks()
    tokens, batch, ctx = 2048, 8, 1024
    design, beside = getattr(args, "design", "fegilix"), getattr(args, "design_beside", "qwen3")
    beside_config = qwen3_config if beside == "qwen3" else DESIGNS[beside]
    result = {"metric": f"prefill and decode tok/s of {design.capitalize()} beside {beside.capitalize()} at equal layer sizes (6 layers, bf16, random weights)",
              "peaks": {**{k: pk[k] for k in ("hbm_gbs", "bf16_tflops")}, "source": pk_src},
              "workload": {"prefill_tokens": tokens, "decode_batch": batch, "decode_context": ctx, "page_size": PAGE}, "sizes": {}}
    for size in (args.design_sizes.split(",") if args.design_sizes else list(SIZES)):
        s = SIZES[size]
        entry = {}
        for label, cfg in ((design, DESIGNS[design](s)), (beside, beside_config(s))):
            b = DesignBench(cfg)
            pre = b.prefill_ms(tokens)
            dec, _, launches = b.device_decode(batch, ctx, max(args.warmup, 3), args.steps, check=False)
            row = {"prefill_ms": round(pre, 3), "prefill_tok_s": round(tokens / pre * 1e3), "decode_ms_per_step": round(dec, 4),
                   "decode_tok_s": round(batch / dec * 1e3), "kernels_per_decode_step": launches // args.steps,
                   "weight_mb": round(b.model.weight_bytes() / 2 ** 20, 1)}
            if args.kernels:
                row["prefill_by_op"] = b.op_table(0, 0, pk, prefill_tokens=tokens)
                row["decode_by_op"] = b.op_table(batch, ctx, pk)
            entry[label] = row
            b.close()
            torch.cuda.empty_cache()
        result["sizes"][size] = entry
    print(json.dumps(result))
    return 0
