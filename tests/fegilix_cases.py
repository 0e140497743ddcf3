"""Small Fegilix configurations that differ from one another in every size and option, and helpers
shared by the host-only and the GPU tests of that architecture."""

from __future__ import annotations

import math
from pathlib import Path

import torch

SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}

# Three lanes; keys and values of different head sizes; grouped heads everywhere; a partial rotation
# with scaled frequencies; a layer that reads another layer's keys and values; 3 taps.
CONFIG_A = {
    "architecture": "Fegilix", "vocab": 89, "width": 64, "norm": {"eps": 1e-5}, "streams": 3, "logit_softcap": 20.0,
    "layers": [
        {"type": "channel_delta", "mlp": None,
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "conv": 3, "step_rank": 8, "gate_rank": 12}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2,
                   "rot": {"dims": 16, "base": 10000.0, "scaling": SCALING}}},
        {"type": "mlstm", "mlp": None, "mixer": {"heads": 3, "dim": 16, "vdim": 48, "gate_cap": 10.0}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 80},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.15, "kv_from": 1,
                   "rot": {"dims": 16, "base": 10000.0, "scaling": SCALING}}},
    ],
}

# No lanes (a plain residual stream), no soft cap, equal key and value sizes, a full unscaled
# rotation and a layer with none, one kv head, a key size that is no multiple of 32, 2 taps,
# recurrent layers with a feed-forward.
CONFIG_B = {
    "architecture": "Fegilix", "vocab": 131, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 32 ** -0.5, "rot": {"dims": 32, "base": 500.0}}},
        {"type": "mlstm", "mlp": {"kind": "dense", "ff": 64}, "mixer": {"heads": 2, "dim": 40, "vdim": 24, "gate_cap": 15.0}},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 40, "vdim": 24, "conv": 2, "step_rank": 4, "gate_rank": 4}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 72},
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 48, "scale": 0.3}},
    ],
}

# One lane with learned connections, one head everywhere, 5 taps, a key size above 32.
CONFIG_C = {
    "architecture": "Fegilix", "vocab": 61, "width": 32, "norm": {"eps": 1e-5}, "streams": 1, "logit_softcap": 8.0,
    "layers": [
        {"type": "mlstm", "mlp": None, "mixer": {"heads": 1, "dim": 48, "vdim": 16, "gate_cap": 6.0}},
        {"type": "channel_delta", "mlp": None,
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 48, "vdim": 40, "conv": 5, "step_rank": 3, "gate_rank": 5}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25, "rot": {"dims": 8, "base": 100.0}}},
    ],
}

# Sizes at which bfloat16 attention runs on the tensor cores (equal key and value sizes of 64, grouped heads),
# four lanes, two layers that read the keys and values of one earlier layer, the recurrent layers last.
ATTN_D = {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "rot": {"dims": 32, "base": 5000.0, "scaling": SCALING}}
CONFIG_D = {
    "architecture": "Fegilix", "vocab": 211, "width": 128, "norm": {"eps": 1e-5}, "streams": 4, "logit_softcap": 25.0,
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 256}, "mixer": dict(ATTN_D)},
        {"type": "attention", "mlp": None, "mixer": {**ATTN_D, "kv_from": 0}},
        {"type": "channel_delta", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 64, "conv": 4, "step_rank": 16, "gate_rank": 16}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 256}, "mixer": {**ATTN_D, "kv_from": 0}},
        {"type": "mlstm", "mlp": None, "mixer": {"heads": 2, "dim": 64, "vdim": 64, "gate_cap": 12.0}},
    ],
}

CONFIGS = {"A": (CONFIG_A, 11), "B": (CONFIG_B, 12), "C": (CONFIG_C, 13), "D": (CONFIG_D, 14)}


def write_model(folder: Path, which: str, std_scale: float = 6.0) -> Path:
    """The configuration with random weights, through the framework's random-weights mode."""
    import tinyserve_b200.architectures  # noqa: F401
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model

    cfg, seed = CONFIGS[which]
    return write_random_model(folder, config_from_dict(cfg), seed, torch.bfloat16, std_scale=std_scale)


def run_steps(model, page: int, steps, max_tokens: int, max_live: int = 4, poison: bool = True):
    """Replay a schedule; returns logits by request and position, and the replayer."""
    from tinyserve_b200.engine.replay import Replayer

    rep = Replayer(model, max_tokens, page_size=page, max_live=max_live)
    if poison:
        for g in rep.cache.groups:
            g.kv.fill_(float("nan"))        # a read outside a request's own tokens shows
        for st in rep.cache._slot_storage:
            st[-1].fill_(float("nan"))      # the pad slot belongs to nobody
    got: dict[str, dict[int, torch.Tensor]] = {}
    fed: dict[str, int] = {}
    for entries, end in steps:
        logits = rep.run_step(entries, end)
        row = 0
        for rid, toks, places in entries:
            base = fed.get(rid, 0)
            for p in places:
                got.setdefault(rid, {})[base + p] = logits[row].float().cpu().clone()
                row += 1
            fed[rid] = base + len(toks)
    rep.cache.check_invariant()
    assert all(g.allocator.num_used == 0 for g in rep.cache.groups), "pages leaked"
    assert rep.cache.state_pool.num_free == (max_live if rep.cache.has_state else 0), "state slots leaked"
    return got, rep


def relative_error(rows: torch.Tensor, want: torch.Tensor) -> float:
    """Root mean square of the difference over that of the centred oracle."""
    w = want.double() - want.double().mean(-1, keepdim=True)
    return float((rows.double() - want.double()).pow(2).mean().sqrt() / w.pow(2).mean().sqrt())


def assert_close(rows: torch.Tensor, want: torch.Tensor, dtype: torch.dtype, what: str = "") -> None:
    assert not rows.isnan().any(), f"{what}: NaN in the logits"
    err = relative_error(rows, want)
    # bfloat16: products round their inputs to 8 bits; with these wide random weights and a handful of
    # rows that alone scatters the logits by 3 to 5 % of their spread
    limit = 2e-5 if dtype == torch.float32 else 6e-2
    assert err < limit, f"{what}: relative error {err:.3g} (limit {limit})"


class _Scratch:
    def __init__(self, device) -> None:
        self.device = device

    def take(self, shape, dtype):
        return torch.full(tuple(shape), float("nan"), dtype=dtype, device=self.device)


class FakeStep:
    """The fields of a step that the recurrent references and kernels read."""

    def __init__(self, query_lens: list[int], slots: list[int], device="cpu") -> None:
        cu = [0]
        for n in query_lens:
            cu.append(cu[-1] + n)
        self.num_seqs = len(query_lens)
        self.cu_query_lens = torch.tensor(cu, dtype=torch.int32, device=device)
        self.state_slots = torch.tensor(slots, dtype=torch.int32, device=device)
        self.max_query_len = max(query_lens, default=0)
        self.query_lens = list(query_lens)
        self.arena = _Scratch(device)


def gelu_tanh(z: float) -> float:
    return 0.5 * z * (1.0 + math.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
