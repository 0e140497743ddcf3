"""Small Gasavik configurations that differ from one another in every size and option, a generator of
random ones, and helpers shared by the host-only and the GPU tests of that architecture."""

from __future__ import annotations

import random
from pathlib import Path

import torch


def _side_by_side(heads, kv_heads, dim, vdim, scale, mask, rheads, rdim, rvdim, decay, left_scale=None, right_scale=None):
    m = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale},
         "right": {"heads": rheads, "dim": rdim, "vdim": rvdim, "decay": decay}}
    if mask is not None:
        m["left"]["mask"] = mask
    if left_scale is not None:
        m["left_scale"] = left_scale
    if right_scale is not None:
        m["right_scale"] = right_scale
    return m


# A short window with kept first tokens inside one page and across pages, grouped heads, keys and values of
# different sizes, a layer without a feed-forward, 3 taps, a multiplier on the residual sum.
CONFIG_A = {
    "architecture": "Gasavik", "vocab": 97, "width": 64, "max_positions": 160, "norm": {"eps": 1e-5},
    "residual_mult": 0.7, "token_side": {"dim": 8},
    "layers": [
        {"type": "wkv", "mlp": {"kind": "dense", "ff": 80}, "mixer": {"heads": 2, "dim": 16, "decay_rank": 8}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 96},
         "mixer": _side_by_side(4, 2, 32, 16, 0.2, {"size": 9, "keep_first": 3}, 2, 16, 32, [0.5, 0.97], 0.8, 1.3)},
        {"type": "delta", "mlp": None, "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 3}},
        {"type": "parallel", "mlp": None,
         "mixer": _side_by_side(2, 1, 16, 32, 0.3, {"size": 21, "keep_first": 18}, 3, 8, 16, [0.9, 0.99, 0.3], 1.1, 0.4)},
    ],
}

# No token input, no multiplier, no scales on the two mixers, one window without kept tokens and one layer
# without a window, equal head counts, a key size that is no multiple of 32, 2 taps, equal key and value sizes.
CONFIG_B = {
    "architecture": "Gasavik", "vocab": 131, "width": 48, "max_positions": 200, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 64},
         "mixer": _side_by_side(3, 3, 16, 16, 0.25, {"size": 12}, 1, 40, 24, [0.95])},
        {"type": "delta", "mlp": {"kind": "dense", "ff": 56}, "mixer": {"heads": 2, "kv_heads": 2, "dim": 40, "vdim": 16, "conv": 2}},
        {"type": "wkv", "mlp": None, "mixer": {"heads": 3, "dim": 24, "decay_rank": 5}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 64},
         "mixer": _side_by_side(2, 1, 32, 32, 0.18, None, 2, 16, 8, [0.8, 0.6])},
    ],
}

# One head everywhere, one tap and five taps, more kept tokens than the window is wide, key sizes above 32,
# a token input as wide as one column, every layer kind twice in another order.
CONFIG_C = {
    "architecture": "Gasavik", "vocab": 61, "width": 32, "max_positions": 128, "norm": {"eps": 1e-5},
    "residual_mult": 1.5, "token_side": {"dim": 1},
    "layers": [
        {"type": "delta", "mlp": None, "mixer": {"heads": 1, "kv_heads": 1, "dim": 48, "vdim": 40, "conv": 5}},
        {"type": "delta", "mlp": {"kind": "dense", "ff": 40}, "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 1}},
        {"type": "wkv", "mlp": {"kind": "dense", "ff": 24}, "mixer": {"heads": 1, "dim": 48, "decay_rank": 3}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 40},
         "mixer": _side_by_side(1, 1, 16, 16, 0.25, {"size": 4, "keep_first": 6}, 1, 48, 40, [0.9], 2.0, 0.5)},
        {"type": "wkv", "mlp": None, "mixer": {"heads": 4, "dim": 8, "decay_rank": 16}},
        {"type": "parallel", "mlp": None,
         "mixer": _side_by_side(2, 2, 48, 8, 0.1, {"size": 1, "keep_first": 1}, 2, 8, 8, [1.0, 0.1])},
    ],
}

# Sizes at which bfloat16 attention without kept tokens runs on the tensor cores (equal key and value sizes
# of 64, grouped heads), a wide window, key sizes of 64 and 128 in the recurrent layers.
CONFIG_D = {
    "architecture": "Gasavik", "vocab": 211, "width": 128, "max_positions": 256, "norm": {"eps": 1e-5},
    "residual_mult": 0.5, "token_side": {"dim": 16},
    "layers": [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 256},
         "mixer": _side_by_side(4, 2, 64, 64, 0.125, {"size": 40, "keep_first": 0}, 2, 64, 64, [0.9, 0.99], 0.6, 0.5)},
        {"type": "wkv", "mlp": {"kind": "dense", "ff": 128}, "mixer": {"heads": 2, "dim": 64, "decay_rank": 16}},
        {"type": "delta", "mlp": None, "mixer": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 64, "conv": 4}},
        {"type": "parallel", "mlp": None,
         "mixer": _side_by_side(4, 2, 64, 64, 0.125, {"size": 33, "keep_first": 17}, 1, 128, 32, [0.97], 0.6, 0.5)},
    ],
}

CONFIGS = {"A": (CONFIG_A, 21), "B": (CONFIG_B, 22), "C": (CONFIG_C, 23), "D": (CONFIG_D, 24)}


def random_config(seed: int) -> dict:
    """A configuration with every size, constant and the layer order drawn at random."""
    rng = random.Random(seed)
    width = rng.choice([24, 40, 64, 72])
    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["parallel", "wkv", "delta"])
        if kind == "wkv":
            mixer = {"heads": rng.randint(1, 3), "dim": rng.choice([8, 16, 24, 40]), "decay_rank": rng.randint(1, 9)}
        elif kind == "delta":
            groups = rng.randint(1, 2)
            mixer = {"heads": groups * rng.randint(1, 3), "kv_heads": groups, "dim": rng.choice([8, 16, 40]),
                     "vdim": rng.choice([8, 24, 40]), "conv": rng.randint(1, 5)}
        else:
            groups, rheads = rng.randint(1, 2), rng.randint(1, 3)
            mask = None
            if rng.random() < 0.85:
                mask = {"size": rng.randint(1, 40)}
                if rng.random() < 0.8:
                    mask["keep_first"] = rng.randint(0, 24)
            mixer = _side_by_side(groups * rng.randint(1, 3), groups, rng.choice([8, 16, 24, 32]), rng.choice([8, 16, 40]),
                                  rng.uniform(0.1, 0.4), mask, rheads, rng.choice([8, 16, 40]), rng.choice([8, 16, 24]),
                                  [rng.uniform(0.2, 1.0) for _ in range(rheads)],
                                  rng.choice([None, rng.uniform(0.3, 1.5)]), rng.choice([None, rng.uniform(0.3, 1.5)]))
        mlp = {"kind": "dense", "ff": rng.choice([16, 40, 72])} if rng.random() < 0.7 else None
        layers.append({"type": kind, "mlp": mlp, "mixer": mixer})
    cfg = {"architecture": "Gasavik", "vocab": rng.randint(40, 150), "width": width, "max_positions": 96,
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.7:
        cfg["residual_mult"] = rng.uniform(0.4, 1.4)
    if rng.random() < 0.7:
        cfg["token_side"] = {"dim": rng.choice([1, 3, 8, 12])}
    return cfg


def write_model(folder: Path, which: "str | dict", seed: int | None = None, std_scale: float = 6.0) -> Path:
    """The configuration with random weights, through the framework's random-weights mode."""
    import tinyserve_b200.architectures  # noqa: F401
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model

    cfg, s = CONFIGS[which] if isinstance(which, str) else (which, seed)
    return write_random_model(folder, config_from_dict(cfg), s, torch.bfloat16, std_scale=std_scale)


def oracle(folder: Path, tokens: list[int]) -> tuple[torch.Tensor, torch.Tensor]:
    """The plain model's logits in 64-bit, and for every position how far the same plain model in
    32-bit lies from them (its conditioning: the read-out of a near-empty state divided by its own
    root mean square can lose many digits, whoever computes it)."""
    import plain_gasavik as plain

    cfg = plain.read_config(folder)
    want = plain.forward(cfg, plain.read_weights(folder, torch.float64), tokens)
    low = plain.forward(cfg, plain.read_weights(folder, torch.float32), tokens).double()
    return want.float(), row_errors(low, want)


def row_errors(rows: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: root mean square of the difference over that of the centred oracle."""
    w = want.double() - want.double().mean(-1, keepdim=True)
    return (rows.double() - want.double()).pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt()


def assert_rows_close(rows: torch.Tensor, want: torch.Tensor, cond: torch.Tensor, dtype: torch.dtype, what: str = "") -> None:
    """float32: every position within 2e-5 of the oracle's spread, a limit that grows with the position's
    conditioning. bfloat16: products round their inputs to 8 bits, which wide random weights and read-outs
    divided by their own size scatter unevenly over the positions (the same amounts whatever the schedule), so
    the positions are judged together: half of them within 5 %, nine in ten within 15 %; exactness is float32's."""
    assert not rows.isnan().any(), f"{what}: NaN in the logits"
    err = row_errors(rows, want)
    if dtype == torch.float32:
        limit = 2e-5 * torch.clamp(cond / 2e-6, min=1.0)
        worst = int((err / limit).argmax())
        assert bool((err <= limit).all()), f"{what}: position {worst}: relative error {float(err[worst]):.3g} (limit {float(limit[worst]):.3g})"
        return
    half, most = float(err.median()), float(torch.quantile(err, 0.9))
    assert half < 5e-2 and most < 0.15, f"{what}: relative error {half:.3g} at the median, {most:.3g} at nine in ten"
