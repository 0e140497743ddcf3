"""Small Diderax configurations that differ from one another in every size and option, a generator of
random ones, and helpers shared by the host-only and the GPU tests of that architecture."""

from __future__ import annotations

import random
from pathlib import Path

import torch

from gasavik_cases import assert_rows_close as _assert_rows_close, row_errors


def attention(heads, kv_heads, dim, scale, dims, base, factor=None):
    rot = {"dims": dims, "base": base}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, dims, base, factor=None):
    rot = {"dims": dims, "base": base}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "rot": rot}


def gla(heads, dim, vdim, tau, decay_rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": decay_rank}


def moe(experts, top, ff, identity=None, groups=None, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    out = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def dense(ff):
    return {"kind": "dense", "ff": ff}


# Grouped heads, partial rotation with scaled frequencies, a linear-attention layer with unequal key and value
# sizes, routed experts with identity experts in four groups of which two are kept, a layer without a feed-forward,
# routed experts without groups, identity experts or a shared expert.
CONFIG_A = {
    "architecture": "Diderax", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "gla", "mixer": gla(2, 16, 24, 4.0, 6), "mlp": moe(6, 3, 24, identity=2, groups=(4, 2), scale=2.0, shared=40)},
        {"type": "attention", "mixer": attention(4, 2, 32, 0.2, 8, 1e4, 4.0), "mlp": dense(80)},
        {"type": "latent_attention", "mixer": latent(3, 16, 8, 24, 32, 20, 0.2, 8, 1e3), "mlp": None},
        {"type": "attention", "mixer": attention(2, 1, 16, 0.3, 16, 5e4), "mlp": moe(5, 2, 16)},
    ],
}

# The latent attention first, with a rotation of part of the rotated key part and scaled frequencies; a key size
# that is no multiple of 16; as many key/value heads as query heads; as many identity experts as real ones in two
# groups of which one is kept; all groups kept; a scale on the weights below one.
CONFIG_B = {
    "architecture": "Diderax", "vocab": 131, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": latent(2, 8, 8, 16, 24, 40, 0.25, 4, 1e4, 2.0), "mlp": moe(3, 3, 24, identity=3, groups=(2, 1), shared=16)},
        {"type": "gla", "mixer": gla(1, 40, 16, 16.0, 3), "mlp": dense(56)},
        {"type": "attention", "mixer": attention(3, 3, 16, 0.25, 4, 300000.0, 6.0), "mlp": moe(6, 2, 8, groups=(3, 3), scale=0.5, shared=24)},
        {"type": "gla", "mixer": gla(3, 8, 8, 1.0, 12), "mlp": None},
    ],
}

# One head everywhere, one expert of which one is used beside one identity expert, head sizes above 32 that
# differ between keys and values, every layer kind twice in another order, a large tau and a tau below one.
CONFIG_C = {
    "architecture": "Diderax", "vocab": 61, "width": 32, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": attention(1, 1, 48, 0.15, 2, 100.0), "mlp": None},
        {"type": "latent_attention", "mixer": latent(1, 40, 16, 48, 16, 8, 0.1, 16, 1e4), "mlp": moe(1, 1, 24, identity=1, scale=1.5, shared=8)},
        {"type": "gla", "mixer": gla(1, 48, 40, 64.0, 1), "mlp": dense(24)},
        {"type": "gla", "mixer": gla(4, 8, 8, 0.5, 5), "mlp": moe(4, 4, 8, groups=(2, 2))},
        {"type": "latent_attention", "mixer": latent(4, 8, 4, 8, 8, 16, 0.3, 2, 50.0, 3.0), "mlp": dense(40)},
        {"type": "attention", "mixer": attention(2, 2, 8, 0.35, 8, 1e6, 1.0), "mlp": dense(16)},
    ],
}

# Sizes at which the bfloat16 kernels run on the tensor cores: attention heads of 64 and of 128, a latent of 64
# with a rotated part of 32, linear attention with keys of 64 and of 128, experts as wide as a tile. (Scales well below
# dim^-1/2: with these wide random weights a sharper softmax turns bfloat16 rounding of a score into a large change.)
CONFIG_D = {
    "architecture": "Diderax", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": attention(4, 2, 64, 0.06, 32, 500000.0, 4.0), "mlp": moe(11, 2, 96, identity=1, groups=(3, 2), scale=1.25, shared=160)},
        {"type": "gla", "mixer": gla(2, 64, 64, 12.0, 16), "mlp": dense(256)},
        {"type": "latent_attention", "mixer": latent(6, 48, 32, 64, 64, 56, 0.06, 32, 500000.0), "mlp": dense(128)},
        {"type": "gla", "mixer": gla(1, 128, 32, 8.0, 8), "mlp": None},
        {"type": "attention", "mixer": attention(2, 1, 128, 0.04, 128, 1e4), "mlp": moe(4, 2, 128)},
    ],
}

CONFIGS = {"A": (CONFIG_A, 21), "B": (CONFIG_B, 22), "C": (CONFIG_C, 23), "D": (CONFIG_D, 24)}


def random_config(seed: int) -> dict:
    """A configuration with every size, constant and the layer order drawn at random."""
    rng = random.Random(seed)
    width = rng.choice([24, 40, 64, 72])
    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["attention", "latent_attention", "gla"])
        factor = rng.choice([None, 1.0, 2.0, 6.0])
        if kind == "attention":
            groups, dim = rng.randint(1, 2), rng.choice([8, 16, 24, 32, 64])
            mixer = attention(groups * rng.randint(1, 3), groups, dim, rng.uniform(0.1, 0.4), rng.choice([2, dim // 2, dim]),
                              rng.choice([100.0, 1e4, 5e5]), factor)
        elif kind == "latent_attention":
            rot_dim = rng.choice([2, 8, 16])
            mixer = latent(rng.randint(1, 4), rng.choice([8, 16, 24]), rot_dim, rng.choice([8, 24, 32]), rng.choice([8, 16, 40]),
                           rng.choice([4, 16, 24]), rng.uniform(0.1, 0.4), rng.choice([2, rot_dim]), rng.choice([100.0, 1e4]), factor)
        else:
            mixer = gla(rng.randint(1, 3), rng.choice([8, 16, 24, 40]), rng.choice([8, 16, 24]), rng.choice([0.5, 1.0, 4.0, 16.0]),
                        rng.randint(1, 9))
        pick = rng.random()
        if pick < 0.25:
            mlp = None
        elif pick < 0.55:
            mlp = dense(rng.choice([16, 40, 72]))
        else:
            count = rng.choice([1, 2, 3, 4])
            size = rng.randint(1, 3)
            outputs = count * size
            identity = rng.randint(0, outputs - 1)
            keep = rng.randint(1, count)
            top = rng.randint(1, min(keep * size, 4))
            mlp = moe(outputs - identity, top, rng.choice([8, 16, 24]), identity=rng.choice([identity, None]) if identity == 0 else identity,
                      groups=None if count == 1 and rng.random() < 0.5 else (count, keep),
                      scale=rng.choice([None, 0.5, 1.5, 2.5]), shared=rng.choice([None, 8, 24]))
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Diderax", "vocab": rng.randint(40, 150), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])},
            "layers": layers}


def write_model(folder: Path, which: "str | dict", seed: int | None = None, std_scale: float = 6.0) -> Path:
    """The configuration with random weights, through the framework's random-weights mode."""
    import tinyserve_b200.architectures  # noqa: F401
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model

    cfg, s = CONFIGS[which] if isinstance(which, str) else (which, seed)
    return write_random_model(folder, config_from_dict(cfg), s, torch.bfloat16, std_scale=std_scale)


def oracle(folder: Path, tokens: list[int]) -> tuple[torch.Tensor, torch.Tensor]:
    """The plain model's logits in 64-bit, and for every position how far the same plain model in
    32-bit lies from them (its conditioning)."""
    import plain_diderax as plain

    cfg = plain.read_config(folder)
    want = plain.forward(cfg, plain.read_weights(folder, torch.float64), tokens)
    low = plain.forward(cfg, plain.read_weights(folder, torch.float32), tokens).double()
    return want.float(), row_errors(low, want)


def assert_rows_close(rows: torch.Tensor, want: torch.Tensor, cond: torch.Tensor, dtype: torch.dtype, what: str = "") -> None:
    """float32: every position within 2e-5 of the oracle's spread, a limit that grows with the position's
    conditioning (how far the plain model in 32-bit lies from itself in 64-bit). The linear-attention layer's
    read-out at a request's first tokens is ``(k . q) v`` divided by its own root mean square: where ``k . q``
    nearly cancels, any 32-bit computation loses the digits that cancel, whichever order it sums in; such
    positions get twenty times their conditioning. bfloat16: as for the other designs, judged over all positions."""
    if dtype != torch.float32:
        _assert_rows_close(rows, want, cond, dtype, what)
        return
    assert not rows.isnan().any(), f"{what}: NaN in the logits"
    err = row_errors(rows, want)
    limit = 2e-5 * torch.clamp(cond / 1e-6, min=1.0)
    worst = int((err / limit).argmax())
    assert bool((err <= limit).all()), f"{what}: position {worst}: relative error {float(err[worst]):.3g} (limit {float(limit[worst]):.3g})"
