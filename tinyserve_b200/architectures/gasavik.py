"""Gasavik: a decoder whose layers are listed one by one in ``config.json``. Every layer has ONE norm
whose output all its sub-layers read (a parallel residual layer): one of three mixers, optionally a
biased SwiGLU feed-forward beside it, and after their sum a per-layer input looked up by token id.
The mixers: ``parallel`` (windowed grouped-query attention that also keeps the first tokens, with a
gate per head, side by side with linear attention under a constant decay per head), ``wkv`` (time
mixing with a decay per key channel and a bonus for the current token) and ``delta`` (the gated
delta rule with one decay per head behind short causal convolutions). The embedding adds a learned
position row and is normed.

``config.json`` keys read here: ``architecture`` = "Gasavik"; ``vocab``, ``width``, ``max_positions``
(rows of the position table); ``norm.eps``; ``residual_mult`` (absent = 1); ``token_side.dim``
(absent or null = no per-layer token input); ``layers``: a list of ``{"type", "mixer": {...},
"mlp": {"kind": "dense", "ff"} | null}``. Mixer keys by type: ``parallel``: ``left`` (``heads,
kv_heads, dim, vdim, scale``, optional ``mask`` with ``size`` and ``keep_first``), ``right`` (``heads,
dim, vdim, decay`` (one constant per head)), ``left_scale``, ``right_scale`` (absent = 1); ``wkv``:
``heads, dim`` (and, only in configurations written by this framework, ``decay_rank``, which a
checkpoint's shapes give otherwise); ``delta``: ``heads, kv_heads, dim, vdim, conv``. Every size and
constant comes from these keys.

What the design fixes, passed to the parts as arguments by ``to_spec``: plain-weight RMS norms
computed in 32-bit and rounded once; q/k RMS norm per head and no rotation in the attention; biases on
q, k, v and on every feed-forward projection; SiLU in the feed-forward and the tanh form of GELU in the
token input; tensor names ``embed``, ``pos``, ``embed.norm``, ``side.embed``, ``l<i>.norm1``,
``l<i>.mix.*`` (``.left.*`` / ``.right.*`` for the two mixers side by side), ``l<i>.mlp.gate|up|down``
(+ ``.b``), ``l<i>.side.gate|proj|norm``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from ..config.base import LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec, UnsupportedConfigError
from ..config.registry import register_architecture

ARCHITECTURE = "Gasavik"
MIXER_TYPES = ("parallel", "wkv", "delta")
_MIXER_KEYS = {"wkv": ("heads", "dim"), "delta": ("heads", "kv_heads", "dim", "vdim", "conv")}
_LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale")
_RIGHT_KEYS = ("heads", "dim", "vdim", "decay")


def _need(d: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise UnsupportedConfigError(f"{where} has no {key!r}")
    return d[key]


@dataclass(frozen=True)
class GasavikConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    norm_eps: float
    max_positions: int
    layers: tuple[Mapping[str, Any], ...]
    residual_mult: float = 1.0
    token_side_dim: int | None = None
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    architecture = ARCHITECTURE

    def __post_init__(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or self.max_positions <= 0 or not self.norm_eps > 0:
            raise UnsupportedConfigError("vocab, width, max_positions and norm.eps must be positive")
        if self.token_side_dim is not None and self.token_side_dim <= 0:
            raise UnsupportedConfigError(f"token_side.dim={self.token_side_dim} must be positive")
        if not self.layers:
            raise UnsupportedConfigError("layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXER_TYPES:
                raise UnsupportedConfigError(f"{where}: unknown mixer type {kind!r}; known: {MIXER_TYPES}")
            m = _need(layer, "mixer", where)
            if kind == "parallel":
                left, right = _need(m, "left", f"{where}.mixer"), _need(m, "right", f"{where}.mixer")
                for key in _LEFT_KEYS:
                    _need(left, key, f"{where}.mixer.left")
                for key in _RIGHT_KEYS:
                    _need(right, key, f"{where}.mixer.right")
                if len(right["decay"]) != int(right["heads"]):
                    raise UnsupportedConfigError(f"{where}.mixer.right: {len(right['decay'])} decay constants for {right['heads']} heads")
                mask = left.get("mask")
                if mask is not None:
                    if int(_need(mask, "size", f"{where}.mixer.left.mask")) <= 0 or int(mask.get("keep_first", 0)) < 0:
                        raise UnsupportedConfigError(f"{where}.mixer.left.mask: size must be positive and keep_first not negative")
            else:
                for key in _MIXER_KEYS[kind]:
                    _need(m, key, f"{where}.mixer")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise UnsupportedConfigError(f"{where}: mlp.kind={mlp.get('kind')!r}: only 'dense' is implemented")
                _need(mlp, "ff", f"{where}.mlp")

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "GasavikConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != ARCHITECTURE:
            raise UnsupportedConfigError(f"expected {ARCHITECTURE}, got {name!r}")
        side = d.get("token_side")
        return cls(
            vocab_size=int(_need(d, "vocab", "config.json")),
            hidden_size=int(_need(d, "width", "config.json")),
            norm_eps=float(_need(_need(d, "norm", "config.json"), "eps", "norm")),
            max_positions=int(_need(d, "max_positions", "config.json")),
            layers=tuple(copy.deepcopy(dict(layer)) for layer in _need(d, "layers", "config.json")),
            residual_mult=float(d.get("residual_mult", 1.0)),
            token_side_dim=None if side is None else int(_need(side, "dim", "token_side")),
        )

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                             "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                             "residual_mult": self.residual_mult,
                             "layers": [copy.deepcopy(dict(layer)) for layer in self.layers]}
        if self.token_side_dim is not None:
            d["token_side"] = {"dim": self.token_side_dim}
        return d

    # ------------------------------------------------------------------ the spec
    def _mixers(self, kind: str, m: Mapping[str, Any]) -> tuple[dict[str, PartSpec], dict[str, float]]:
        """The mixer roles of a layer and the block's own constants for them."""
        h, eps = self.hidden_size, self.norm_eps
        if kind == "wkv":
            return {"mixer": PartSpec("time_mix", {
                "prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]),
                "norm_eps": eps, "decay_rank": int(m.get("decay_rank", -1))})}, {}
        if kind == "delta":
            return {"mixer": PartSpec("gated_delta", {
                "prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "conv_taps": int(m["conv"]), "norm_eps": eps})}, {}
        left, right = m["left"], m["right"]
        mask = left.get("mask") or {}
        return {
            "mixer": PartSpec("gated_sink_attention", {
                "prefix": "mix.left.", "hidden_size": h, "num_heads": int(left["heads"]),
                "num_kv_heads": int(left["kv_heads"]), "key_dim": int(left["dim"]), "value_dim": int(left["vdim"]),
                "scale": float(left["scale"]), "qk_norm": True, "qk_norm_eps": eps, "sink": False, "gate": "head",
                "window": None if mask.get("size") is None else int(mask["size"]),
                "keep_first": int(mask.get("keep_first", 0)) if mask.get("size") is not None else 0, "qkv_bias": True,
                "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "q_norm": "q.norm", "k_norm": "k.norm"}}),
            "second_mixer": PartSpec("decay_linear_attention", {
                "prefix": "mix.right.", "hidden_size": h, "num_heads": int(right["heads"]), "key_dim": int(right["dim"]),
                "value_dim": int(right["vdim"]), "decay": [float(x) for x in right["decay"]], "norm_eps": eps}),
        }, {"mixer_scale": float(m.get("left_scale", 1.0)), "second_mixer_scale": float(m.get("right_scale", 1.0))}

    def to_spec(self) -> ModelSpec:
        h, eps = self.hidden_size, self.norm_eps
        layers = []
        for i, layer in enumerate(self.layers):
            mixers, block_args = self._mixers(layer["type"], layer["mixer"])
            parts = {"norm": PartSpec("rms_norm", {"name": "norm1", "size": h, "eps": eps, "round_once": True}), **mixers}
            if layer.get("mlp") is not None:
                parts["feed_forward"] = PartSpec("gated_mlp", {
                    "prefix": "mlp.", "hidden_size": h, "intermediate_size": int(layer["mlp"]["ff"]), "activation": "silu",
                    "names": {"gate": "gate", "up": "up", "down": "down"}, "bias": True})
            if self.token_side_dim is not None:
                parts["token_input"] = PartSpec("gated_token_table", {
                    "prefix": "side.", "table_name": "side.embed", "vocab_size": self.vocab_size, "hidden_size": h,
                    "dim": self.token_side_dim, "index": i, "count": len(self.layers), "activation": "gelu_tanh"})
                parts["token_input_post_norm"] = PartSpec("post_rms_norm", {"name": "side.norm", "size": h, "eps": eps,
                                                                           "mult": self.residual_mult})
            layers.append(LayerSpec(prefix=f"l{i}.", block="parallel_residual", parts=parts,
                                    block_args={"residual_mult": self.residual_mult, **block_args}))
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab_size, hidden_size=h, layers=tuple(layers),
            order=tuple(LayerCall(i) for i in range(len(layers))),
            embedding=PartSpec("positioned_embedding", {
                "name": "embed", "vocab_size": self.vocab_size, "hidden_size": h, "position_name": "pos",
                "max_positions": self.max_positions, "norm_name": "embed.norm", "eps": eps}),
            final_norm=PartSpec("rms_norm", {"name": "final.norm", "size": h, "eps": eps, "round_once": True}),
            head=PartSpec("lm_head", {"name": "head", "tied": False, "vocab_size": self.vocab_size, "hidden_size": h}),
            max_position_embeddings=self.max_positions,
        )


register_architecture(ARCHITECTURE, GasavikConfig)
