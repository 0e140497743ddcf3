"""Diderax: a pre-norm decoder whose layers are listed one by one in ``config.json``. Each layer has
one of three mixers and optionally a feed-forward; every sub-layer's output is multiplied by a learned
factor per column (a layer scale) before the 32-bit residual sum.

The mixers: ``attention`` (grouped-query attention whose values are the keys as projected; q and k are
RMS-normed over the whole projection, partly rotated with linearly scaled frequencies; one is added to
the softmax's denominator; a sigmoid gate per output element), ``latent_attention`` (queries through a
normed latent of their own; keys and values from one cached normed latent per token plus a rotated key
part shared by the heads; a learned sink logit per head) and ``gla`` (gated linear attention: a matrix
memory per head with a decay per key channel and token, ``sigmoid(z)^(1/tau)``). The feed-forwards: a
biased SwiGLU, or a routed mixture of SwiGLU experts chosen by score plus correction inside the best
groups, with identity experts and a gated shared expert.

``config.json`` keys read here: ``architecture`` = "Diderax"; ``vocab``, ``width``; ``norm.eps``;
``layers``: a list of ``{"type", "mixer": {...}, "mlp": {...} | null}``. Mixer keys by type:
``attention``: ``heads, kv_heads, dim, vdim, scale``, ``rot`` (``dims, base``, optional
``scaling.factor``); ``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, q_rank, scale``, ``rot``
(``dims, base``, optional ``scaling.factor``); ``gla``: ``heads, dim, vdim, tau`` (and, only in
configurations written by this framework, ``decay_rank``, which a checkpoint's shapes give otherwise).
``mlp``: ``kind`` = "dense" with ``ff``, or "moe" with ``router`` (``experts, top``, optional ``identity``,
``scale``, ``groups.count``, ``groups.keep``), ``expert.ff`` and optional ``shared.ff``. Optional
``max_positions`` bounds a request's length for the engine's bookkeeping. Every size and constant comes
from these keys.

What the design fixes, passed to the parts as arguments by ``to_spec``: plain-weight RMS norms computed
in 32-bit and rounded once; the "half" rotation pairing; a sink of score 0 and a gate per element in the
attention; a learned sink in the latent attention; ``dim^-1/2`` on the queries of the linear attention,
whose read-out is normed per head with a weight shared by the heads and gated by SiLU; biases on the
dense feed-forward; softmax scores over all router outputs, a correction for the choice only, a gate on
the shared expert; tensor names ``embed``, ``l<i>.norm1|norm2``, ``l<i>.ls1|ls2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from ..config.base import LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec, UnsupportedConfigError
from ..config.registry import register_architecture

ARCHITECTURE = "Diderax"
MIXER_TYPES = ("attention", "latent_attention", "gla")
DEFAULT_MAX_POSITIONS = 1 << 17
_MIXER_KEYS = {"attention": ("heads", "kv_heads", "dim", "vdim", "scale", "rot"),
               "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot"),
               "gla": ("heads", "dim", "vdim", "tau")}


def _need(d: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise UnsupportedConfigError(f"{where} has no {key!r}")
    return d[key]


def _rotation(m: Mapping[str, Any], head_dim: int, where: str) -> PartSpec:
    rot = m["rot"]
    dims, base = int(_need(rot, "dims", f"{where}.rot")), float(_need(rot, "base", f"{where}.rot"))
    if dims % 2 or not 0 < dims <= head_dim:
        raise UnsupportedConfigError(f"{where}: rot.dims={dims} must be even and at most {head_dim}")
    args: dict[str, Any] = {"head_dim": head_dim, "rotary_dim": dims, "theta": base, "pairing": "half"}
    scaling = rot.get("scaling")
    if scaling is not None:
        factor = float(_need(scaling, "factor", f"{where}.rot.scaling"))
        if not factor > 0:
            raise UnsupportedConfigError(f"{where}: rot.scaling.factor={factor} must be positive")
        if factor != 1.0:
            args["scaling"] = {"factor": factor}
    return PartSpec("rope", args)


@dataclass(frozen=True)
class DideraxConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[Mapping[str, Any], ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    architecture = ARCHITECTURE

    def __post_init__(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or not self.norm_eps > 0:
            raise UnsupportedConfigError("vocab, width and norm.eps must be positive")
        if not self.layers:
            raise UnsupportedConfigError("layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXER_TYPES:
                raise UnsupportedConfigError(f"{where}: unknown mixer type {kind!r}; known: {MIXER_TYPES}")
            m = _need(layer, "mixer", where)
            for key in _MIXER_KEYS[kind]:
                _need(m, key, f"{where}.mixer")
            if kind == "attention":
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise UnsupportedConfigError(f"{where}: heads={m['heads']} is not a multiple of kv_heads={m['kv_heads']}")
                if int(m["vdim"]) != int(m["dim"]):
                    raise UnsupportedConfigError(f"{where}: the values are the keys, so vdim={m['vdim']} must equal dim={m['dim']}")
                _rotation(m, int(m["dim"]), f"{where}.mixer")
            elif kind == "latent_attention":
                _rotation(m, int(m["rot_dim"]), f"{where}.mixer")
            elif not float(m["tau"]) > 0:
                raise UnsupportedConfigError(f"{where}: tau={m['tau']} must be positive")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            mk = _need(mlp, "kind", f"{where}.mlp")
            if mk == "dense":
                _need(mlp, "ff", f"{where}.mlp")
            elif mk == "moe":
                router = _need(mlp, "router", f"{where}.mlp")
                experts, top = int(_need(router, "experts", "router")), int(_need(router, "top", "router"))
                outputs = experts + int(router.get("identity", 0))
                groups = router.get("groups") or {}
                count, keep = int(groups.get("count", 1)), int(groups.get("keep", 1))
                if experts <= 0 or int(router.get("identity", 0)) < 0 or not 0 < top <= outputs:
                    raise UnsupportedConfigError(f"{where}: top={top} of {experts} experts and {router.get('identity', 0)} identity experts")
                if count < 1 or outputs % count or not 1 <= keep <= count or outputs // count * keep < top:
                    raise UnsupportedConfigError(f"{where}: groups count={count} keep={keep} do not fit {outputs} router outputs and top={top}")
                _need(_need(mlp, "expert", f"{where}.mlp"), "ff", f"{where}.mlp.expert")
                if mlp.get("shared") is not None:
                    _need(mlp["shared"], "ff", f"{where}.mlp.shared")
            else:
                raise UnsupportedConfigError(f"{where}: mlp.kind={mk!r}: 'dense' and 'moe' are implemented")

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DideraxConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != ARCHITECTURE:
            raise UnsupportedConfigError(f"expected {ARCHITECTURE}, got {name!r}")
        return cls(
            vocab_size=int(_need(d, "vocab", "config.json")),
            hidden_size=int(_need(d, "width", "config.json")),
            norm_eps=float(_need(_need(d, "norm", "config.json"), "eps", "norm")),
            layers=tuple(copy.deepcopy(dict(layer)) for layer in _need(d, "layers", "config.json")),
            max_positions=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
        )

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.norm_eps}, "layers": [copy.deepcopy(dict(layer)) for layer in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d

    # ------------------------------------------------------------------ the spec
    def _mixer(self, kind: str, m: Mapping[str, Any]) -> tuple[PartSpec, PartSpec | None]:
        h, eps = self.hidden_size, self.norm_eps
        if kind == "attention":
            return PartSpec("gated_sink_attention", {
                "prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]), "qk_norm": "all",
                "qk_norm_eps": eps, "sink": "zero", "gate": "element", "values": "keys"}), _rotation(m, int(m["dim"]), "mixer")
        if kind == "latent_attention":
            return PartSpec("latent_attention", {
                "prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]), "nope_dim": int(m["dim"]),
                "rope_dim": int(m["rot_dim"]), "value_dim": int(m["vdim"]), "rank": int(m["kv_rank"]),
                "q_rank": int(m["q_rank"]), "scale": float(m["scale"]), "norm_eps": eps, "sink": True}), \
                _rotation(m, int(m["rot_dim"]), "mixer")
        return PartSpec("gated_linear_attention", {
            "prefix": "mix.", "hidden_size": h, "num_heads": int(m["heads"]), "key_dim": int(m["dim"]),
            "value_dim": int(m["vdim"]), "tau": float(m["tau"]), "norm_eps": eps,
            "decay_rank": int(m.get("decay_rank", -1))}), None

    def _feed_forward(self, mlp: Mapping[str, Any]) -> PartSpec:
        h = self.hidden_size
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"prefix": "mlp.", "hidden_size": h, "intermediate_size": int(mlp["ff"]),
                                          "activation": "silu", "bias": True,
                                          "names": {"gate": "gate", "up": "up", "down": "down"}})
        router, shared = mlp["router"], mlp.get("shared")
        groups = router.get("groups") or {}
        return PartSpec("routed_experts", {
            "prefix": "mlp.", "hidden_size": h, "num_experts": int(router["experts"]), "top": int(router["top"]),
            "expert_size": int(mlp["expert"]["ff"]), "shared_size": None if shared is None else int(shared["ff"]),
            "routing": "scored", "correction": True, "groups": int(groups.get("count", 1)),
            "group_keep": int(groups.get("keep", 1)), "route_scale": float(router.get("scale", 1.0)),
            "identity": int(router.get("identity", 0)), "shared_gate": shared is not None})

    def to_spec(self) -> ModelSpec:
        h, eps = self.hidden_size, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"name": name, "size": h, "eps": eps, "round_once": True})

        layers = []
        for i, layer in enumerate(self.layers):
            mixer, position = self._mixer(layer["type"], layer["mixer"])
            parts = {"mixer_norm": norm("norm1"), "mixer": mixer,
                     "mixer_post_norm": PartSpec("layer_scale", {"name": "ls1", "size": h})}
            if layer.get("mlp") is not None:
                parts["feed_forward_norm"] = norm("norm2")
                parts["feed_forward"] = self._feed_forward(layer["mlp"])
                parts["feed_forward_post_norm"] = PartSpec("layer_scale", {"name": "ls2", "size": h})
            layers.append(LayerSpec(prefix=f"l{i}.", block="sandwich", parts=parts, position=position))
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab_size, hidden_size=h, layers=tuple(layers),
            order=tuple(LayerCall(i) for i in range(len(layers))),
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": self.vocab_size, "hidden_size": h}),
            final_norm=PartSpec("rms_norm", {"name": "final.norm", "size": h, "eps": eps, "round_once": True}),
            head=PartSpec("lm_head", {"name": "head", "tied": False, "vocab_size": self.vocab_size, "hidden_size": h}),
            max_position_embeddings=self.max_positions,
        )


register_architecture(ARCHITECTURE, DideraxConfig)
