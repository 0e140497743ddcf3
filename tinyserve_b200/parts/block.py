"""Pre-norm residual block: ``x += mixer(norm(x)); x += feed_forward(norm(x))``
(upstream src/tinyserve/model.py:154-179). The two sums are not made here: each sub-layer's
output is left pending on the stream and the next norm adds it in 32-bit.
"""

from __future__ import annotations

from typing import Any, Mapping

from .base import Block, Part, ResidualStream, StepContext, register_block


class PreNormBlock(Block):
    # the order is the order of the layer's tensors in ``tensor_specs``
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, parts: Mapping[str, Part]) -> None:
        super().__init__(parts)
        self.mixer, self.feed_forward = parts["mixer"], parts["feed_forward"]
        self.mixer_norm, self.feed_forward_norm = parts["mixer_norm"], parts["feed_forward_norm"]

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, Any], writes_cache: bool,
                position: Any) -> None:
        # Scratch of this layer goes to the other half of the arena than the previous
        # layer's, whose pending output the first norm below still has to read.
        ctx.arena.next_frame()
        mixer, ff = self.mixer, self.feed_forward
        cache = caches.get("mixer")
        ctx.upcoming_weights = ff.streamed_weights()
        hn = self.mixer_norm.lazy(stream, ctx) if mixer.takes_lazy_input else self.mixer_norm.forward(stream, ctx)
        if mixer.adds_to_stream:
            mixed = mixer.forward(hn, ctx, cache, writes_cache, position, stream=stream)
        else:
            mixed = mixer.forward(hn, ctx, cache, writes_cache, position)
        self._leave(stream, mixed)
        hn = self.feed_forward_norm.lazy(stream, ctx) if ff.takes_lazy_input else self.feed_forward_norm.forward(stream, ctx)
        self._leave(stream, ff.forward(hn, ctx, stream=stream) if ff.adds_to_stream else ff.forward(hn, ctx))

    @staticmethod
    def _leave(stream: ResidualStream, out: Any) -> None:
        """A sub-layer's output stays pending on the stream, unless the part has added it itself."""
        if out is not None:
            stream.delta = out
            stream.sumsq = None


class SandwichBlock(Block):
    """A norm before and after each sub-layer: ``x += post(mixer(norm(x)))`` and, when the layer has
    a feed-forward, ``x += post(feed_forward(norm(x)))``. The post norms (``PostRMSNorm``, which may
    carry a layer scale, or a ``LayerScale`` alone) stay pending with the output and are applied by the next
    norm's kernel; a ``LayerScale`` also takes over the feed-forward's output bias."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    optional_roles = frozenset({"feed_forward_norm", "feed_forward", "feed_forward_post_norm"})

    def __init__(self, parts: Mapping[str, Part]) -> None:
        super().__init__(parts)
        ff = [r for r in ("feed_forward_norm", "feed_forward", "feed_forward_post_norm") if r in parts]
        if ff and len(ff) != 3:
            raise ValueError("a feed-forward comes with its norm and its post norm")
        for role in ("mixer_post_norm", "feed_forward_post_norm"):
            if role in parts and not hasattr(parts[role], "leave"):
                raise TypeError(f"role {role!r} takes a norm that can stay pending (a 'post_rms_norm')")

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, Any], writes_cache: bool,
                position: Any) -> None:
        p = self.parts
        ctx.arena.next_frame()
        ctx.upcoming_weights = []
        hn = p["mixer_norm"].forward(stream, ctx)
        p["mixer_post_norm"].leave(stream, p["mixer"].forward(hn, ctx, caches.get("mixer"), writes_cache, position))
        if "feed_forward" in p:
            hn = p["feed_forward_norm"].forward(stream, ctx)
            ff, post = p["feed_forward"], p["feed_forward_post_norm"]
            bias = getattr(ff, "output_bias", None)
            if bias is not None and getattr(post, "accepts_bias", False):
                # the feed-forward's output bias rides along with the pending output: no pass of its own
                post.leave(stream, ff.forward(hn, ctx, add_output_bias=False), bias)
            else:
                post.leave(stream, ff.forward(hn, ctx))


class ParallelResidualBlock(Block):
    """One norm whose output every sub-layer reads; their outputs are summed into the stream at once:
    ``h = norm(x)``; ``x <- x + m * (a * mixer(h) + b * second_mixer(h) + feed_forward(h))``, with the
    constants ``residual_mult`` m, ``mixer_scale`` a and ``second_mixer_scale`` b. Then, when the layer
    has a ``token_input``, ``y = token_input(x)`` (it reads the new stream) is left pending with its
    post norm (``token_input_post_norm``, which carries its own multiplier). The second mixer, the
    feed-forward and the token input are optional. The sum is one kernel over the 32-bit stream; it
    takes over the feed-forward's output bias and writes the copy of the stream that the token input
    reads."""

    roles = {"norm": "norm", "mixer": "mixer", "second_mixer": "mixer", "feed_forward": "feed_forward",
             "token_input": "token_input", "token_input_post_norm": "norm"}
    optional_roles = frozenset({"second_mixer", "feed_forward", "token_input", "token_input_post_norm"})

    def __init__(self, parts: Mapping[str, Part], residual_mult: float = 1.0, mixer_scale: float = 1.0,
                 second_mixer_scale: float = 1.0) -> None:
        super().__init__(parts)
        if ("token_input" in parts) != ("token_input_post_norm" in parts):
            raise ValueError("a token input comes with its post norm")
        if "token_input_post_norm" in parts and not hasattr(parts["token_input_post_norm"], "leave"):
            raise TypeError("role 'token_input_post_norm' takes a norm that can stay pending (a 'post_rms_norm')")
        self.mult, self.scale_a, self.scale_b = float(residual_mult), float(mixer_scale), float(second_mixer_scale)

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, Any], writes_cache: bool,
                position: Any) -> None:
        from ..kernels import ops

        p = self.parts
        ctx.arena.next_frame()
        ctx.upcoming_weights = []
        hn = p["norm"].forward(stream, ctx)
        terms = [p["mixer"].forward(hn, ctx, caches.get("mixer"), writes_cache, position)]
        scales = [self.mult * self.scale_a]
        if "second_mixer" in p:
            terms.append(p["second_mixer"].forward(hn, ctx, caches.get("second_mixer"), writes_cache, position))
            scales.append(self.mult * self.scale_b)
        bias = None
        if "feed_forward" in p:
            ff = p["feed_forward"]
            bias = getattr(ff, "output_bias", None)
            terms.append(ff.forward(hn, ctx) if bias is None else ff.forward(hn, ctx, add_output_bias=False))
            scales.append(self.mult)
        copy = ctx.arena.take(tuple(stream.resid.shape), ctx.dtype) if "token_input" in p else None
        ops.stream_sum(stream.resid, terms, scales, bias=bias, bias_scale=self.mult, copy=copy)
        stream.sumsq = None
        if copy is not None:
            p["token_input_post_norm"].leave(stream, p["token_input"].forward(copy, ctx))


register_block("parallel_residual", ParallelResidualBlock)
register_block("prenorm", PreNormBlock)
register_block("sandwich", SandwichBlock)
