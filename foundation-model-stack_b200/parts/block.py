"""One layer: norms, mixer and feed-forward in their arrangement.

The residual stream is float32.  A sublayer's output is not added to it by the sublayer: it is handed to the
next norm, which adds it to the stream in the same pass that norms it.  So a block's ``forward`` takes the
pending output of the layer before and returns its own last sublayer's output, still pending.

Interface of a block (what the decoder calls); ``BlockSpec.arrangement`` names the class in the registry:

    cache_request() -> what its mixer asks of the cache (KVRequest | StateRequest | None)
    forward(residual, pending, batch, cache_view, writes_cache, dtype) -> pending
        residual [tokens, dim] float32, updated in place; pending [tokens, dim] in the compute dtype or None

``PreNormBlock`` ("pre_norm", fms/models/llama.py:118-167): x += mixer(norm(x)); x += feed_forward(norm(x)).

``PostNormBlock`` ("post_norm"): x = norm1(alpha x + mixer(x)); x = norm2(alpha x + feed_forward(x)); the sublayers
read the stream itself, and what the block hands on is a ``StreamCopy`` (nothing pending).

``SandwichBlock`` ("sandwich"): a norm before and after each sublayer, x += post1(mixer(pre1(x)));
x += post2(feed_forward(pre2(x))).  What it hands on as pending is a ``NormedDelta``: the next norm (this layer's, the
next layer's or the decoder's last) norms it, adds it and takes its own norm in one kernel.  A layer without a
feed-forward ends after its mixer.

``ParallelResidualBlock`` ("parallel_residual"): x += mixer(norm1(x)) + feed_forward(norm2(x)), both norms of the same
stream and from one kernel; what it hands on is the list of its outputs with their factors.

``OutputNormBlock`` ("output_norm"): a norm on each sublayer's output only, x += norm1(mixer(x));
x += norm2(feed_forward(x)); the sublayers read the stream itself.  What it hands on is a ``NormedDelta`` as well; the
kernel that adds it also leaves the summed stream in the compute dtype for the sublayer that reads it next.
"""
from __future__ import annotations

from ..config.specs import BlockSpec
from .base import Part
from ..kernels import ops
from .norm import NormedDelta, StreamCopy
from .registry import build_feed_forward, build_mixer, build_norm, register_block


class PreNormBlock(Part):
    def __init__(self, spec: BlockSpec) -> None:
        super().__init__()
        n_mixer_norm, n_mixer, n_ff_norm, n_ff = spec.names
        self.mixer_norm = self.add(n_mixer_norm, build_norm(spec.mixer_norm))
        self.mixer = self.add(n_mixer, build_mixer(spec.mixer))
        self.feed_forward_norm = self.add(n_ff_norm, build_norm(spec.feed_forward_norm))
        self.feed_forward = self.add(n_ff, build_feed_forward(spec.feed_forward))

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, residual, pending, batch, cache_view, writes_cache, dtype):
        h = self.mixer_norm.apply(residual, pending, dtype)
        a = self.mixer.forward(h, batch, cache_view, writes_cache)
        h = self.feed_forward_norm.apply(residual, a, dtype)
        return self.feed_forward.forward(h)


class SandwichBlock(Part):
    def __init__(self, spec: BlockSpec) -> None:
        super().__init__()
        n_mixer_norm, n_mixer, n_ff_norm, n_ff = spec.names
        n_mixer_post, n_ff_post = spec.post_names
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and (
                spec.feed_forward_norm is None or spec.feed_forward_post_norm is None)):
            raise ValueError("a sandwich layer needs a norm before and after each of its sublayers")
        self.mixer_norm = self.add(n_mixer_norm, build_norm(spec.mixer_norm))
        self.mixer = self.add(n_mixer, build_mixer(spec.mixer))
        self.mixer_post_norm = self.add(n_mixer_post, build_norm(spec.mixer_post_norm))
        self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = self.add(n_ff_norm, build_norm(spec.feed_forward_norm))
            self.feed_forward = self.add(n_ff, build_feed_forward(spec.feed_forward))
            self.feed_forward_post_norm = self.add(n_ff_post, build_norm(spec.feed_forward_post_norm))

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, residual, pending, batch, cache_view, writes_cache, dtype):
        h = self.mixer_norm.apply(residual, pending, dtype)
        pending = NormedDelta(self.mixer.forward(h, batch, cache_view, writes_cache), self.mixer_post_norm)
        if self.feed_forward is None:
            return pending
        h = self.feed_forward_norm.apply(residual, pending, dtype)
        return NormedDelta(self.feed_forward.forward(h), self.feed_forward_post_norm)


class ScaledParts:
    """What a mixer made of several returns instead of one tensor: [(output, factor), ...], whose weighted sum is the
    mixer's output.  The norm that follows takes the sum in float32 on its way, so it is never rounded."""

    __slots__ = ("parts",)

    def __init__(self, parts) -> None:
        self.parts = list(parts)


class PostNormBlock(Part):
    """``post_norm``: the sublayers read the stream itself and the norm follows the sum,
    x = norm1(alpha x + mixer(x)); x = norm2(alpha x + feed_forward(x)); option ``alpha`` (1 by default).  A layer
    without a feed-forward ends after its first norm.  The stream stays float32; each norm also leaves it in the
    compute dtype for the sublayer that reads it next."""

    def __init__(self, spec: BlockSpec) -> None:
        super().__init__()
        n_mixer_norm, n_mixer, n_ff_norm, n_ff = spec.names
        self.alpha = float(dict(spec.options).get("alpha", 1.0))
        self.mixer = self.add(n_mixer, build_mixer(spec.mixer))
        self.mixer_norm = self.add(n_mixer_norm, build_norm(spec.mixer_norm))
        self.feed_forward = None
        if spec.feed_forward is not None:
            if spec.feed_forward_norm is None:
                raise ValueError("a post-norm layer with a feed-forward needs the norm that follows it")
            self.feed_forward = self.add(n_ff, build_feed_forward(spec.feed_forward))
            self.feed_forward_norm = self.add(n_ff_norm, build_norm(spec.feed_forward_norm))

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, residual, pending, batch, cache_view, writes_cache, dtype):
        if isinstance(pending, StreamCopy):
            h = pending.rows
        elif pending is None:
            h = ops.cast_rows(residual, dtype)
        else:
            raise ValueError("a post-norm layer follows a layer that left its output pending; only layers whose norms "
                             "bring the stream up to date may come before it")
        a = self.mixer.forward(h, batch, cache_view, writes_cache)
        parts = a.parts if isinstance(a, ScaledParts) else [(a, 1.0)]
        h = self.mixer_norm.apply_after_sum(residual, self.alpha, parts, dtype)
        if self.feed_forward is not None:
            h = self.feed_forward_norm.apply_after_sum(residual, self.alpha, [(self.feed_forward.forward(h), 1.0)], dtype)
        return StreamCopy(h)

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["elementwise"]


class OutputNormBlock(Part):
    """``output_norm``: x += norm1(mixer(x)); x += norm2(feed_forward(x)), with no norm in front of a sublayer.  The
    norms need ``add(residual, delta, dtype)`` (``LayerNorm`` has it).  A layer without a feed-forward ends after its
    mixer.  The last sublayer's output stays pending with its norm, so that whatever comes next (this arrangement's
    next layer, or the decoder's last norm) adds it in the kernel that it runs anyway."""

    def __init__(self, spec: BlockSpec) -> None:
        super().__init__()
        n_mixer_norm, n_mixer, n_ff_norm, n_ff = spec.names
        self.mixer = self.add(n_mixer, build_mixer(spec.mixer))
        self.mixer_norm = self.add(n_mixer_norm, build_norm(spec.mixer_norm))
        self.feed_forward = None
        if spec.feed_forward is not None:
            if spec.feed_forward_norm is None:
                raise ValueError("an output-norm layer with a feed-forward needs the norm of its output")
            self.feed_forward = self.add(n_ff, build_feed_forward(spec.feed_forward))
            self.feed_forward_norm = self.add(n_ff_norm, build_norm(spec.feed_forward_norm))

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, residual, pending, batch, cache_view, writes_cache, dtype):
        if isinstance(pending, NormedDelta) and hasattr(pending.norm, "add"):
            h = pending.norm.add(residual, pending.delta, dtype)
        elif isinstance(pending, StreamCopy):
            h = pending.rows
        elif pending is None:
            h = ops.cast_rows(residual, dtype)
        else:
            raise ValueError("an output-norm layer follows a layer whose pending output it cannot add: only a normed "
                             "output whose norm has add(), or an up-to-date stream, may come before it")
        a = self.mixer.forward(h, batch, cache_view, writes_cache)
        if self.feed_forward is None:
            return NormedDelta(a, self.mixer_norm)
        h = self.mixer_norm.add(residual, a, dtype)
        return NormedDelta(self.feed_forward.forward(h), self.feed_forward_norm)

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["elementwise"]


class ParallelResidualBlock(Part):
    """``parallel_residual``: both sublayers read the same stream, each through a norm of its own, and their outputs are
    added together: x += mixer(norm1(x)) + feed_forward(norm2(x)).  The two norms come from one kernel
    (``apply_pair``), which first adds what the layer before left pending; what this layer hands on is the list of its
    outputs with their factors (``ScaledParts``: a mixer made of two gives two), added in float32 by whichever norm
    comes next.  A layer without a feed-forward is x += mixer(norm1(x))."""

    def __init__(self, spec: BlockSpec) -> None:
        super().__init__()
        n_mixer_norm, n_mixer, n_ff_norm, n_ff = spec.names
        self.mixer_norm = self.add(n_mixer_norm, build_norm(spec.mixer_norm))
        self.mixer = self.add(n_mixer, build_mixer(spec.mixer))
        self.feed_forward = None
        if spec.feed_forward is not None:
            if spec.feed_forward_norm is None:
                raise ValueError("a layer with a feed-forward needs its norm")
            self.feed_forward_norm = self.add(n_ff_norm, build_norm(spec.feed_forward_norm))
            self.feed_forward = self.add(n_ff, build_feed_forward(spec.feed_forward))
        if not hasattr(self.mixer_norm, "apply_pair"):
            raise ValueError("a parallel_residual layer needs norms with apply_pair (group_rmsnorm)")

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, residual, pending, batch, cache_view, writes_cache, dtype):
        if self.feed_forward is None:
            h = self.mixer_norm.apply(residual, pending, dtype)
            a = self.mixer.forward(h, batch, cache_view, writes_cache)
            return a if isinstance(a, ScaledParts) else ScaledParts([(a, 1.0)])
        h1, h2 = self.mixer_norm.apply_pair(residual, pending, self.feed_forward_norm, dtype)
        a = self.mixer.forward(h1, batch, cache_view, writes_cache)
        parts = list(a.parts) if isinstance(a, ScaledParts) else [(a, 1.0)]
        return ScaledParts(parts + [(self.feed_forward.forward(h2), 1.0)])

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["elementwise"]


Block = PreNormBlock  # the name under which earlier callers know it
register_block("parallel_residual", ParallelResidualBlock)
register_block("output_norm", OutputNormBlock)
register_block("post_norm", PostNormBlock)
register_block("pre_norm", PreNormBlock)
register_block("sandwich", SandwichBlock)
