"""Mixers that carry a matrix of state per head from token to token instead of a cache that grows, each with a short
causal convolution in front of it, and the mixer that runs two mixers side by side.

``SelectiveStateSpace`` ("selective_state_space"; the state-space-duality form of a selective scan).  With h the
mixer's input, H heads of ``vdim`` values (inner = H * vdim), a state of ``state`` rows, ``groups`` groups:

    [z | x | B | C | dt] = Win h                    inner, inner, groups * state, groups * state, H values
    (x, B, C) = silu(conv(x | B | C) + bias)        per channel over time, ``conv`` taps, zeros before the start
    dt = softplus(dt + dt_bias)                     head h uses group h // (H / groups)
    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T        y_t = S_t^T C_t + D_h x_t
    out = Wo (norm(y * silu(z)) * w)                the norm in ``norm_groups`` equal parts of the row, each by its own
                                                    root mean square; the gate comes before the norm

``GatedDeltaRule`` ("gated_delta_rule").  ``kvheads`` query/key heads of ``head_dim``, H value heads of ``vdim``
(head h uses query/key head h // (H / kvheads)):

    q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))      no bias
    q, k unit vectors per head: x / sqrt(sum(x^2) + 1e-6); q also times head_dim^-1/2
    beta = sigmoid(Wb h) per head;  g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 h) + dt_bias)) per head and key channel
    S = diag(g) S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q         (the read-out sees the token's own write)
    out = Wo (o / rms(o) * w * sigmoid(Wg2 (Wg1 h)))       rms per head over vdim, w [vdim] shared by the heads

Option ``decay`` "head": one decay a head instead of one a key channel, g = exp(-exp(A_log_h) softplus(Wa h + dt_bias_h))
with Wa [heads, width], and the gate is silu(Wg h) with Wg [heads * vdim, width] (no low-rank pairs); everything that
reads h is then ONE projection [q; k; v; b; a; zeros up to a multiple of 8 rows; g].

Projections that read h are fused into one matrix ([q; k; v; b] here, the checkpoint's one matrix there); the two
low-rank pairs keep their first factors as products of their own, whose results the second factors read as they lie.
Per sequence the cache holds the state matrices in float32 ([heads, vdim, rows], the rows contiguous) and the
convolution's last taps - 1 inputs: two ``StateRequest``s, so the mixer's view of the cache is a pair.  Everything after
the projections is float32 up to the rows that the output projection reads.

``ParallelMixers`` ("parallel"): two mixers read the same input; the result is left_factor * left + right_factor *
right.  Its cache request is the tuple of its mixers' requests.  It returns the two outputs with their factors
(``ScaledParts``); the norm that follows adds them in float32.
"""
from __future__ import annotations

import torch

from ..cache.requests import StateRequest
from ..config.specs import MixerSpec
from ..kernels import ops
from .base import Part
from .block import ScaledParts
from .linear import Linear
from .registry import build_mixer, register_mixer


def _as_requests(request):
    if request is None:
        return ()
    return tuple(request) if isinstance(request, (tuple, list)) else (request,)


class SelectiveStateSpace(Part):
    def __init__(self, spec: MixerSpec) -> None:
        super().__init__()
        o = dict(spec.options)
        self.heads, self.vdim = int(spec.nheads), int(o["vdim"])
        self.state, self.groups = int(o["state"]), int(o["groups"])
        self.taps, self.norm_groups = int(o["conv"]), int(o["norm_groups"])
        self.eps = float(o["eps"])
        self.inner = self.heads * self.vdim
        if min(self.heads, self.vdim, self.state, self.groups, self.taps, self.norm_groups) <= 0 \
                or self.heads % self.groups or self.inner % self.norm_groups:
            raise ValueError(f"selective_state_space: {self.heads} heads of {self.vdim}, state {self.state}, "
                             f"{self.groups} groups, {self.taps} taps, norm in {self.norm_groups} parts")
        self.channels = self.inner + 2 * self.groups * self.state
        self.in_proj = self.add("in_proj", Linear(spec.dim, self.inner + self.channels + self.heads, False))
        self.declare("conv", (self.channels, self.taps), role="vector")
        self.declare("conv_bias", (self.channels,), role="vector")
        for name in ("dt_bias", "A_log", "D"):
            self.declare(name, (self.heads,), role="vector")
        self.declare("norm", (self.inner,), role="vector")
        self.dense = self.add("dense", Linear(self.inner, spec.dim, False))
        self._f32 = {}

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        # the small vectors in float32, once: they enter the recurrence
        self._f32 = {n: self.tensor(n).float().contiguous() for n in ("conv", "conv_bias", "dt_bias", "A_log", "D", "norm")}

    def cache_request(self):
        return (StateRequest((self.heads, self.vdim, self.state), torch.float32, "state_matrix"),
                StateRequest((self.taps - 1, self.channels), torch.float32, "conv_tail"))

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        matrix, tail = cache_view
        p = self._f32
        proj = self.in_proj.forward(x)
        xbc = ops.causal_conv(proj, self.inner, self.channels, p["conv"], p["conv_bias"], tail.state, batch, True,
                              writes_cache)
        y = ops.selective_scan(xbc, proj, self.inner + self.channels, p["dt_bias"], p["A_log"], p["D"], matrix.state, batch,
                               self.heads, self.vdim, self.state, self.groups, writes_cache)
        y = ops.gated_group_rmsnorm(y, proj, 0, ops.GATE_SILU_BEFORE, p["norm"], self.eps, self.inner // self.norm_groups,
                                    proj.dtype)
        return self.dense.forward(y)

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["state_scan"]


class GatedDeltaRule(Part):
    def __init__(self, spec: MixerSpec) -> None:
        super().__init__()
        o = dict(spec.options)
        self.heads, self.kvheads, self.head_dim = int(spec.nheads), int(spec.kvheads), int(spec.head_dim)
        self.vdim, self.taps, self.eps = int(o["vdim"]), int(o["conv"]), float(o["eps"])
        self.per_head = o.get("decay", "channel") == "head"
        if o.get("decay", "channel") not in ("channel", "head"):
            raise ValueError(f"gated_delta_rule: decay {o.get('decay')!r}; known: channel, head")
        self.decay_rank, self.gate_rank = (1, 1) if self.per_head else (int(o["decay_rank"]), int(o["gate_rank"]))
        self.out_factor = float(o.get("out_factor", 1.0))
        if min(self.heads, self.kvheads, self.head_dim, self.vdim, self.taps, self.decay_rank, self.gate_rank) <= 0 \
                or self.heads % self.kvheads:
            raise ValueError(f"gated_delta_rule: {self.heads} heads of {self.vdim} over {self.kvheads} of {self.head_dim}, "
                             f"{self.taps} taps, ranks {self.decay_rank} and {self.gate_rank}")
        self.channels = 2 * self.kvheads * self.head_dim + self.heads * self.vdim
        if self.per_head:
            self.gate_col = self.gate_column(self.kvheads, self.head_dim, self.heads, self.vdim)
            self.in_proj = self.add("in_proj", Linear(spec.dim, self.gate_col + self.heads * self.vdim, False))
        else:
            self.in_proj = self.add("in_proj", Linear(spec.dim, self.channels + self.heads, False))  # [q; k; v; b]
            self.decay_in = self.add("decay_in", Linear(spec.dim, self.decay_rank, False))
            self.decay_out = self.add("decay_out", Linear(self.decay_rank, self.heads * self.head_dim, False))
            self.gate_in = self.add("gate_in", Linear(spec.dim, self.gate_rank, False))
            self.gate_out = self.add("gate_out", Linear(self.gate_rank, self.heads * self.vdim, False))
        self.declare("conv", (self.channels, self.taps), role="vector")
        self.declare("dt_bias", (self.heads if self.per_head else self.heads * self.head_dim,), role="vector")
        self.declare("A_log", (self.heads,), role="vector")
        self.declare("norm", (self.vdim,), role="vector")
        self.dense = self.add("dense", Linear(self.heads * self.vdim, spec.dim, False))
        self._f32 = {}

    @staticmethod
    def gate_column(kvheads: int, head_dim: int, heads: int, vdim: int) -> int:
        """With one decay a head: the row of the fused projection [q; k; v; b; a; zeros; g] at which the gates begin (a
        multiple of 8, so that their rows are read four at a time): what a checkpoint adapter has to put together."""
        return (2 * kvheads * head_dim + heads * vdim + 2 * heads + 7) // 8 * 8

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        self._f32 = {n: self.tensor(n).float().contiguous() for n in ("conv", "dt_bias", "A_log", "norm")}

    def cache_request(self):
        return (StateRequest((self.heads, self.vdim, self.head_dim), torch.float32, "state_matrix"),
                StateRequest((self.taps - 1, self.channels), torch.float32, "conv_tail"))

    def heads_out(self, x, batch, cache_view, writes_cache: bool = True):
        """The normed and gated heads' results [tokens, heads * vdim], before the output projection."""
        matrix, tail = cache_view
        p = self._f32
        proj = self.in_proj.forward(x)
        qkv = ops.causal_conv(proj, 0, self.channels, p["conv"], None, tail.state, batch, True, writes_cache)
        if self.per_head:
            o = ops.delta_rule_scan(qkv, proj, self.channels, None, p["dt_bias"], p["A_log"], matrix.state, batch, self.heads,
                                    self.kvheads, self.head_dim, self.vdim, writes_cache,
                                    decay_offset=self.channels + self.heads)
            return ops.gated_group_rmsnorm(o, proj, self.gate_col, ops.GATE_SILU_AFTER, p["norm"], self.eps, self.vdim,
                                           proj.dtype, self.out_factor)
        a = self.decay_out.forward(self.decay_in.forward(x))
        o = ops.delta_rule_scan(qkv, proj, self.channels, a, p["dt_bias"], p["A_log"], matrix.state, batch, self.heads,
                                self.kvheads, self.head_dim, self.vdim, writes_cache)
        gate = self.gate_out.forward(self.gate_in.forward(x))
        return ops.gated_group_rmsnorm(o, gate, 0, ops.GATE_SIGMOID_AFTER, p["norm"], self.eps, self.vdim, proj.dtype,
                                       self.out_factor)

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        return self.dense.forward(self.heads_out(x, batch, cache_view, writes_cache))

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["state_scan"]


class ParallelMixers(Part):
    def __init__(self, spec: MixerSpec) -> None:
        super().__init__()
        o = dict(spec.options)
        self.left = self.add("left", build_mixer(o["left"]))
        self.right = self.add("right", build_mixer(o["right"]))
        self.left_factor, self.right_factor = float(o.get("left_factor", 1.0)), float(o.get("right_factor", 1.0))
        self._n_left = len(_as_requests(self.left.cache_request()))

    def cache_request(self):
        return _as_requests(self.left.cache_request()) + _as_requests(self.right.cache_request())

    @staticmethod
    def _view_for(mixer, views):
        request = mixer.cache_request()
        if request is None:
            return None
        return tuple(views) if isinstance(request, (tuple, list)) else views[0]

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        views = tuple(cache_view)
        left = self.left.forward(x, batch, self._view_for(self.left, views[: self._n_left]), writes_cache)
        right = self.right.forward(x, batch, self._view_for(self.right, views[self._n_left:]), writes_cache)
        return ScaledParts([(left, self.left_factor), (right, self.right_factor)])


register_mixer("selective_state_space", SelectiveStateSpace)
register_mixer("gated_delta_rule", GatedDeltaRule)
register_mixer("parallel", ParallelMixers)
