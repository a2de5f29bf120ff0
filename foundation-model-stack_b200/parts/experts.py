"""Routed feed-forwards: many small experts, of which every token uses a few.

``RoutedExperts`` ("routed_experts").  With h the feed-forward's input:

    s = sigmoid(Wr h)                         router scores, float32
    the ``top`` experts with the largest scores are the token's; their scores are its weights, as they are
    expert_e(v) = Wdown,e (g * sigmoid(alpha g) * (u + 1)),  g = min(Wgate,e v, limit),  u = clamp(Wup,e v, -limit, limit)
    y = sum over the chosen e of expert_e(s_e * h)        the weight multiplies the expert's INPUT

The experts' matrices are stacked: ``gate_up`` [experts, 2 hidden, dim] (gate rows, then up rows) and ``down``
[experts, dim, hidden].  A step sorts its (token, choice) pairs by expert on the device (no answer from the device is
waited for), runs the two products group by group with the gated unit in the first one's epilogue, and sums every
token's rows.  Options of the ``FeedForwardSpec``: ``experts``, ``top``, ``limit``, ``alpha`` (1.702).

Further options, each of which leaves the above as it is when absent:

    ``scoring`` "softmax"     s = softmax(Wr h) over all experts; a token's experts are the ``top`` largest of
                              s + ``correction`` (a vector of the checkpoint, one number an expert, where ``correction``
                              is set); its weights are the chosen scores s (without the correction) over their sum
                              (+ 1e-20), times ``route_scale``; the weight multiplies the expert's OUTPUT
    ``unit`` "relu_squared"   expert_e(v) = Wdown,e relu(Wup,e v)^2: no gate; ``up`` [experts, hidden, dim]
"""
from __future__ import annotations

from ..config.specs import FeedForwardSpec
from ..kernels import ops
from .base import Part
from .linear import Linear
from .registry import register_feed_forward


class RoutedExperts(Part):
    def __init__(self, spec: FeedForwardSpec) -> None:
        super().__init__()
        o = dict(spec.options)
        self.experts, self.top = int(o["experts"]), int(o["top"])
        self.limit, self.alpha = float(o.get("limit", 0.0)), float(o.get("alpha", 1.702))
        self.hidden = int(spec.hidden)
        if not (0 < self.top <= self.experts) or self.hidden <= 0:
            raise ValueError(f"routed_experts: {self.experts} experts, top {self.top}, hidden {self.hidden}")
        self.scoring, self.unit = o.get("scoring", "sigmoid"), o.get("unit", "gated_clamped")
        if self.scoring not in ("sigmoid", "softmax") or self.unit not in ("gated_clamped", "relu_squared"):
            raise ValueError(f"routed_experts: scoring {self.scoring!r}, unit {self.unit!r}")
        if self.unit == "gated_clamped" and "limit" not in o:
            raise ValueError("routed_experts: the gated unit needs its limit")
        self.route_scale, self.has_correction = float(o.get("route_scale", 1.0)), bool(o.get("correction", False))
        self.router = self.add("router", Linear(spec.dim, self.experts, False))
        if self.has_correction:
            self.declare("correction", (self.experts,), role="vector")
        if self.unit == "relu_squared":
            self.declare("up", (self.experts, self.hidden, spec.dim), role="matrix")
        else:
            self.declare("gate_up", (self.experts, 2 * self.hidden, spec.dim), role="matrix")
        self.declare("down", (self.experts, spec.dim, self.hidden), role="matrix")
        self._correction = None

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        if self.has_correction:
            self._correction = self.tensor("correction").float().contiguous()

    def forward(self, x):
        if self.scoring == "softmax":
            routing = ops.route(x, self.router.tensor("weight"), self.top, ops.ROUTE_SOFTMAX, self._correction,
                                self.route_scale)
        else:
            routing = ops.route(x, self.router.tensor("weight"), self.top)
        if self.unit == "relu_squared":
            hidden = ops.routed_linear(routing.rows, self.tensor("up"), routing, relu_squared=True)
            return ops.route_gather(ops.routed_linear(hidden, self.tensor("down"), routing), routing)
        hidden = ops.routed_linear(routing.rows, self.tensor("gate_up"), routing, True, self.limit, self.alpha)
        return ops.route_gather(ops.routed_linear(hidden, self.tensor("down"), routing), routing)

    def kernel_libraries(self, dtype):
        return ["grouped"]


register_feed_forward("routed_experts", RoutedExperts)
