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
        self.limit, self.alpha = float(o["limit"]), float(o.get("alpha", 1.702))
        self.hidden = int(spec.hidden)
        if not (0 < self.top <= self.experts) or self.hidden <= 0:
            raise ValueError(f"routed_experts: {self.experts} experts, top {self.top}, hidden {self.hidden}")
        self.router = self.add("router", Linear(spec.dim, self.experts, False))
        self.declare("gate_up", (self.experts, 2 * self.hidden, spec.dim), role="matrix")
        self.declare("down", (self.experts, spec.dim, self.hidden), role="matrix")

    def forward(self, x):
        routing = ops.route(x, self.router.tensor("weight"), self.top)
        hidden = ops.routed_linear(routing.rows, self.tensor("gate_up"), routing, True, self.limit, self.alpha)
        return ops.route_gather(ops.routed_linear(hidden, self.tensor("down"), routing), routing)

    def kernel_libraries(self, dtype):
        return ["grouped"]


register_feed_forward("routed_experts", RoutedExperts)
