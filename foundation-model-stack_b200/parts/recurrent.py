"""Recurrent mixers: a state of fixed size per sequence instead of a cache that grows.

``MinGRU`` ("mingru"): a gated recurrence whose gates read the current token only.  With h the mixer's input,

    z = sigmoid(Wz h + bz)        u = Wx h + bx        c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
    S_t = (1 - z) S_(t-1) + z c   (element by element, S_(-1) = 0)
    y = Wo (S_t * silu(Wg h))

The three input projections are one fused matrix [Wz; Wx; Wg] with the bias [bz; bx; 0].  Gates, candidate, state and
the product with the output gate are float32; the state [width] lives in the cache's per-slot state (float32 in every
mode) and is carried from step to step.  Options of the ``MixerSpec``: ``width``.
"""
from __future__ import annotations

import torch

from ..cache.requests import StateRequest
from ..config.specs import MixerSpec
from ..kernels import ops
from .base import Part
from .linear import Linear
from .registry import register_mixer


class MinGRU(Part):
    def __init__(self, spec: MixerSpec) -> None:
        super().__init__()
        self.width = int(dict(spec.options)["width"])
        if self.width <= 0:
            raise ValueError(f"mingru: width {self.width}")
        self.in_proj = self.add("zxg_fused", Linear(spec.dim, 3 * self.width, bias=True))
        self.dense = self.add("dense", Linear(self.width, spec.dim, False))

    def cache_request(self):
        return StateRequest((self.width,), torch.float32, "mingru")

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        proj = self.in_proj.forward(x)
        y = ops.mingru_scan(proj, cache_view.state, batch, self.width, writes_cache)
        return self.dense.forward(y)

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["recurrent"]


register_mixer("mingru", MinGRU)
