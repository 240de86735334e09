"""Attention whose cache holds one small latent row per position instead of keys and values per head.

``LatentAttention`` ("latent_attention").  With h the mixer's input, H heads, and per head ``dim`` unrotated and ``rot``
rotated query/key values, ``vdim`` value values and a latent of ``rank`` values:

    q = Wq h                      per head [dim unrotated | rot rotated]
    [c' | kr] = Wdkv h            c = rmsnorm(c') * gain (rank values), kr: rot values, one rotated key part for all heads
    k_h = [Wuk,h c | kr]          v_h = Wuv,h c
    s_h(i, j) = (q_h(i) . k_h(j)) * scale for j <= i, rotation of the rot parts by position (adjacent pairs, the first
                rot_dims values, angle = position * base^(-2i / rot_dims))
    p = exp(s) / (sum_j exp(s) + exp(sink_h))           a learned sink per head: no key, no value, counted once
    o_h = sigmoid(Wg h)_h * sum_j p v_h(j)              y = Wo [o_1 .. o_H]

Only [c | kr] is cached (a key/value group with one head, one plane).  The up-projections never touch the cache:
q_h . Wuk,h c = (Wuk,h^T q_h) . c, so the query is taken into the latent's space before attention (a product per head,
``uk`` transposed once at load time), attention runs over the latent rows as they lie, and the head's result, a
weighted sum of latents, goes through Wuv,h afterwards.  [Wq; Wdkv; Wg] is one fused projection.

Options of the ``MixerSpec``: ``rot`` (rotated values per head), ``vdim``, ``rank``, ``rot_dims``; ``head_dim`` is the
unrotated size, ``position.theta`` the rotation's base, ``scale`` the factor on the scores.
"""
from __future__ import annotations

import torch

from ..cache.requests import KVRequest
from ..config.specs import MixerSpec
from ..kernels import ops
from .base import Part
from .linear import Linear
from .registry import register_mixer


class LatentAttention(Part):
    def __init__(self, spec: MixerSpec) -> None:
        super().__init__()
        o = dict(spec.options)
        self.heads, self.dim = int(spec.nheads), int(spec.head_dim)
        self.rot, self.vdim, self.rank = int(o["rot"]), int(o["vdim"]), int(o["rank"])
        self.rot_dims = int(o.get("rot_dims", self.rot))
        if min(self.heads, self.vdim, self.rank) <= 0 or self.dim < 0 or self.rot < 0 or self.dim + self.rot == 0:
            raise ValueError(f"latent_attention: heads {self.heads}, dim {self.dim}, rot {self.rot}, vdim {self.vdim}, "
                             f"rank {self.rank}")
        if self.rot_dims % 2 or not (0 <= self.rot_dims <= self.rot):
            raise ValueError(f"latent_attention: {self.rot_dims} rotated values of {self.rot}")
        if spec.scale is None:
            raise ValueError("latent_attention: the scale of the scores is given by the configuration")
        self.scale = float(spec.scale)
        self.eps = float(o["eps"])
        self.theta = float(spec.position.theta)
        self.q_cols = self.heads * (self.dim + self.rot)
        self.gate_col = self.q_cols + self.rank + self.rot
        self.in_proj = self.add("in_proj", Linear(spec.dim, self.gate_col + self.heads, False))
        self.declare("latent_norm", (self.rank,), role="vector")
        self.declare("sink", (self.heads,), role="vector")
        self.declare("uk", (self.heads * self.dim, self.rank), role="matrix")
        self.declare("uv", (self.heads * self.vdim, self.rank), role="matrix")
        self.dense = self.add("dense", Linear(self.heads * self.vdim, spec.dim, False))
        self._uk_t = self._uv = self._inv_freq = None

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        uk = self.tensor("uk")
        # [heads, rank, dim]: head h's matrix that takes its unrotated query into the latent's space
        self._uk_t = uk.view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self._uv = self.tensor("uv").view(self.heads, self.vdim, self.rank)
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        freq = torch.tensor(self.theta, dtype=torch.float64) ** (-2.0 * i / max(self.rot_dims, 1))
        self._inv_freq = freq.to(torch.float32).to(device).contiguous()

    def cache_request(self):
        return KVRequest(1, self.rank + self.rot, 0, planes=1)

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        n, width = x.shape[0], self.rank + self.rot
        proj = self.in_proj.forward(x)
        q_full = torch.empty((n, self.heads, width), dtype=proj.dtype, device=proj.device)
        ops.latent_prepare(proj, q_full, self.tensor("latent_norm"), self.eps, self._inv_freq, self.rot_dims, batch,
                           cache_view, self.heads, self.dim, self.rot, self.rank, writes_cache)
        if self.dim:
            ops.grouped_linear(proj, self._uk_t, self.heads, n, self.rank, self.dim, proj.shape[1], self.dim + self.rot,
                               q_full, self.heads * width, width)
        else:
            q_full[:, :, : self.rank].zero_()
        latent = ops.latent_attention(q_full, batch, cache_view, proj, self.gate_col, self.tensor("sink"), self.heads,
                                      self.rank, self.rot, self.scale)
        o = torch.empty((n, self.heads * self.vdim), dtype=proj.dtype, device=proj.device)
        ops.grouped_linear(latent, self._uv, self.heads, n, self.vdim, self.rank, self.heads * self.rank, self.rank, o,
                           self.heads * self.vdim, self.vdim)
        return self.dense.forward(o)

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["latent_attention", "grouped"]


register_mixer("latent_attention", LatentAttention)
