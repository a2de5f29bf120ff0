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
unrotated size, ``position.theta`` the rotation's base, ``scale`` the factor on the scores.  Further options, each of
which leaves the above as it is when absent:

    ``q_rank`` = r      queries through a latent of their own: cq = rmsnorm(Wdq h) * gain (``q_norm`` [r]),
                        q = Wuq cq (``q_up``); [Wdkv; Wdq] is then the fused projection, rows [c' | kr | cq']
    ``sink`` False      no sink in the denominator;  ``gate`` False: no gate on the heads' results
    ``pairing`` "halves"    value i of the rotated run turns with value i + rot_dims / 2 instead of its neighbour
    ``position.scaling``    "yarn": stretched frequencies, and their constant on the sines and cosines
    ``window`` (the spec's) the row at position p sees the keys p - window + 1 .. p only (the cache keeps every row)
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
        self.position_spec = spec.position
        self.q_rank = int(o.get("q_rank", 0))
        self.has_sink, self.has_gate = bool(o.get("sink", True)), bool(o.get("gate", True))
        self.halves = o.get("pairing", "adjacent") == "halves"
        self.window = int(spec.window)
        if self.q_rank < 0 or self.window < 0 or o.get("pairing", "adjacent") not in ("adjacent", "halves"):
            raise ValueError(f"latent_attention: q_rank {self.q_rank}, window {self.window}, pairing {o.get('pairing')!r}")
        self.q_cols = self.heads * (self.dim + self.rot)
        if self.q_rank:
            if self.has_gate:
                raise ValueError("latent_attention: queries through a latent come without the gate")
            # [c' | kr | cq']: the key side first, so that it is a run of columns from column 0
            self.gate_col = 0
            self.in_proj = self.add("in_proj", Linear(spec.dim, self.rank + self.rot + self.q_rank, False))
            self.declare("q_norm", (self.q_rank,), role="vector")
            self.q_up = self.add("q_up", Linear(self.q_rank, self.q_cols, False))
        else:
            self.gate_col = self.q_cols + self.rank + self.rot
            self.in_proj = self.add("in_proj", Linear(spec.dim, self.gate_col + (self.heads if self.has_gate else 0), False))
        self.declare("latent_norm", (self.rank,), role="vector")
        if self.has_sink:
            self.declare("sink", (self.heads,), role="vector")
        self.rot_mult = 1.0
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
        from .position import rotary_inverse_frequencies, rotary_multiplier

        # every frequency in float64, rounded to float32 once
        scaling = self.position_spec.scaling_dict()
        freq = rotary_inverse_frequencies(max(self.rot_dims, 2), self.theta, scaling, dtype=torch.float64)[: self.rot_dims // 2]
        self._inv_freq = freq.to(torch.float32).to(device).contiguous()
        self.rot_mult = rotary_multiplier(scaling)

    def cache_request(self):
        return KVRequest(1, self.rank + self.rot, 0, planes=1)

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        n, width = x.shape[0], self.rank + self.rot
        proj = self.in_proj.forward(x)
        q_full = torch.empty((n, self.heads, width), dtype=proj.dtype, device=proj.device)
        kv, queries = None, proj
        if self.q_rank:
            kv = proj
            queries = self.q_up.forward(ops.latent_query_norm(proj, width, self.q_rank, self.tensor("q_norm"), self.eps))
        ops.latent_prepare(queries, q_full, self.tensor("latent_norm"), self.eps, self._inv_freq, self.rot_dims, batch,
                           cache_view, self.heads, self.dim, self.rot, self.rank, writes_cache, halves=self.halves,
                           rot_mult=self.rot_mult, kv=kv)
        if self.dim:
            ops.grouped_linear(queries, self._uk_t, self.heads, n, self.rank, self.dim, queries.shape[1], self.dim + self.rot,
                               q_full, self.heads * width, width)
        else:
            q_full[:, :, : self.rank].zero_()
        latent = ops.latent_attention(q_full, batch, cache_view, proj if self.has_gate else None, self.gate_col,
                                      self.tensor("sink") if self.has_sink else None, self.heads, self.rank, self.rot,
                                      self.scale, window=self.window)
        o = torch.empty((n, self.heads * self.vdim), dtype=proj.dtype, device=proj.device)
        ops.grouped_linear(latent, self._uv, self.heads, n, self.vdim, self.rank, self.heads * self.rank, self.rank, o,
                           self.heads * self.vdim, self.vdim)
        return self.dense.forward(o)

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["latent_attention", "grouped"]


register_mixer("latent_attention", LatentAttention)
