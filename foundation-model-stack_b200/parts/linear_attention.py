"""Mixers that keep, per head, a matrix S of key-value products under a scalar decay instead of a cache that grows:
S_t = a_t S_(t-1) + b_t k_t v_t^T, read out with the query as o_t = S_t^T q_t.  With h the mixer's input, H heads, keys and
queries of ``head_dim``, values of ``vdim``, all laid out head by head:

``LightningAttention`` ("lightning_attention"): one decay per head and nothing else,

    q, k, v = silu(Wq h), silu(Wk h), silu(Wv h)
    S_t = decay_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t                      option ``decay``: a number per head
    out = Wo (o / rms(o) * w * sigmoid(Wg h))                                 the root mean square over all heads' values together

``MatrixLSTM`` ("mlstm"; the matrix memory of the xLSTM with exponential gates, kept in range by a running maximum),

    q = Wq h / sqrt(head_dim), k = Wk h, v = Wv h
    i = cap tanh((Wi h + bi) / cap);  f = logsigmoid(cap tanh((Wf h + bf) / cap))        per head; option ``gate_cap``
    m_t = max(f + m_(t-1), i)                                                             m = 0 before the first token
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T;  n_t the same with k alone
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
    out = Wo (o / rms(o) * w * sigmoid(Wg h))                                 the root mean square per head; w [H * vdim]

Everything that reads h is one fused projection, [q; k; v; g] or [q; k; v; g; i; f], its rows filled up with zeros to a
multiple of 8; the gates' biases are added in float32 by the kernel that takes the gates.  Per sequence the cache holds
the state matrices in float32 ([heads, vdim, head_dim], a column's rows contiguous) and, for the gated form, the
normalizer with the running maximum behind it ([heads, head_dim + 1]).  Everything after the projection is float32 up
to the rows that the output projection reads.
"""
from __future__ import annotations

import torch

from ..cache.requests import StateRequest
from ..config.specs import MixerSpec
from ..kernels import ops
from .base import Part
from .linear import Linear
from .registry import register_mixer


def _round8(n: int) -> int:
    return (n + 7) // 8 * 8


class _DecayedStateMixer(Part):
    """What the two kinds share: sizes, the fused projection, the output norm's weight, the output projection."""

    extra_rows_per_head = 0  # rows of the fused projection behind [q; k; v; g], per head

    def __init__(self, spec: MixerSpec) -> None:
        super().__init__()
        o = dict(spec.options)
        self.heads, self.head_dim = int(spec.nheads), int(spec.head_dim)
        self.vdim, self.eps = int(o.get("vdim", spec.head_dim)), float(o.get("eps", 1e-6))
        if min(self.heads, self.head_dim, self.vdim) <= 0 or self.head_dim > 256:
            raise ValueError(f"{spec.kind}: {self.heads} heads of {self.head_dim} (up to 256) with values of {self.vdim}")
        self.inner = self.heads * self.vdim
        self.gate_col = self.heads * (2 * self.head_dim + self.vdim)  # where [g] starts in the fused projection's rows
        self.in_proj = self.add("in_proj", Linear(spec.dim, self.fused_rows(self.heads, self.head_dim, self.vdim), False))
        self.declare("norm", (self.inner,), role="vector")
        self.dense = self.add("dense", Linear(self.inner, spec.dim, False))
        self._norm = None

    @classmethod
    def fused_rows(cls, heads: int, head_dim: int, vdim: int) -> int:
        """Rows of the fused projection: what a checkpoint adapter has to put together."""
        return _round8(heads * (2 * head_dim + 2 * vdim + cls.extra_rows_per_head))

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        self._norm = self.tensor("norm").float().contiguous()

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["state_scan"]


class LightningAttention(_DecayedStateMixer):
    def __init__(self, spec: MixerSpec) -> None:
        super().__init__(spec)
        self.decay = tuple(float(d) for d in dict(spec.options)["decay"])
        if len(self.decay) != self.heads:
            raise ValueError(f"lightning_attention: {len(self.decay)} decays for {self.heads} heads")
        self._decay = None

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        self._decay = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(device)

    def cache_request(self):
        return StateRequest((self.heads, self.vdim, self.head_dim), torch.float32, "state_matrix")

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        proj = self.in_proj.forward(x)
        o = ops.decay_scan(proj, cache_view.state, batch, self.heads, self.head_dim, self.vdim, activation=ops.ACT_SILU,
                           decay=self._decay, writes_state=writes_cache)
        y = ops.gated_group_rmsnorm(o, proj, self.gate_col, ops.GATE_SIGMOID_AFTER, self._norm, self.eps, self.inner,
                                    proj.dtype)
        return self.dense.forward(y)


class MatrixLSTM(_DecayedStateMixer):
    extra_rows_per_head = 2  # the input gate's and the forget gate's row

    def __init__(self, spec: MixerSpec) -> None:
        super().__init__(spec)
        self.gate_cap = float(dict(spec.options)["gate_cap"])
        if not self.gate_cap > 0.0:
            raise ValueError(f"mlstm: gate_cap {self.gate_cap}")
        self.exp_gate_col = self.gate_col + self.inner  # [i: heads | f: heads] behind [g]
        self.declare("gate_bias", (2 * self.heads,), role="vector")  # the input gates' biases, then the forget gates'
        self._gate_bias = None

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        self._gate_bias = self.tensor("gate_bias").float().contiguous()

    def cache_request(self):
        return (StateRequest((self.heads, self.vdim, self.head_dim), torch.float32, "state_matrix"),
                StateRequest((self.heads, self.head_dim + 1), torch.float32, "normalizer_and_maximum"))

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        matrix, normalizer = cache_view
        proj = self.in_proj.forward(x)
        o = ops.decay_scan(proj, matrix.state, batch, self.heads, self.head_dim, self.vdim,
                           q_scale=self.head_dim ** -0.5, gate_offset=self.exp_gate_col, gate_bias=self._gate_bias,
                           gate_cap=self.gate_cap, norm_state=normalizer.state, writes_state=writes_cache)
        y = ops.gated_group_rmsnorm(o, proj, self.gate_col, ops.GATE_SIGMOID_AFTER, self._norm, self.eps, self.vdim,
                                    proj.dtype)
        return self.dense.forward(y)


register_mixer("lightning_attention", LightningAttention)
register_mixer("mlstm", MatrixLSTM)
