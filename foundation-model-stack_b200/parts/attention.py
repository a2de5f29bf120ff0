"""Grouped-query softmax attention over the cache: the reference's ``MultiHeadAttention`` with fused
QKV (fms/modules/attention.py:707-943, :622-704).

    qkv = x Wqkv^T (+ b), rows [q heads; k heads; v heads]          attention.py:653-657, :704
    q, k rotated by the position encoding, before caching           attention.py:878-881
    k, v written at each token's position into its slot's blocks    (reference: torch.cat, :186-212)
    o = softmax(q k^T * scale, causal by position, window) v        attention.py:215-294
    y = o Wdense^T (+ b)                                            attention.py:937

Query head h uses key/value head h // (nheads / kvheads).  A token at position p sees the cached
positions p-window+1..p (all of 0..p without a window), whatever else is in the batch and however the
sequence was cut into steps.

Interface of a mixer (what a block calls):

    cache_request() -> KVRequest | StateRequest | None
    forward(x, batch, cache_view, writes_cache) -> y       x, y: [tokens, dim] in the compute dtype
"""
from __future__ import annotations

import math

import torch

from ..cache.requests import KVRequest
from ..config.specs import MixerSpec
from ..kernels import ops
from .base import Part
from .linear import Linear
from .registry import build_position, register_mixer


class MultiHeadAttention(Part):
    def __init__(self, spec: MixerSpec) -> None:
        super().__init__()
        if spec.nheads <= 0 or spec.kvheads <= 0 or spec.nheads % spec.kvheads:
            raise ValueError(f"nheads {spec.nheads} must be a positive multiple of kvheads {spec.kvheads}")
        if spec.head_dim <= 0 or spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"head size {spec.head_dim} is not supported: a multiple of 16 up to 256 is")
        self.spec = spec
        self.nheads, self.kvheads, self.head_dim = spec.nheads, spec.kvheads, spec.head_dim
        self.scale = 1.0 / math.sqrt(spec.head_dim) if spec.scale is None else float(spec.scale)
        self.window = int(spec.window)
        qkv_rows = (spec.nheads + 2 * spec.kvheads) * spec.head_dim
        in_proj = self.add("in_proj", Part())
        self.qkv = in_proj.add("qkv_fused", Linear(spec.dim, qkv_rows, spec.bias))
        self.dense = self.add("dense", Linear(spec.nheads * spec.head_dim, spec.dim, spec.bias))
        # not a child: the encoding has no checkpoint tensors of its own and may be shared
        self.position = build_position(spec.position)
        if self.position.score_bias() is not None:
            raise ValueError(f"position encoding {spec.position.kind!r} adds to the attention scores; the attention "
                             "kernels of this mixer take no such term")

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        self.position.finalize(device, dtype)

    def cache_request(self):
        return KVRequest(self.kvheads, self.head_dim, self.window)

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        # the position part applies the projection, encodes q and k and writes k and v into the cache
        q = self.position.project(x, self.qkv, batch, cache_view, self.nheads, self.kvheads, self.head_dim, writes_cache)
        o = ops.attention(q, batch, cache_view, self.nheads, self.kvheads, self.head_dim, self.scale, self.window)
        return self.dense.forward(o)

    def kernel_libraries(self, dtype):
        return (super().kernel_libraries(dtype) + self.position.kernel_libraries(dtype)
                + ["elementwise", f"attention_hd{self.head_dim}"])


class SinkAttention(Part):
    """``sink_attention``: grouped-query softmax attention over the cache with, each of them optional,

        rotation of only the first ``rot_dims`` values of every head (adjacent pairs; ``position`` gives base and scaling;
            ``pairing`` "halves": value i turns with value i + rot_dims / 2 instead)
        q and k divided by their root mean square over the head, after the rotation (``qk_norm``, eps ``eps``; no gain);
            ``qk_norm`` "before": the norm comes before the rotation and has gains ``q_norm`` and ``k_norm`` [head_dim],
            each shared by all heads
        a learned sink per head in the softmax's denominator: p_j = exp(s_j) / (sum_i exp(s_i) + exp(sink_h))   (``sink``);
            ``sink_logit``: a fixed number in the place of the learned ones (0.0: one added to the denominator)
        a gate on the heads' results before the output projection: o * sigmoid(Wg h) (``gate``), one gate a value, or
            with ``gate`` "head" one a head
        values of another size than keys (``vdim``); ``values`` "keys": no value projection, a value is its key as
            projected, before norm and rotation
        keys seen in runs (``chunk`` = n: the positions of a sequence are cut into runs of n, counted from its position 0,
            and a query sees the keys of its own run up to itself; instead of a window)
        capped scores (``softcap`` = c: s becomes c * tanh(s / c) after the scale)
        a bias on the output projection (``out_bias``)
        frequencies stretched by a ramp ("yarn" scaling of ``position``): the sines and cosines are then also multiplied
            by the constant that belongs to it

    [Wq; Wk; Wv; Wg] is one fused projection (``in_proj``; bias [bq; bk; bv; 0] where ``bias``; without Wv where the
    values are the keys; its rows filled up with zeros to a multiple of 8 where the gates are one a head).  The cache holds heads
    of ``pad`` = max(head_dim, vdim) rounded up to 16 values, zeros beyond each one's own size, so that the attention
    kernels built for one head size serve keys and values alike; q is padded the same way and the padding of the
    result is dropped by the gate kernel.  ``out_factor`` multiplies the result before the output projection (a mixer
    that stands beside another one carries its weight there)."""

    def __init__(self, spec: MixerSpec) -> None:
        super().__init__()
        o = dict(spec.options)
        if spec.nheads <= 0 or spec.kvheads <= 0 or spec.nheads % spec.kvheads:
            raise ValueError(f"nheads {spec.nheads} must be a positive multiple of kvheads {spec.kvheads}")
        self.nheads, self.kvheads, self.head_dim = spec.nheads, spec.kvheads, spec.head_dim
        self.vdim = int(o.get("vdim", spec.head_dim))
        self.pad = (max(self.head_dim, self.vdim) + 15) // 16 * 16
        if self.head_dim <= 0 or self.vdim <= 0 or self.pad > 256:
            raise ValueError(f"sink_attention: heads of {self.head_dim} and values of {self.vdim}: up to 256 are supported")
        self.rot_dims = int(o.get("rot_dims", 0))
        if self.rot_dims % 2 or not (0 <= self.rot_dims <= self.head_dim):
            raise ValueError(f"sink_attention: {self.rot_dims} rotated values of {self.head_dim}")
        self.qk_norm, self.eps = bool(o.get("qk_norm", False)), float(o.get("eps", 1e-6))
        self.norm_first = o.get("qk_norm") == "before"
        self.halves = o.get("pairing", "adjacent") == "halves"
        if o.get("pairing", "adjacent") not in ("adjacent", "halves") or o.get("values", "projected") not in ("projected", "keys"):
            raise ValueError(f"sink_attention: pairing {o.get('pairing')!r}, values {o.get('values')!r}")
        self.values_are_keys = o.get("values", "projected") == "keys"
        if self.values_are_keys and self.vdim != self.head_dim:
            raise ValueError(f"sink_attention: values that are the keys have their size, {self.head_dim}, not {self.vdim}")
        self.sink_logit = None if o.get("sink_logit") is None else float(o["sink_logit"])
        self.has_sink, self.has_gate = bool(o.get("sink", False)), bool(o.get("gate", False))
        self.gate_per_head = o.get("gate") == "head"
        if self.has_sink and self.sink_logit is not None:
            raise ValueError("sink_attention: either learned sinks or one fixed logit")
        self.out_factor = float(o.get("out_factor", 1.0))
        self.scale = 1.0 / math.sqrt(spec.head_dim) if spec.scale is None else float(spec.scale)
        self.window = int(spec.window)
        self.chunk, self.softcap = int(o.get("chunk", 0)), float(o.get("softcap", 0.0))
        if self.chunk < 0 or self.softcap < 0 or (self.chunk and self.window):
            raise ValueError(f"sink_attention: chunk {self.chunk}, window {self.window}, softcap {self.softcap}")
        self.rot_mult = 1.0
        self.position_spec = spec.position
        self.gate_col = (self.nheads + self.kvheads) * self.head_dim + (0 if self.values_are_keys else self.kvheads * self.vdim)
        rows = self.fused_rows(self.nheads, self.kvheads, self.head_dim, self.vdim, self.values_are_keys,
                               o.get("gate", False))
        self.in_proj = self.add("in_proj", Linear(spec.dim, rows, spec.bias))
        if self.has_sink:
            self.declare("sink", (self.nheads,), role="vector")
        if self.norm_first:
            self.declare("q_norm", (self.head_dim,), role="vector")
            self.declare("k_norm", (self.head_dim,), role="vector")
        self.dense = self.add("dense", Linear(self.nheads * self.vdim, spec.dim, bool(o.get("out_bias", False))))
        self._inv_freq = self._sink = self._q_gain = self._k_gain = None

    @staticmethod
    def fused_rows(nheads: int, kvheads: int, head_dim: int, vdim: int, values_are_keys: bool, gate) -> int:
        """Rows of the fused projection [q; k; v; g]: what a checkpoint adapter has to put together."""
        rows = (nheads + kvheads) * head_dim + (0 if values_are_keys else kvheads * vdim)
        if gate == "head":
            return (rows + nheads + 7) // 8 * 8
        return rows + (nheads * vdim if gate else 0)

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        if self.rot_dims:
            from .position import rotary_inverse_frequencies, rotary_multiplier

            # every frequency in float64, rounded to float32 once
            f = rotary_inverse_frequencies(self.rot_dims, float(self.position_spec.theta), self.position_spec.scaling_dict(),
                                           dtype=torch.float64)
            self._inv_freq = f.to(torch.float32).to(device).contiguous()
            self.rot_mult = rotary_multiplier(self.position_spec.scaling_dict())
        if self.has_sink:
            self._sink = self.tensor("sink").float().contiguous()
        elif self.sink_logit is not None:
            self._sink = torch.full((self.nheads,), self.sink_logit, dtype=torch.float32, device=device)
        if self.norm_first:
            self._q_gain = self.tensor("q_norm").float().contiguous()
            self._k_gain = self.tensor("k_norm").float().contiguous()

    def cache_request(self):
        return KVRequest(self.kvheads, self.pad, self.window)

    def heads_out(self, x, batch, cache_view, writes_cache: bool = True):
        """The gated heads' results [tokens, nheads * vdim], before the output projection."""
        proj = self.in_proj.forward(x)
        q = ops.qk_prepare_store(proj, self._inv_freq, self.rot_dims, self.qk_norm, self.eps, batch, cache_view,
                                 self.nheads, self.kvheads, self.head_dim, self.vdim, self.pad, writes_cache,
                                 norm_first=self.norm_first, q_gain=self._q_gain, k_gain=self._k_gain, halves=self.halves,
                                 values_are_keys=self.values_are_keys, rot_mult=self.rot_mult)
        o = ops.attention(q, batch, cache_view, self.nheads, self.kvheads, self.pad, self.scale, self.window, self._sink,
                          chunk=self.chunk, softcap=self.softcap)
        if not self.has_gate and self.pad == self.vdim and self.out_factor == 1.0:
            return o  # no gate, no padding to drop, no factor: the heads' results as attention left them
        return ops.sigmoid_gate(o, proj if self.has_gate else None, self.gate_col, self.nheads, self.vdim, self.pad,
                                self.out_factor, self.gate_per_head)

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        return self.dense.forward(self.heads_out(x, batch, cache_view, writes_cache))

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["elementwise", f"attention_hd{self.pad}"]


register_mixer("attention", MultiHeadAttention)
register_mixer("sink_attention", SinkAttention)
