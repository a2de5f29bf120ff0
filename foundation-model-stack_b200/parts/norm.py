"""Norms.  ``RMSNorm``: y = gain * x * rsqrt(mean(x^2) + eps), statistics in float32, eps inside the
root, no mean subtraction, no bias — the reference's ``LayerNormParameterized`` as Llama configures it
(fms/modules/layernorm.py:56-69; fms/models/llama.py:72-87).

Interface of a norm (what a block and the decoder call):

    apply(residual, delta, out_dtype, rows=None) -> normed

``residual`` is the float32 residual stream ``[tokens, dim]``.  ``delta`` (or None) is the previous
sublayer's output, which the norm first adds to the stream in place, in float32: the residual sum and
the norm are one pass over the row.  With ``rows`` only those rows are normed and returned and the
stream is left as it is (used before the output head).

``delta`` may also be a ``NormedDelta``: a sublayer's output that is itself normed before it is added (a layer with a
norm after each sublayer as well as before it).  The adding norm then does both in one kernel:
d = post_norm(delta); residual += d; out = norm(residual), all float32.

``ScalarRMSNorm`` ("rmsnorm_scalar"): y = g * x / sqrt(mean(x^2) + eps) with ONE number g for the whole row (a tensor
without dimensions in the checkpoint).  The number is read once when the weights are loaded and handed to the kernel
by value.

``GroupRMSNorm`` ("group_rmsnorm"): the row in equal consecutive runs, each by its own root mean square, the whole times
the weight; adds several pending outputs with a factor each; ``apply_pair`` gives two norms of the same stream from
one kernel.

``LayerNorm`` ("layernorm"): y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w, no bias.  Option
``layer_scale``: a second vector ``scale`` multiplies the result element by element (the gain the kernel sees is
w * scale, taken in float32 once).  It norms a sublayer's output on its way into the stream (as the ``norm`` of a
``NormedDelta``), and as a norm of the stream itself it adds what is pending and norms the sum in one kernel; with
``mode_and_gain() == None`` in the place of a norm, the same kernel hands the summed stream on in the compute dtype.
"""
from __future__ import annotations

import torch

from ..config.specs import NormSpec
from ..kernels import ops
from .base import Part
from .registry import register_norm


class NormedDelta:
    """A sublayer's output ``delta`` that ``norm`` (an RMS norm of this module) is applied to before it is added to the
    residual stream; the norm that adds it does so."""

    __slots__ = ("delta", "norm")

    def __init__(self, delta, norm) -> None:
        self.delta = delta
        self.norm = norm


class StreamCopy:
    """What a layer hands on when its own norms have already brought the stream up to date (a layer whose norm follows
    the sum): nothing is pending; ``rows`` is the stream in the compute dtype (the stream itself where that is
    float32), so that a next layer that reads the stream need not make that copy again."""

    __slots__ = ("rows",)

    def __init__(self, rows) -> None:
        self.rows = rows


class RMSNorm(Part):
    """Option ``offset``: the stored weight lies around zero and the gain is offset + weight (taken in float32 once,
    when the weights are loaded, so that a weight stored in 16 bits loses nothing in the sum)."""

    def __init__(self, spec: NormSpec) -> None:
        super().__init__()
        self.dim = spec.dim
        self.eps = float(spec.eps)
        self.offset = float(dict(spec.options).get("offset", 0.0))
        self.declare("weight", (spec.dim,), role="vector")
        self._gain = None

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        if self.offset != 0.0:
            self._gain = (self.tensor("weight").float() + self.offset).contiguous()

    def gain_vector(self):
        return self._gain if self._gain is not None else self.tensor("weight")

    def gain(self):
        """(vector or None, the one number where there is no vector, eps): what the fused kernel takes."""
        return self.gain_vector(), 1.0, self.eps

    def apply(self, residual, delta, out_dtype, rows=None):
        if isinstance(delta, StreamCopy):
            delta = None
        if isinstance(delta, NormedDelta):
            return ops.normed_add_rmsnorm(residual, delta.delta, delta.norm.gain(), self.gain(), out_dtype, rows)
        return ops.add_rmsnorm(residual, delta, self.gain_vector(), self.eps, out_dtype, rows)

    def apply_after_sum(self, residual, alpha, parts, out_dtype):
        """residual = norm(alpha * residual + sum of factor * delta over ``parts``), in place; returns the new rows in
        the compute dtype (the stream itself where that is float32)."""
        copy = ops.scaled_add_rmsnorm(residual, alpha, parts, self.gain_vector(), self.eps, out_dtype)
        return residual if copy is None else copy

    def kernel_libraries(self, dtype):
        return ["elementwise"]


class ScalarRMSNorm(Part):
    def __init__(self, spec: NormSpec) -> None:
        super().__init__()
        self.dim = spec.dim
        self.eps = float(spec.eps)
        self.declare("weight", (), role="vector")
        self._gain = None

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        self._gain = float(self.tensor("weight").float().item())

    def gain(self):
        return None, self._gain, self.eps

    def apply(self, residual, delta, out_dtype, rows=None):
        post = None
        if isinstance(delta, StreamCopy):
            delta = None
        if isinstance(delta, NormedDelta):
            delta, post = delta.delta, delta.norm.gain()
        return ops.normed_add_rmsnorm(residual, delta, post, self.gain(), out_dtype, rows)

    def kernel_libraries(self, dtype):
        return ["elementwise"]


class LayerNorm(Part):
    def __init__(self, spec: NormSpec) -> None:
        super().__init__()
        self.dim = spec.dim
        self.eps = float(spec.eps)
        self.layer_scale = bool(dict(spec.options).get("layer_scale", False))
        self.declare("weight", (spec.dim,), role="vector")
        if self.layer_scale:
            self.declare("scale", (spec.dim,), role="vector")
        self._gain = None

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        g = self.tensor("weight").float()
        if self.layer_scale:
            g = g * self.tensor("scale").float()
        self._gain = g.contiguous()

    def mode_and_gain(self):
        """(mode, float32 gain vector, eps): what ``ops.normed_add_norm`` takes for either of its two norms."""
        return ops.NORM_LAYER, self._gain, self.eps

    def add(self, residual, delta, out_dtype):
        """residual += this norm of ``delta`` (a sublayer's output), in float32; returns the stream in ``out_dtype``
        (the stream itself where that is float32)."""
        if out_dtype == torch.float32:
            ops.normed_add_norm(residual, delta, self.mode_and_gain(), None, out_dtype, want_out=False)
            return residual
        return ops.normed_add_norm(residual, delta, self.mode_and_gain(), None, out_dtype)

    def apply(self, residual, delta, out_dtype, rows=None):
        post = None
        if isinstance(delta, StreamCopy):
            delta = None
        if isinstance(delta, NormedDelta):
            if not hasattr(delta.norm, "mode_and_gain"):
                raise ValueError("a layer norm adds a pending output that is normed by a norm with mode_and_gain()")
            delta, post = delta.delta, delta.norm.mode_and_gain()
        return ops.normed_add_norm(residual, delta, post, self.mode_and_gain(), out_dtype, rows)

    def kernel_libraries(self, dtype):
        return ["elementwise"]


class GroupRMSNorm(Part):
    """``group_rmsnorm``: the row is cut into ``groups`` equal consecutive runs (option; 1 by default), each divided by
    its own root mean square (eps inside the root), and the whole multiplied by the weight.  What is pending may be a
    tensor or several outputs with a factor each (an object with ``parts``: [(delta, factor), ...]); the norm adds them
    to the stream in float32 in the pass that norms it.  ``apply_pair`` norms the same stream with this norm and a
    second one of the same kind in one kernel (layers whose sublayers read the same stream side by side)."""

    def __init__(self, spec: NormSpec) -> None:
        super().__init__()
        self.dim = spec.dim
        self.eps = float(spec.eps)
        self.groups = int(dict(spec.options).get("groups", 1))
        if self.groups <= 0 or self.dim % self.groups:
            raise ValueError(f"group_rmsnorm: a row of {self.dim} values in {self.groups} runs")
        self.declare("weight", (spec.dim,), role="vector")
        self._gain = None

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        self._gain = self.tensor("weight").float().contiguous()

    @staticmethod
    def _parts(delta):
        if delta is None or isinstance(delta, StreamCopy):
            return []
        if isinstance(delta, NormedDelta):
            raise ValueError("group_rmsnorm adds plain outputs, not one that is normed on its way")
        return list(delta.parts) if hasattr(delta, "parts") else [(delta, 1.0)]

    def apply(self, residual, delta, out_dtype, rows=None):
        return ops.parts_group_rmsnorm(residual, self._parts(delta), [self._gain], self.eps, self.groups, out_dtype, rows)[0]

    def apply_pair(self, residual, delta, other: "GroupRMSNorm", out_dtype):
        """(this norm of the stream, ``other``'s norm of it), after what is pending has been added."""
        if not isinstance(other, GroupRMSNorm) or (other.eps, other.groups, other.dim) != (self.eps, self.groups, self.dim):
            raise ValueError("apply_pair: two group_rmsnorm norms with the same runs and eps")
        out = ops.parts_group_rmsnorm(residual, self._parts(delta), [self._gain, other._gain], self.eps, self.groups, out_dtype)
        return out[0], out[1]

    def kernel_libraries(self, dtype):
        return ["elementwise"]


register_norm("group_rmsnorm", GroupRMSNorm)
register_norm("layernorm", LayerNorm)
register_norm("rmsnorm", RMSNorm)
register_norm("rmsnorm_scalar", ScalarRMSNorm)
