"""The operations a decoder step is made of, each a call into a hand-written CUDA kernel.

Tensors are torch tensors on a CUDA device (torch is used for memory and for the library matrix
product only); every function launches on torch's current stream.  There is no CPU implementation and
no fallback: a tensor on another device, a missing compiler or a failed build raises.

Matrix products: float32 runs ``gemm_f32`` (FFMA, no tensor-core mode).  bfloat16 runs the weight-streaming
``mma.sync`` kernel up to 8 rows (decode of few sequences) and otherwise the library product (cuBLAS through
``torch.nn.functional.linear``), as the reference does for every linear layer (fms/modules/linear.py:119-156) —
except the gated feed-forward product, which from ``TENSOR_CORE_ROWS_GLU`` (512) rows on, where its tiles of 256
rows fit the number of rows to 6%, takes the tcgen05 kernel
with the tokens on the instruction's rows (prefill; pairs of thread blocks on one tile, the activation in its
epilogue), and the fused projection of queries, keys and values, which from ``TENSOR_CORE_ROWS_QKV`` (2,048) rows
on takes the same kernel with the rotation and the cache write in its epilogue.  The same kernel takes the plain
products from ``FMS_B200_TC_ROWS`` rows on where that is set; measured through whole prefills the library's plain
products are ahead, so by default it is not.
The gated feed-forward product of 9 to 128 rows takes a tcgen05 kernel of this library with the weights on the
instruction's rows and the activation in its epilogue (``gemm_bf16_mid.cu``); the same kernel can take the plain
products and the fused projection up to 256 rows (clusters of blocks share a tile along K; projection + rotation
+ cache write in its epilogue; ``FMS_B200_MID_OPS``), where the library's product is still ahead of it.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_P, _I, _F, _U64, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_ulonglong, ctypes.c_long

_SIGNATURES = {
    "fms_embed_rows": [_P, _I, _P, _P, _I, _I, _I, _F, _P, _P],
    "fms_add_rmsnorm": [_P, _P, _P, _I, _F, _P, _I, _P, _I, _I, _I, _P],
    "fms_gated_activation": [_P, _P, _I, _I, _I, _I, _P],
    "fms_rope_store": [_P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _I, _I, _P],
    "fms_decode_advance": [_P, _P, _P, _P, _P, _I, _I, _P],
    "fms_rotary_table": [_P, _P, _P, _P, _I, _I, _P],
    "fms_gemm_f32": [_P, _P, _P, _P, _I, _I, _I, _P],
    "fms_linear_bf16_skinny": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    "fms_glu_bf16_skinny": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    "fms_qkv_rope_store_bf16_skinny": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P,
                                       _I, _I, _I, _P],
    "fms_linear_bf16_mid": [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "fms_glu_bf16_mid": [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "fms_qkv_rope_store_bf16_mid": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P,
                                    _I, _I, _I, _P],
    "fms_gemm_bf16_tc": [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "fms_glu_bf16_tc": [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "fms_qkv_rope_store_bf16_tc": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P,
                                   _I, _I, _I, _P],
    "fms_embed_pair_hash": [_P, _P, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _F, _I, _I, _I, _P, _P],
    "fms_normed_add_rmsnorm": [_P, _P, _I, _P, _F, _F, _P, _F, _F, _I, _P, _I, _P, _I, _I, _I, _P],
    "fms_mingru_scan": [_P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _I, _P, _P],
    "fms_grouped_linear": [_P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _I, _F, _F, _I, _P],
    "fms_route": [_P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _F, _P],
    "fms_route_gather": [_P, _I, _P, _P, _I, _I, _I, _P, _P],
    "fms_relu_squared": [_P, _I, _L, _P],
    "fms_gated_clamped": [_P, _P, _I, _I, _I, _F, _F, _P],
    "fms_latent_attention_prefill_bf16": [_P, _P, _P, _P, _L, _P, _I, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                                          _F, _I, _I, _I, _P, _I, _P, _P, _I, _P],
    "fms_latent_prepare": [_P, _I, _I, _P, _P, _I, _F, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I,
                           _I, _I, _P, _I, _F, _P, _I, _P],
    "fms_latent_query_norm": [_P, _I, _I, _I, _P, _I, _F, _P, _I, _P],
    "fms_latent_attention": [_P, _P, _I, _P, _P, _L, _P, _I, _P, _I, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _F, _I,
                             _I, _I, _I, _P],
    "fms_scaled_add_rmsnorm": [_P, _F, _P, _F, _P, _F, _P, _I, _F, _P, _I, _I, _I, _P],
    "fms_cast_rows": [_P, _P, _I, _L, _P],
    "fms_parts_group_rmsnorm": [_P, _P, _F, _P, _F, _P, _F, _P, _F, _P, _P, _F, _I, _P, _P, _I, _P, _I, _I, _I, _P],
    "fms_qk_prepare_store": [_P, _I, _I, _P, _P, _I, _F, _I, _F, _P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I,
                             _I, _I, _I, _I, _I, _P, _I, _I, _I, _P],
    "fms_sigmoid_gate": [_P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _P],
    "fms_normed_add_norm": [_P, _P, _I, _P, _F, _I, _P, _F, _P, _I, _P, _I, _I, _I, _P],
    "fms_linear_prepare": [_P, _I, _I, _P, _I, _I, _I, _F, _I, _P],
    "fms_decay_scan": [_P, _P, _I, _I, _P, _F, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "fms_attention_prefill_sink": [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P,
                                   _P],
    "fms_attention_prefill_masked": [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P,
                                     _I, _F, _P],
    "fms_attention_decode_masked": [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _F, _I, _I, _I, _L,
                                    _P, _P, _P, _I, _F, _P],
    "fms_attention_decode_sink": [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _F, _I, _I, _I, _L,
                                  _P, _P, _P, _P],
    "fms_causal_conv": [_P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "fms_selective_scan": [_P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "fms_delta_rule_scan": [_P, _P, _I, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "fms_gated_group_rmsnorm": [_P, _P, _I, _I, _I, _P, _I, _F, _F, _P, _I, _I, _I, _P],
    "fms_argmax": [_P, _P, _I, _I, _P],
    "fms_sample": [_P, _P, _I, _I, _F, _I, _U64, _P, _I, _P],
    "fms_attention_prefill": [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P],
    "fms_attention_decode": [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _F, _I, _I, _I, _L, _P, _P,
                             _P],
}
_functions = {}
# kernels launched through this module since import (a decode-attention call over several splits launches two)
launches = 0


class KernelError(RuntimeError):
    pass


def _fn(library: str, name: str):
    key = (library, name)
    f = _functions.get(key)
    if f is None:
        lib = load_library(library)
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = ctypes.c_int
        _functions[key] = f = (f, lib)
    return f


def _call(library: str, name: str, *args):
    global launches
    f, lib = _fn(library, name)
    launches += 1
    rc = f(*args)
    if rc != 0:
        raise KernelError(f"{name}: {lib.fms_last_error().decode(errors='replace')}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (the direct getter where torch has it: a step makes some hundred launches)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dtype} has no kernel: float32 and bfloat16 have")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a tensor on the CPU reached a CUDA kernel; this library has no CPU path")
    if not t.is_contiguous():
        raise KernelError("a non-contiguous tensor reached a CUDA kernel")
    return t.data_ptr()


_error_flags = {}


def error_flag(device) -> torch.Tensor:
    """An int32 on the device that kernels set when they meet what the host should have prevented (a token
    id outside the vocabulary, a position without a cache block).  ``check_error_flag`` reads it."""
    device = torch.device(device)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


_work_counters = {}
WORK_COUNTERS = 4096


def _work_counter(device) -> torch.Tensor:
    """An int32 on the device that is 0 between launches: the persistent decode-attention kernel's warps draw
    their units from it, and the kernel that merges the splits puts it back.  Every call hands out the next of
    4,096, so that launches in flight at the same time (other streams, the launches inside captured graphs) do
    not share one."""
    device = torch.device(device)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _work_counters:
        _work_counters[key] = [torch.zeros(WORK_COUNTERS, dtype=torch.int32, device=device), 0]
    entry = _work_counters[key]
    entry[1] = (entry[1] + 1) % WORK_COUNTERS
    return entry[0][entry[1]:entry[1] + 1]


def check_error_flag(device) -> None:
    """Raises if a kernel met something the host should have prevented; in a bounds-checked build
    (FMS_B200_DEBUG_BOUNDS=1) also if any kernel computed an index outside its array.  Synchronises."""
    flag = error_flag(device)
    v = int(flag.item())
    from .build import bounds_violations

    outside = bounds_violations()
    if outside:
        raise KernelError("bounds-checked build: " + "; ".join(outside))
    if v:
        flag.zero_()
        raise KernelError({1: "a token id outside the vocabulary reached the embedding",
                           2: "a token's position has no cache block",
                           4: "a kernel gave up waiting for a copy or for the tensor cores",
                           8: "decode attention was launched with fewer key splits than a sequence's length needs",
                           16: "a kernel's bounds check met an index outside its array"}.get(v, f"device error flag {v}"))


# ---- embedding ---------------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Float32 rows of ``table`` at ``tokens``, times ``scale``: the start of the residual stream."""
    n, dim = tokens.shape[0], table.shape[1]
    out = torch.empty((n, dim), dtype=torch.float32, device=table.device)
    _call("elementwise", "fms_embed_rows", _ptr(table), _code(table.dtype), _ptr(tokens), _ptr(out), n, dim,
          table.shape[0], float(scale), _ptr(error_flag(table.device)), _stream())
    return out


def embed_pair_hash(table: torch.Tensor, pairs: torch.Tensor, batch, last_token: torch.Tensor, buckets: int,
                    mul_prev: int, mul_cur: int, scale: float = 1.0) -> torch.Tensor:
    """Float32 rows table[token] + pairs[(previous * mul_prev + token * mul_cur) mod buckets] (pairs[buckets] for the
    token at place 0 of its sequence), times ``scale``.  ``last_token`` [slots, 1] int32 is each sequence's last
    token so far: read for a step's first row, then set to the step's last token."""
    n, dim = batch.tokens.shape[0], table.shape[1]
    if pairs.dtype != table.dtype or pairs.shape != (buckets + 1, dim) or last_token.dtype != torch.int32:
        raise KernelError("embed_pair_hash: the pair table has the token table's dtype and buckets + 1 rows of its width; "
                          "the state is int32")
    out = torch.empty((n, dim), dtype=torch.float32, device=table.device)
    _call("elementwise", "fms_embed_pair_hash", _ptr(table), _ptr(pairs), _code(table.dtype), _ptr(batch.tokens),
          _ptr(batch.positions), _ptr(batch.token_seq), _ptr(batch.first_row), _ptr(batch.slots), _ptr(last_token),
          _ptr(out), n, dim, table.shape[0], int(buckets), int(mul_prev), int(mul_cur), float(scale), 1,
          batch.slots.shape[0], last_token.shape[0], _ptr(error_flag(table.device)), _stream())
    return out


# ---- norm --------------------------------------------------------------------------------------------
def normed_add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], post, gain, out_dtype: torch.dtype,
                       rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual (float32, in place) += post_norm(delta); returns norm(residual) in ``out_dtype``.  ``post`` and ``gain``
    are (vector or None, number, eps): an RMS norm's gain as a vector of the row's width or as one number.  ``post``
    None adds delta as it is.  With ``rows`` only those rows are computed and the residual is not written."""
    dim = residual.shape[1]
    n = rows.shape[0] if rows is not None else residual.shape[0]
    if residual.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    if delta is not None and delta.dtype != out_dtype:
        raise KernelError(f"sublayer output is {delta.dtype}, compute dtype is {out_dtype}")
    post_vec, post_num, post_eps = post if post is not None else (None, 1.0, 0.0)
    gain_vec, gain_num, eps = gain
    vecs = [v for v in (post_vec, gain_vec) if v is not None]
    if len({v.dtype for v in vecs}) > 1:
        raise KernelError("normed_add_rmsnorm: the two gain vectors differ in dtype")
    out = torch.empty((n, dim), dtype=out_dtype, device=residual.device)
    _call("elementwise", "fms_normed_add_rmsnorm", _ptr(residual), _ptr(delta), 0 if post is None else 1, _ptr(post_vec),
          float(post_num), float(post_eps), _ptr(gain_vec), float(gain_num), float(eps),
          _code(vecs[0].dtype) if vecs else F32, _ptr(out), _code(out_dtype), _ptr(rows), n, dim, residual.shape[0],
          _stream())
    return out


NORM_NONE, NORM_RMS, NORM_LAYER = 0, 1, 2


def normed_add_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], post, out_norm, out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None, want_out: bool = True) -> Optional[torch.Tensor]:
    """residual (float32, in place) += post(delta); returns out_norm(residual) in ``out_dtype``.  ``post`` and
    ``out_norm`` are (mode, gain, eps) with mode ``NORM_NONE`` (the rows as they are), ``NORM_RMS`` or ``NORM_LAYER``
    (the mean taken off, the variance the mean of the squared deviations, no bias) and gain a float32 vector of the
    row's width (None with ``NORM_NONE``).  With ``rows`` only those rows are computed and the residual is not written.
    ``want_out`` False: only the sum is wanted and nothing is returned."""
    dim = residual.shape[1]
    n = rows.shape[0] if rows is not None else residual.shape[0]
    if residual.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    if delta is not None and delta.dtype != out_dtype:
        raise KernelError(f"sublayer output is {delta.dtype}, compute dtype is {out_dtype}")
    post_mode, post_gain, post_eps = post if post is not None else (NORM_NONE, None, 0.0)
    out_mode, gain, eps = out_norm if out_norm is not None else (NORM_NONE, None, 0.0)
    for g in (post_gain, gain):
        if g is not None and (g.dtype != torch.float32 or g.shape[0] != dim):
            raise KernelError("normed_add_norm: gains are float32 vectors of the row's width")
    out = torch.empty((n, dim), dtype=out_dtype, device=residual.device) if want_out else None
    _call("elementwise", "fms_normed_add_norm", _ptr(residual), _ptr(delta), int(post_mode), _ptr(post_gain), float(post_eps),
          int(out_mode), _ptr(gain), float(eps), _ptr(out), _code(out_dtype), _ptr(rows), n, dim, residual.shape[0], _stream())
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual (float32, in place) += delta; returns gain * rmsnorm(residual) in ``out_dtype``.  With
    ``rows`` only those rows are computed and the residual is not written."""
    dim = residual.shape[1]
    n = rows.shape[0] if rows is not None else residual.shape[0]
    if residual.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    if delta is not None and delta.dtype != out_dtype:
        raise KernelError(f"sublayer output is {delta.dtype}, compute dtype is {out_dtype}")
    out = torch.empty((n, dim), dtype=out_dtype, device=residual.device)
    _call("elementwise", "fms_add_rmsnorm", _ptr(residual), _ptr(delta), _ptr(gain), _code(gain.dtype), float(eps),
          _ptr(out), _code(out_dtype), _ptr(rows), n, dim, residual.shape[0], _stream())
    return out


def scaled_add_rmsnorm(residual: torch.Tensor, alpha: float, parts, gain: torch.Tensor, eps: float,
                       out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """The norm that follows the residual sum: residual (float32, in place) = gain * rmsnorm(alpha * residual +
    sum of factor * delta over ``parts``, a list of one or two (delta, factor)).  Returns the new rows in ``out_dtype``
    too, or None where that is float32 (the stream itself then serves)."""
    n, dim = residual.shape
    if residual.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    if not 1 <= len(parts) <= 2 or any(d.dtype != out_dtype or tuple(d.shape) != (n, dim) for d, _ in parts):
        raise KernelError("scaled_add_rmsnorm: one or two sublayer outputs of the stream's shape, in the compute dtype")
    (da, sa), (db, sb) = parts[0], (parts[1] if len(parts) > 1 else (None, 0.0))
    copy = None if out_dtype == torch.float32 else torch.empty((n, dim), dtype=out_dtype, device=residual.device)
    _call("elementwise", "fms_scaled_add_rmsnorm", _ptr(residual), float(alpha), _ptr(da), float(sa), _ptr(db), float(sb),
          _ptr(gain), _code(gain.dtype), float(eps), _ptr(copy), _code(out_dtype), n, dim, _stream())
    return copy


def parts_group_rmsnorm(residual: torch.Tensor, parts, gains, eps: float, groups: int, out_dtype: torch.dtype,
                        rows: Optional[torch.Tensor] = None):
    """residual (float32, in place) += sum of factor * delta over ``parts`` (up to four (delta, factor), deltas in
    ``out_dtype``); then the row in ``groups`` equal consecutive runs, each divided by its own root mean square, and
    one output per entry of ``gains`` (one or two float32 vectors of the row's width): the normed row times that gain,
    in ``out_dtype``.  Two norms of the same stream so share one pass and one set of statistics.  With ``rows`` only
    those rows are computed and the residual is not written.  Returns the list of outputs."""
    dim = residual.shape[1]
    n = rows.shape[0] if rows is not None else residual.shape[0]
    parts = [(d, float(f)) for d, f in (parts or []) if d is not None]
    if residual.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    if len(parts) > 4 or any(d.dtype != out_dtype or tuple(d.shape) != tuple(residual.shape) for d, _ in parts):
        raise KernelError("parts_group_rmsnorm: up to four sublayer outputs of the stream's shape, in the compute dtype")
    if not 1 <= len(gains) <= 2 or any(g.dtype != torch.float32 or g.shape[0] != dim for g in gains):
        raise KernelError("parts_group_rmsnorm: one or two float32 gains of the row's width")
    outs = [torch.empty((n, dim), dtype=out_dtype, device=residual.device) for _ in gains]
    flat = []
    for i in range(4):
        flat += [_ptr(parts[i][0]), parts[i][1]] if i < len(parts) else [None, 0.0]
    _call("elementwise", "fms_parts_group_rmsnorm", _ptr(residual), *flat, _ptr(gains[0]),
          _ptr(gains[1]) if len(gains) > 1 else None, float(eps), int(groups), _ptr(outs[0]),
          _ptr(outs[1]) if len(outs) > 1 else None, _code(out_dtype), _ptr(rows), n, dim, residual.shape[0], _stream())
    return outs


def cast_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Float32 rows in ``dtype`` (the same tensor where that is float32)."""
    if dtype == torch.float32:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _call("elementwise", "fms_cast_rows", _ptr(x), _ptr(out), _code(dtype), x.numel(), _stream())
    return out


# ---- linear ------------------------------------------------------------------------------------------
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [rows, in] times weight [out, in] transposed (+ bias).  ``out_dtype`` defaults to x's dtype."""
    out_dtype = out_dtype or x.dtype
    _ptr(x), _ptr(weight)
    if weight.dtype == torch.float32:
        # true float32: also taken by a float32-stored matrix inside a bfloat16 model
        x32 = x if x.dtype == torch.float32 else x.float()
        b32 = None if bias is None else (bias if bias.dtype == torch.float32 else bias.float())
        y = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        _call("gemm_f32", "fms_gemm_f32", _ptr(x32), _ptr(weight), _ptr(b32), _ptr(y), x.shape[0], weight.shape[0],
              weight.shape[1], _stream())
        return y if out_dtype == torch.float32 else y.to(out_dtype)
    if weight.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
        raise KernelError(f"linear: x {x.dtype}, weight {weight.dtype}")
    if x.shape[0] <= SKINNY_ROWS and weight.shape[1] % 8 == 0 and (bias is None or bias.dtype == torch.bfloat16):
        # few rows (decode): the weight-streaming tensor-core kernel
        y = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
        _call("gemm_bf16_skinny", "fms_linear_bf16_skinny", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _code(out_dtype),
              x.shape[0], weight.shape[0], weight.shape[1], _stream())
        return y
    if _mid_fits(x, weight, bias):
        y = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
        _call("gemm_bf16_mid", "fms_linear_bf16_mid", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _code(out_dtype),
              x.shape[0], weight.shape[0], weight.shape[1], _ptr(error_flag(x.device)), _stream())
        return y
    if _tensor_core_fits(x, weight, bias):
        return linear_tensor_core(x, weight, bias, out_dtype)
    if out_dtype == torch.float32:
        y = torch.mm(x, weight.t(), out_dtype=torch.float32)
        return y if bias is None else y + bias.float()
    b = None if bias is None else bias.to(torch.bfloat16)
    return torch.nn.functional.linear(x, weight, b)


# Rows from which the tcgen05 kernel with the tokens on the instruction's rows (gemm_bf16_tc.cu) is used instead of the
# library's product.  Measured through whole prefills at the 8B sizes (ms; library for everything / own gated product
# only / own for everything).  The policies taking turns in one warmed-up process: 1,100 tokens 15.4 / 16.4 / 19.6;
# 2,048 tokens 27.5 / 27.5 / 27.5; 4,096 tokens 56.0 / 54.8 / 54.9.  Each in a process of its own: 512 tokens 8.0 /
# 7.8 / 7.8; 1,024 tokens 14.8 / 12.8 / -; 1,280 tokens 17.7 / 17.6 / 19.1; 8,192 tokens 117.0 / 118.7 / 123.2.  The
# own kernel works on tiles of 256 rows, so it loses where the last tile is mostly padding (1,100 rows: a sixth is).
# So the gated product, whose activation the own kernel has in its epilogue, takes the own kernel from 512 rows on
# where at most 6% of the computed rows are padding, and everything else stays with the library unless
# FMS_B200_TC_ROWS / FMS_B200_TC_ROWS_GLU / FMS_B200_TC_MAX_PADDING say otherwise (both row limits were 1,024 once, which
# cost prompts of 1,025 to 1,800 tokens up to a quarter of their time).
TENSOR_CORE_ROWS = int(os.environ.get("FMS_B200_TC_ROWS", str(1 << 30)))
TENSOR_CORE_ROWS_GLU = int(os.environ.get("FMS_B200_TC_ROWS_GLU", "512"))
# The projection with the rotation and the cache write in the own kernel's epilogue, against the library's product and
# the rotation kernel after it, whole prefills in processes of their own (ms, fused / two kernels): 1,024 tokens 14.5 /
# 14.1; 2,048 tokens 26.5 / 26.6; 3,000 tokens 40.0 / 41.0; 4,096 tokens 53.3 / 54.3; 8,192 tokens 121.2 / 120.1.
TENSOR_CORE_ROWS_QKV = int(os.environ.get("FMS_B200_TC_ROWS_QKV", "2048"))
TENSOR_CORE_MAX_PADDING = float(os.environ.get("FMS_B200_TC_MAX_PADDING", "1.06"))  # rows computed over rows asked for
USE_TENSOR_CORE_GEMM = os.environ.get("FMS_B200_TC_GEMM", "1") != "0"


# The tcgen05 kernel with the weights on the instruction's rows (gemm_bf16_mid.cu), for SKINNY_ROWS + 1 to MID_ROWS
# rows.  By default it takes the gated feed-forward product up to 128 rows, where it is ahead of the library's
# product followed by the activation kernel (a decode step of batch 16 at the 8B sizes: 3.75 against 3.86 ms; batch 32:
# 4.59 against 4.66; batch 64: at par; batch 96: 6.80 against 6.90; batch 128: 7.89 against 7.93; batch 256: 13.70
# against 12.99, hence no further).  The plain products and the fused projection, whose matrices have too few
# rows for one block a tile and so run as clusters that add their sums, are 3 to 9 us a product behind the library
# (batch 16: 4.02 ms with them, batch 64: 6.47) and stay with it unless FMS_B200_MID_OPS names them
# ("linear,glu,qkv"; FMS_B200_MID_ROWS up to 256; FMS_B200_MID_GEMM=0 turns the kernel off).
MID_ROWS = min(256, int(os.environ.get("FMS_B200_MID_ROWS", "128")))
USE_MID_GEMM = os.environ.get("FMS_B200_MID_GEMM", "1") != "0"
MID_OPS = os.environ.get("FMS_B200_MID_OPS", "glu").split(",")


def _mid_fits(x, weight, bias, op: str = "linear") -> bool:
    return (USE_MID_GEMM and op in MID_OPS and SKINNY_ROWS < x.shape[0] <= MID_ROWS and weight.shape[1] % 8 == 0
            and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and (bias is None or bias.dtype == torch.bfloat16))


def _tensor_core_fits(x, weight, bias, rows_from: Optional[int] = None) -> bool:
    rows_from = TENSOR_CORE_ROWS if rows_from is None else rows_from
    return (USE_TENSOR_CORE_GEMM and x.shape[0] >= rows_from and weight.shape[1] % 8 == 0
            and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and (bias is None or bias.dtype == torch.bfloat16))


def linear_tensor_core(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                       out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The product on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory): bfloat16 in, bfloat16 or
    float32 out.  K must be a multiple of 8."""
    out_dtype = out_dtype or x.dtype
    y = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
    _call("gemm_bf16_tc", "fms_gemm_bf16_tc", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _code(out_dtype), x.shape[0],
          weight.shape[0], weight.shape[1], _ptr(error_flag(x.device)), _stream())
    return y


def gated_linear_tensor_core(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                             activation: int) -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) in one tcgen05 kernel: gate and up rows share a tile, the epilogue multiplies."""
    hidden = weight.shape[0] // 2
    y = torch.empty((x.shape[0], hidden), dtype=torch.bfloat16, device=x.device)
    _call("gemm_bf16_tc", "fms_glu_bf16_tc", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), x.shape[0], hidden,
          weight.shape[1], int(activation), _ptr(error_flag(x.device)), _stream())
    return y


SKINNY_ROWS = 8  # rows up to which the weight-streaming kernels are used (more rows re-read x too often)


# ---- feed-forward ------------------------------------------------------------------------------------
def gated_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], activation: int) -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) for weight = [Wg; Wu]: one kernel for few bfloat16 rows, else the product
    followed by ``gated_activation``."""
    hidden = weight.shape[0] // 2
    if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_ROWS
            and weight.shape[1] % 8 == 0 and (bias is None or bias.dtype == torch.bfloat16)):
        _ptr(x), _ptr(weight)
        y = torch.empty((x.shape[0], hidden), dtype=torch.bfloat16, device=x.device)
        _call("gemm_bf16_skinny", "fms_glu_bf16_skinny", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), x.shape[0], hidden,
              weight.shape[1], int(activation), _stream())
        return y
    if _mid_fits(x, weight, bias, "glu"):
        _ptr(x), _ptr(weight)
        y = torch.empty((x.shape[0], hidden), dtype=torch.bfloat16, device=x.device)
        _call("gemm_bf16_mid", "fms_glu_bf16_mid", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), x.shape[0], hidden,
              weight.shape[1], int(activation), _ptr(error_flag(x.device)), _stream())
        return y
    # the own kernel works on tiles of 256 rows: where the last one would be mostly padding, the library is ahead
    if (_tensor_core_fits(x, weight, bias, TENSOR_CORE_ROWS_GLU)
            and (x.shape[0] + 255) // 256 * 256 <= TENSOR_CORE_MAX_PADDING * x.shape[0]):
        return gated_linear_tensor_core(x, weight, bias, activation)
    return gated_activation(linear(x, weight, bias), activation)


def gated_activation(gate_up: torch.Tensor, activation: int) -> torch.Tensor:
    """act(gate) * up for rows [gate | up]."""
    n, two_f = gate_up.shape
    hidden = two_f // 2
    out = torch.empty((n, hidden), dtype=gate_up.dtype, device=gate_up.device)
    _call("elementwise", "fms_gated_activation", _ptr(gate_up), _ptr(out), _code(gate_up.dtype), n, hidden,
          int(activation), _stream())
    return out


# ---- attention ---------------------------------------------------------------------------------------
def rope_store(qkv: torch.Tensor, inv_freq: Optional[torch.Tensor], batch, view, nheads: int, kvheads: int,
               head_dim: int, writes_cache: bool = True) -> torch.Tensor:
    """Rotates q and k of ``qkv`` [tokens, (nheads + 2 kvheads) head_dim] by each token's position, writes k
    and v into the cache at the token's slot and place, returns the rotated q [tokens, nheads head_dim].  The
    rotation sees ``batch.position_ids`` where the batch has them (sequences that did not start at position 0),
    else the token's place in the cache, ``batch.positions``; ``inv_freq`` None rotates nothing."""
    n = qkv.shape[0]
    if view.keys.dtype != qkv.dtype:
        raise KernelError(f"cache is {view.keys.dtype}, activations are {qkv.dtype}")
    q = torch.empty((n, nheads * head_dim), dtype=qkv.dtype, device=qkv.device)
    _call("elementwise", "fms_rope_store", _ptr(qkv), _code(qkv.dtype), _ptr(q), _ptr(inv_freq), _ptr(batch.positions),
          _ptr(getattr(batch, "position_ids", None)), _ptr(batch.token_seq), _ptr(batch.slots), _ptr(view.keys),
          _ptr(view.values), _ptr(view.table),
          view.table.shape[1], view.block_tokens, n, nheads, kvheads, head_dim, 1 if writes_cache else 0,
          _ptr(error_flag(qkv.device)), batch.slots.shape[0], view.table.shape[0], view.keys.shape[0], _stream())
    return q


FUSE_QKV_ROPE = os.environ.get("FMS_B200_FUSE_QKV_ROPE", "1") != "0"


def rotary_table(inv_freq: torch.Tensor, batch) -> torch.Tensor:
    """[tokens, head_dim / 2, 2] float32: (sin, cos) of every token's rotation angles, made once a step and kept
    with the batch (``batch.scratch``, which the decoder empties when a step starts) for every layer that rotates by
    the same frequencies."""
    scratch = getattr(batch, "scratch", None)
    key = ("rotary_table", inv_freq.data_ptr())
    if scratch is not None and key in scratch:
        return scratch[key]
    n, half = batch.positions.shape[0], inv_freq.shape[0]
    out = torch.empty((n, half, 2), dtype=torch.float32, device=inv_freq.device)
    _call("elementwise", "fms_rotary_table", _ptr(inv_freq), _ptr(batch.positions), _ptr(getattr(batch, "position_ids", None)),
          _ptr(out), n, half, _stream())
    if scratch is not None:
        scratch[key] = out
    return out


def qkv_rope_store(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                   batch, view, nheads: int, kvheads: int, head_dim: int, writes_cache: bool = True) -> torch.Tensor:
    """An attention layer's fused projection and what follows it: qkv = x weight^T (+ bias), q and k rotated by each
    token's position, k and v written into the cache, the rotated q returned.  For a few bfloat16 rows (a decode
    step) this is one kernel, the weight-streaming product with the rotation and the cache write in its epilogue;
    else the product and ``rope_store`` one after the other."""
    if (FUSE_QKV_ROPE and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_ROWS
            and weight.shape[1] % 8 == 0 and head_dim % 2 == 0 and (bias is None or bias.dtype == torch.bfloat16)
            and view.keys.dtype == torch.bfloat16 and weight.shape[0] == (nheads + 2 * kvheads) * head_dim):
        n = x.shape[0]
        q = torch.empty((n, nheads * head_dim), dtype=x.dtype, device=x.device)
        _call("gemm_bf16_skinny", "fms_qkv_rope_store_bf16_skinny", _ptr(x), _ptr(weight), _ptr(bias), _ptr(q),
              _ptr(inv_freq), _ptr(batch.positions), _ptr(getattr(batch, "position_ids", None)), _ptr(batch.token_seq),
              _ptr(batch.slots), _ptr(view.keys), _ptr(view.values), _ptr(view.table), view.table.shape[1],
              view.block_tokens, n, weight.shape[1], nheads,
              kvheads, head_dim, 1 if writes_cache else 0, _ptr(error_flag(x.device)), batch.slots.shape[0],
              view.table.shape[0], view.keys.shape[0], _stream())
        return q
    if (FUSE_QKV_ROPE and _mid_fits(x, weight, bias, "qkv") and head_dim % 2 == 0 and view.keys.dtype == torch.bfloat16
            and weight.shape[0] == (nheads + 2 * kvheads) * head_dim):
        n = x.shape[0]
        q = torch.empty((n, nheads * head_dim), dtype=x.dtype, device=x.device)
        _call("gemm_bf16_mid", "fms_qkv_rope_store_bf16_mid", _ptr(x), _ptr(weight), _ptr(bias), _ptr(q), _ptr(inv_freq),
              _ptr(batch.positions), _ptr(getattr(batch, "position_ids", None)), _ptr(batch.token_seq), _ptr(batch.slots),
              _ptr(view.keys), _ptr(view.values), _ptr(view.table), view.table.shape[1], view.block_tokens, n,
              weight.shape[1], nheads, kvheads, head_dim, 1 if writes_cache else 0, _ptr(error_flag(x.device)),
              batch.slots.shape[0], view.table.shape[0], view.keys.shape[0], _stream())
        return q
    if (FUSE_QKV_ROPE and _tensor_core_fits(x, weight, bias, TENSOR_CORE_ROWS_QKV) and head_dim % 16 == 0
            and (x.shape[0] + 255) // 256 * 256 <= TENSOR_CORE_MAX_PADDING * x.shape[0]
            and view.keys.dtype == torch.bfloat16 and weight.shape[0] == (nheads + 2 * kvheads) * head_dim):
        # many tokens: the tcgen05 product with the rotation and the cache write in its epilogue; the angles' sines and
        # cosines come from a table that the step's first such layer makes for all layers with the same frequencies
        n = x.shape[0]
        q = torch.empty((n, nheads * head_dim), dtype=x.dtype, device=x.device)
        table = None if inv_freq is None else rotary_table(inv_freq, batch)
        _call("gemm_bf16_tc", "fms_qkv_rope_store_bf16_tc", _ptr(x), _ptr(weight), _ptr(bias), _ptr(q), _ptr(table),
              _ptr(batch.positions), _ptr(batch.token_seq), _ptr(batch.slots),
              _ptr(view.keys), _ptr(view.values), _ptr(view.table), view.table.shape[1], view.block_tokens, n,
              weight.shape[1], nheads, kvheads, head_dim, 1 if writes_cache else 0, _ptr(error_flag(x.device)),
              batch.slots.shape[0], view.table.shape[0], view.keys.shape[0], _stream())
        return q
    return rope_store(linear(x, weight, bias), inv_freq, batch, view, nheads, kvheads, head_dim, writes_cache)


def _attention_library(head_dim: int) -> str:
    return f"attention_hd{head_dim}"


_attn_constants = {}


def attention_constants(head_dim: int, dtype: torch.dtype, nheads: int, kvheads: int):
    """(keys per decode split, positions per prefill tile) of the library built for this head size."""
    key = (head_dim, dtype, nheads, kvheads)
    if key not in _attn_constants:
        lib = load_library(_attention_library(head_dim))
        _attn_constants[key] = (int(lib.fms_attn_split_tokens()),
                                int(lib.fms_attn_prefill_tile_positions(_code(dtype), nheads, kvheads)))
    return _attn_constants[key]


def qk_prepare_store(proj: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int, qk_norm: bool, eps: float, batch,
                     view, nheads: int, kvheads: int, dim: int, vdim: int, pad: int,
                     writes_cache: bool = True, norm_first: bool = False, q_gain: Optional[torch.Tensor] = None,
                     k_gain: Optional[torch.Tensor] = None, halves: bool = False, values_are_keys: bool = False,
                     rot_mult: float = 1.0) -> torch.Tensor:
    """From rows [q: nheads x dim | k: kvheads x dim | v: kvheads x vdim | ...] of ``proj``: rotates the first ``rot``
    values of every q and k head by the row's position (adjacent pairs; with ``halves`` value i with value i + rot / 2),
    divides q and k by their root mean square over ``dim`` where ``qk_norm`` (after the rotation; with ``norm_first``
    before it, and then times ``q_gain`` / ``k_gain``, float32 [dim], where given), writes k and v into the cache (heads
    of ``pad`` values there, zeros beyond dim and vdim) and returns q [tokens, nheads * pad], padded alike.
    ``values_are_keys``: the rows have no v columns; a value is its key as projected, before norm and rotation.
    ``rot_mult`` multiplies the rotation's sines and cosines (stretched frequencies come with such a constant)."""
    n = proj.shape[0]
    for g in (q_gain, k_gain):
        if g is not None and (g.dtype != torch.float32 or g.shape[0] != dim):
            raise KernelError("qk_prepare_store: gains are float32 vectors of the head's size")
    if view.keys.dtype != proj.dtype or view.keys.shape[-1] != pad:
        raise KernelError(f"cache is {view.keys.dtype} with heads of {view.keys.shape[-1]}, activations are {proj.dtype}, "
                          f"heads of {pad}")
    q = torch.empty((n, nheads * pad), dtype=proj.dtype, device=proj.device)
    _call("elementwise", "fms_qk_prepare_store", _ptr(proj), _code(proj.dtype), proj.shape[1], _ptr(q), _ptr(inv_freq),
          int(rot), float(rot_mult), 1 if qk_norm else 0, float(eps), _ptr(q_gain), _ptr(k_gain), 1 if norm_first else 0,
          1 if halves else 0,
          1 if values_are_keys else 0, _ptr(batch.positions), _ptr(getattr(batch, "position_ids", None)),
          _ptr(batch.token_seq), _ptr(batch.slots), _ptr(view.keys), _ptr(view.values), _ptr(view.table),
          view.table.shape[1], view.block_tokens, n, nheads, kvheads, dim, vdim, pad, 1 if writes_cache else 0,
          _ptr(error_flag(proj.device)), batch.slots.shape[0], view.table.shape[0], view.keys.shape[0], _stream())
    return q


def sigmoid_gate(o: torch.Tensor, gate: Optional[torch.Tensor], gate_offset: int, nheads: int, vdim: int, pad: int,
                 factor: float = 1.0, per_head: bool = False) -> torch.Tensor:
    """out[t, h, :vdim] = factor * o[t, h, :vdim] * sigmoid(gate[t, gate_offset + h * vdim + :vdim]) for o with heads
    of ``pad`` values; ``gate`` is a matrix whose columns from ``gate_offset`` on hold the gates' logits (None: no
    gate, only the padding is dropped).  ``per_head``: one gate a head, sigmoid(gate[t, gate_offset + h])."""
    n = o.shape[0]
    out = torch.empty((n, nheads * vdim), dtype=o.dtype, device=o.device)
    gate_ptr = None if gate is None else _ptr(gate) + gate_offset * gate.element_size()
    _call("elementwise", "fms_sigmoid_gate", _ptr(o), gate_ptr, 0 if gate is None else gate.shape[1], _ptr(out),
          _code(o.dtype), n, nheads, vdim, pad, float(factor), 1 if per_head else 0, _stream())
    return out


def attention(q: torch.Tensor, batch, view, nheads: int, kvheads: int, head_dim: int, scale: float,
              window: int, sink: Optional[torch.Tensor] = None, chunk: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """Causal softmax attention of the step's queries over the cache (which already holds the step's own
    keys and values).  One query per sequence takes the split-key decode kernels, else the prefill kernel.
    ``sink`` [nheads] float32: a term exp(sink[h]) in every row's denominator that belongs to no key.
    ``chunk`` > 0: the positions of a sequence are cut into runs of ``chunk``, counted from its position 0, and a query
    sees the keys of its own run only (not together with a window).  ``softcap`` > 0: a score s becomes
    softcap * tanh(s / softcap) after the scale."""
    masked = bool(chunk) or bool(softcap)
    if chunk < 0 or softcap < 0 or (chunk and window):
        raise KernelError(f"attention: chunk {chunk}, window {window}, softcap {softcap}")
    if sink is not None and (sink.dtype != torch.float32 or sink.shape[0] != nheads):
        raise KernelError("attention: the sinks are float32, one per head")
    out = torch.empty_like(q)
    lib = _attention_library(head_dim)
    split, tile_rows = attention_constants(head_dim, q.dtype, nheads, kvheads)
    common = (_ptr(q), _ptr(out), _code(q.dtype), _ptr(view.keys), _ptr(view.values), _ptr(view.table),
              view.table.shape[1], view.block_tokens, _ptr(batch.slots), _ptr(batch.first_row), _ptr(batch.len_after))
    if batch.decode:
        n_splits = (batch.max_len_after + split - 1) // split
        part_o = torch.empty((batch.n_seqs, nheads, n_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((batch.n_seqs, nheads, n_splits, 2), dtype=torch.float32, device=q.device)
        # total_len (what the host knows of the sequences' lengths) chooses between the two bfloat16 decode kernels
        tail = (_ptr(sink), int(chunk), float(softcap)) if masked else (() if sink is None else (_ptr(sink),))
        _call(lib, "fms_attention_decode_masked" if masked else
              ("fms_attention_decode" if sink is None else "fms_attention_decode_sink"), *common, batch.n_seqs,
              n_splits, _ptr(part_o), _ptr(part_ml), nheads,
              kvheads, head_dim, float(scale), int(window), view.keys.shape[0], view.table.shape[0],
              int(getattr(batch, "total_len", 0)),
              _ptr(_work_counter(q.device)), _ptr(error_flag(q.device)), *tail, _stream())
        if n_splits > 1 or q.dtype == torch.float32:
            global launches
            launches += 1  # the kernel that merges the splits
    else:
        tiles = batch.query_tiles(tile_rows)
        tail = (_ptr(sink), int(chunk), float(softcap)) if masked else (() if sink is None else (_ptr(sink),))
        _call(lib, "fms_attention_prefill_masked" if masked else
              ("fms_attention_prefill" if sink is None else "fms_attention_prefill_sink"), *common, _ptr(tiles),
              tiles.shape[0], nheads, kvheads, head_dim, float(scale), int(window), view.keys.shape[0],
              view.table.shape[0], _ptr(error_flag(q.device)), *tail, _stream())
    return out


def attention_stream_launches(head_dim: int) -> int:
    """How often this process has launched (or captured) the streaming decode-attention kernel of a head size."""
    lib = load_library(f"attention_hd{head_dim}")
    lib.fms_attn_stream_launches.restype = ctypes.c_long
    return int(lib.fms_attn_stream_launches())


def decode_advance(positions: torch.Tensor, lengths: torch.Tensor, offsets: Optional[torch.Tensor] = None,
                   position_ids: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                   spare_slot: int = -1) -> None:
    """positions[i] = lengths[i]; lengths[i] += 1 — the bookkeeping of a decode step, on the device.  With
    ``offsets`` (sequences that did not start at position 0) also position_ids[i] = positions[i] + offsets[i].
    With ``slots``: a row in ``spare_slot`` (one that only fills the step up to a captured size) restarts at
    position 0 every step."""
    _call("elementwise", "fms_decode_advance", _ptr(positions), _ptr(lengths), _ptr(offsets), _ptr(position_ids),
          _ptr(slots), int(spare_slot), positions.shape[0], _stream())


# ---- recurrence --------------------------------------------------------------------------------------
_recurrent_chunk = None
SCAN_CHUNKS_FROM = 192  # tokens of a sequence in one step from which its scan runs chunk by chunk


def mingru_scan(proj: torch.Tensor, state: torch.Tensor, batch, width: int, writes_state: bool = True) -> torch.Tensor:
    """The minGRU recurrence over a step's rows.  ``proj`` [tokens, 3 width] = [z logits | u | g]; ``state``
    [slots, width] float32 is read for every sequence of the batch and, with ``writes_state``, left at its value after
    the step's last token.  Returns S_t * silu(g) [tokens, width] in proj's dtype."""
    global _recurrent_chunk
    n = proj.shape[0]
    if proj.shape[1] != 3 * width or state.dtype != torch.float32 or state.shape[1] != width:
        raise KernelError("mingru_scan: proj is [tokens, 3 width], the state float32 [slots, width]")
    y = torch.empty((n, width), dtype=proj.dtype, device=proj.device)
    chunk_rows = first_chunk = ab = None
    n_chunks = 0
    if batch.max_new >= SCAN_CHUNKS_FROM:
        if _recurrent_chunk is None:
            _recurrent_chunk = int(load_library("recurrent").fms_recurrent_chunk_tokens())
        chunk_rows, first_chunk = batch.row_chunks(_recurrent_chunk)
        n_chunks = chunk_rows.shape[0]
        ab = torch.empty((n_chunks, 2, width), dtype=torch.float32, device=proj.device)
    _call("recurrent", "fms_mingru_scan", _ptr(proj), _code(proj.dtype), _ptr(state), _ptr(y), _ptr(batch.first_row),
          _ptr(batch.slots), batch.n_seqs, width, state.shape[0], 1 if writes_state else 0, _ptr(chunk_rows),
          _ptr(first_chunk), n_chunks, _ptr(ab), _stream())
    global launches
    launches += 2 if n_chunks else 0
    return y


# ---- state matrices carried from token to token -----------------------------------------------------
def causal_conv(x: torch.Tensor, offset: int, channels: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                tail: torch.Tensor, batch, activation: bool = True, writes_state: bool = True) -> torch.Tensor:
    """A short causal convolution per channel over each sequence's rows, then silu (``activation``).  The convolved
    channels are columns ``offset .. offset + channels`` of ``x``; ``weight`` [channels, taps] float32 (its last column
    multiplies the current row), ``bias`` [channels] float32 or None; ``tail`` [slots, taps - 1, channels] float32 holds
    each sequence's last taps - 1 inputs and, with ``writes_state``, is left at those after this step.  Returns float32
    [tokens, channels]."""
    n, taps = x.shape[0], weight.shape[1]
    if weight.dtype != torch.float32 or tuple(weight.shape) != (channels, taps) or tail.dtype != torch.float32 \
            or tuple(tail.shape[1:]) != (taps - 1, channels) or (bias is not None and bias.dtype != torch.float32):
        raise KernelError("causal_conv: weight [channels, taps], bias and tail [slots, taps - 1, channels] are float32")
    out = torch.empty((n, channels), dtype=torch.float32, device=x.device)
    _call("state_scan", "fms_causal_conv", _ptr(x) + offset * x.element_size(), _code(x.dtype), x.shape[1], _ptr(weight),
          _ptr(bias), _ptr(tail), _ptr(batch.token_seq), _ptr(batch.first_row), _ptr(batch.slots), _ptr(out), n,
          batch.n_seqs, channels, taps, 1 if activation else 0, 1 if writes_state else 0, tail.shape[0], _stream())
    global launches
    launches += 1 if writes_state and taps > 1 else 0
    return out


def selective_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_offset: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
                   d_skip: torch.Tensor, state: torch.Tensor, batch, heads: int, vdim: int, n_state: int, groups: int,
                   writes_state: bool = True) -> torch.Tensor:
    """Per head, S = exp(-exp(a_log) dt) S + dt B x^T and y = S^T C + d_skip x over each sequence's rows, with
    dt = softplus(proj[:, dt_offset + head] + dt_bias).  ``xbc`` float32 [tokens, heads * vdim + 2 groups * n_state] =
    [x | B | C]; ``state`` float32 [slots, heads, vdim, n_state].  Returns y float32 [tokens, heads * vdim]."""
    n = xbc.shape[0]
    if xbc.dtype != torch.float32 or state.dtype != torch.float32 or xbc.shape[1] != heads * vdim + 2 * groups * n_state \
            or tuple(state.shape[1:]) != (heads, vdim, n_state):
        raise KernelError("selective_scan: xbc float32 [tokens, x | B | C], state float32 [slots, heads, vdim, state]")
    y = torch.empty((n, heads * vdim), dtype=torch.float32, device=xbc.device)
    _call("state_scan", "fms_selective_scan", _ptr(xbc), _ptr(proj) + dt_offset * proj.element_size(), _code(proj.dtype),
          proj.shape[1], _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(state), _ptr(y), _ptr(batch.first_row),
          _ptr(batch.slots), batch.n_seqs, heads, vdim, n_state, groups, 1 if writes_state else 0, state.shape[0],
          _stream())
    return y


def delta_rule_scan(qkv: torch.Tensor, proj: torch.Tensor, beta_offset: int, a_raw: Optional[torch.Tensor],
                    dt_bias: torch.Tensor, a_log: torch.Tensor, state: torch.Tensor, batch, heads: int, kvheads: int,
                    dim: int, vdim: int, writes_state: bool = True, decay_offset: Optional[int] = None) -> torch.Tensor:
    """Per head, S = diag(g) S; u = beta (v - S^T k); S += k u^T; o = S^T q over each sequence's rows.  ``qkv`` float32
    [tokens, 2 kvheads * dim + heads * vdim] = [q | k | v]; beta = sigmoid(proj[:, beta_offset + head]);
    g = exp(-exp(a_log[head]) softplus(a_raw + dt_bias)), [heads * dim] a row; ``state`` float32 [slots, heads, vdim, dim].
    q and k of ``qkv`` are made unit vectors in place on the way.  Returns o float32 [tokens, heads * vdim].
    ``decay_offset`` (with ``a_raw`` None): one decay a head instead of one a key channel,
    g = exp(-exp(a_log[head]) softplus(proj[:, decay_offset + head] + dt_bias[head])), dt_bias [heads]."""
    n = qkv.shape[0]
    per_head = decay_offset is not None
    if qkv.dtype != torch.float32 or state.dtype != torch.float32 or qkv.shape[1] != 2 * kvheads * dim + heads * vdim \
            or tuple(state.shape[1:]) != (heads, vdim, dim):
        raise KernelError("delta_rule_scan: qkv float32 [tokens, q | k | v], state float32 [slots, heads, vdim, dim]")
    if per_head:
        if a_raw is not None or dt_bias.shape[0] != heads or proj.shape[1] < decay_offset + heads:
            raise KernelError("delta_rule_scan: one decay a head reads its logits from proj and a bias a head")
        a_ptr, a_stride = _ptr(proj) + decay_offset * proj.element_size(), proj.shape[1]
    else:
        if tuple(a_raw.shape) != (n, heads * dim) or a_raw.dtype != proj.dtype or dt_bias.shape[0] != heads * dim:
            raise KernelError("delta_rule_scan: decays' logits [tokens, heads * dim] in the projection's dtype")
        a_ptr, a_stride = _ptr(a_raw), heads * dim
    o = torch.empty((n, heads * vdim), dtype=torch.float32, device=qkv.device)
    # decays [tokens, heads * dim], then betas [tokens, heads]
    scratch = torch.empty((n * heads * (dim + 1),), dtype=torch.float32, device=qkv.device)
    _call("state_scan", "fms_delta_rule_scan", _ptr(qkv), _ptr(proj) + beta_offset * proj.element_size(),
          _code(proj.dtype), proj.shape[1], a_ptr, a_stride, 1 if per_head else 0, _ptr(dt_bias), _ptr(a_log),
          scratch.data_ptr(),
          scratch.data_ptr() + 4 * n * heads * dim, _ptr(state), _ptr(o), _ptr(batch.first_row), _ptr(batch.slots), n,
          batch.n_seqs, heads, kvheads, dim, vdim, 1 if writes_state else 0, state.shape[0], _stream())
    global launches
    launches += 1  # the kernel that makes q, k, the decays and the betas ready
    return o


ACT_NONE, ACT_SILU = 0, 1


def decay_scan(proj: torch.Tensor, state: torch.Tensor, batch, heads: int, dim: int, vdim: int, activation: int = ACT_NONE,
               q_scale: float = 1.0, decay: Optional[torch.Tensor] = None, gate_offset: int = 0,
               gate_bias: Optional[torch.Tensor] = None, gate_cap: float = 0.0, norm_state: Optional[torch.Tensor] = None,
               writes_state: bool = True) -> torch.Tensor:
    """A state matrix per head under scalar decays, over each sequence's rows.  The first columns of ``proj`` are
    [q: heads x dim | k: heads x dim | v: heads x vdim]; they are taken in float32 through ``activation`` (``ACT_SILU``
    or none), q times ``q_scale``.  ``state`` float32 [slots, heads, vdim, dim].

    With ``decay`` (float32 [heads]): S = decay_h S + k v^T; o = S^T q.

    With ``gate_bias`` (float32 [2 heads]: the input gates' biases, then the forget gates'): columns ``gate_offset + h``
    and ``gate_offset + heads + h`` of ``proj`` are head h's gates before their biases, i = cap tanh((. + b) / cap),
    f = logsigmoid(cap tanh((. + b) / cap)); with the running maximum m' = max(f + m, i): S = exp(f + m - m') S +
    exp(i - m') k v^T, n likewise with k alone, o = S^T q / (max(|n.q|, exp(-m')) + 1e-6).  ``norm_state`` float32
    [slots, heads, dim + 1] holds n and then m (zeros for a new sequence).

    Returns o float32 [tokens, heads * vdim]."""
    n = proj.shape[0]
    cols = heads * (2 * dim + vdim)
    gated = gate_bias is not None
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, vdim, dim) or proj.shape[1] < cols:
        raise KernelError("decay_scan: proj [tokens, q | k | v | ...], state float32 [slots, heads, vdim, dim]")
    if gated == (decay is not None):
        raise KernelError("decay_scan: either one decay a head or the gates' biases")
    if gated and (norm_state is None or norm_state.dtype != torch.float32 or tuple(norm_state.shape[1:]) != (heads, dim + 1)
                  or gate_bias.dtype != torch.float32 or gate_bias.shape[0] != 2 * heads
                  or proj.shape[1] < gate_offset + 2 * heads or norm_state.shape[0] != state.shape[0]):
        raise KernelError("decay_scan: gate biases float32 [2 heads], norm_state float32 [slots, heads, dim + 1]")
    if not gated and (decay.dtype != torch.float32 or decay.shape[0] != heads):
        raise KernelError("decay_scan: decays float32 [heads]")
    qkv = torch.empty((n, cols), dtype=torch.float32, device=proj.device)
    _call("state_scan", "fms_linear_prepare", _ptr(proj), _code(proj.dtype), proj.shape[1], _ptr(qkv), n, cols, heads * dim,
          float(q_scale), int(activation), _stream())
    o = torch.empty((n, heads * vdim), dtype=torch.float32, device=proj.device)
    gates = torch.empty((n, heads, 3), dtype=torch.float32, device=proj.device) if gated else None
    norm_in = torch.empty((batch.n_seqs, heads, dim), dtype=torch.float32, device=proj.device) if gated else None
    gate_ptr = _ptr(proj) + gate_offset * proj.element_size() if gated else None
    _call("state_scan", "fms_decay_scan", _ptr(qkv), gate_ptr, _code(proj.dtype), proj.shape[1], _ptr(gate_bias),
          float(gate_cap), _ptr(gates), _ptr(norm_in), _ptr(decay), _ptr(state), _ptr(norm_state), _ptr(o), _ptr(batch.first_row),
          _ptr(batch.slots), n, batch.n_seqs, heads, dim, vdim, 1 if writes_state else 0, state.shape[0], _stream())
    global launches
    launches += 1 if gated else 0  # the kernel that walks the gates
    return o


GATE_NONE, GATE_SILU_BEFORE, GATE_SIGMOID_AFTER, GATE_SILU_AFTER = 0, 1, 2, 3


def gated_group_rmsnorm(x: torch.Tensor, gate: Optional[torch.Tensor], gate_offset: int, gate_mode: int,
                        weight: torch.Tensor, eps: float, group_size: int, out_dtype: torch.dtype,
                        factor: float = 1.0) -> torch.Tensor:
    """Rows of ``x`` (float32) cut into groups of ``group_size``, each divided by its root mean square, times
    ``weight`` (float32; repeated along the row where it is shorter), times ``factor``.  ``gate``: a matrix whose
    columns from ``gate_offset`` on are the gates' logits: ``GATE_SILU_BEFORE`` multiplies x by silu(gate) before the
    norm, ``GATE_SIGMOID_AFTER`` the normed and weighted values by sigmoid(gate), ``GATE_SILU_AFTER`` by silu(gate)."""
    n, width = x.shape
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or width % weight.shape[0]:
        raise KernelError("gated_group_rmsnorm: x and weight are float32, the weight's length divides the row's")
    if gate is not None and gate.dtype != out_dtype:
        raise KernelError(f"gated_group_rmsnorm: gate {gate.dtype}, compute dtype {out_dtype}")
    out = torch.empty((n, width), dtype=out_dtype, device=x.device)
    gate_ptr = None if gate is None else _ptr(gate) + gate_offset * gate.element_size()
    _call("state_scan", "fms_gated_group_rmsnorm", _ptr(x), gate_ptr, _code(out_dtype), 0 if gate is None else gate.shape[1],
          int(gate_mode) if gate is not None else GATE_NONE, _ptr(weight), weight.shape[0], float(eps), float(factor),
          _ptr(out), n, width, int(group_size), _stream())
    return out


# ---- groups of rows, each with a matrix of its own ---------------------------------------------------
GROUPED_FEW_ROWS = 32  # rows of a step up to which the grouped products walk each group's rows (a decode step)
# FMS_B200_GROUPED_LIBRARY=0: the own float32-sum kernel for the ragged products of many bfloat16 rows too
USE_LIBRARY_GROUPED = os.environ.get("FMS_B200_GROUPED_LIBRARY", "1") != "0" and hasattr(torch.nn.functional, "grouped_mm")


def grouped_linear(x: torch.Tensor, weight: torch.Tensor, groups: int, rows: int, n_out: int, k: int, x_row_stride: int,
                   x_group_offset: int, y: torch.Tensor, y_row_stride: int, y_group_offset: int) -> torch.Tensor:
    """Uniform groups: for every group g, y[r, g * y_group_offset + :n_out] = x[r, g * x_group_offset + :k] . weight[g]^T
    for r < rows (x and y are walked by their row strides; weight [groups, n_out, k])."""
    if weight.dtype != x.dtype or y.dtype != x.dtype or tuple(weight.shape) != (groups, n_out, k):
        raise KernelError(f"grouped_linear: x {x.dtype}, weight {weight.dtype} {tuple(weight.shape)}, y {y.dtype}")
    _ptr(x), _ptr(weight), _ptr(y)
    if USE_LIBRARY_GROUPED and x.dtype == torch.bfloat16 and rows > GROUPED_FEW_ROWS:
        # many bfloat16 rows: the library's batched product over strided views of x and y (no copy of either)
        xv = torch.as_strided(x, (groups, rows, k), (x_group_offset, x_row_stride, 1), x.storage_offset())
        yv = torch.as_strided(y, (groups, rows, n_out), (y_group_offset, y_row_stride, 1), y.storage_offset())
        torch.bmm(xv, weight.transpose(1, 2), out=yv)
        return y
    _call("grouped", "fms_grouped_linear", _ptr(x), _ptr(weight), _ptr(y), _code(x.dtype), None, None, None, groups, rows,
          n_out, k, x_row_stride, x_group_offset, y_row_stride, y_group_offset, 0, 0.0, 0.0,
          1 if rows <= GROUPED_FEW_ROWS else 0, _stream())
    return y


class Routing:
    """What ``route`` leaves on the device: each pair's expert and weight, the experts' row ranges in the sorted
    matrix, and the sorted, weighted rows themselves."""

    __slots__ = ("expert", "weight", "offsets", "tile_first", "row_of_pair", "group_of_row", "rows", "top", "experts",
                 "weights_on_output")


ROUTE_SIGMOID, ROUTE_SOFTMAX = 0, 1


def route(x: torch.Tensor, router: torch.Tensor, top: int, mode: int = ROUTE_SIGMOID,
          correction: Optional[torch.Tensor] = None, route_scale: float = 1.0) -> Routing:
    """``ROUTE_SIGMOID``: scores sigmoid(x router^T) in float32; every token's ``top`` best experts; rows
    weight * x[token] sorted by expert.  ``ROUTE_SOFTMAX``: scores softmax(x router^T) over all experts; the ``top``
    experts with the largest score + ``correction`` [experts] (float32, or None) are the token's; its weights are their
    scores over their sum (+ 1e-20), times ``route_scale``; the sorted rows are the tokens' as they are and
    ``route_gather`` multiplies the experts' results by the weights."""
    if correction is not None and (correction.dtype != torch.float32 or correction.shape[0] != router.shape[0]):
        raise KernelError("route: the correction is float32, one number an expert")
    n, dim = x.shape
    experts = router.shape[0]
    dev = x.device
    r = Routing()
    r.top, r.experts = top, experts
    r.weights_on_output = mode == ROUTE_SOFTMAX
    ints = torch.empty((n * top * 3 + 3 * (experts + 1),), dtype=torch.int32, device=dev)
    r.expert = ints[: n * top].view(n, top)
    r.row_of_pair = ints[n * top: 2 * n * top]
    r.group_of_row = ints[2 * n * top: 3 * n * top]
    o = 3 * n * top
    counts = ints[o: o + experts + 1]
    r.offsets = ints[o + experts + 1: o + 2 * (experts + 1)]
    r.tile_first = ints[o + 2 * (experts + 1): o + 3 * (experts + 1)]
    r.weight = torch.empty((n, top), dtype=torch.float32, device=dev)
    r.rows = torch.empty((n * top, dim), dtype=x.dtype, device=dev)
    _call("grouped", "fms_route", _ptr(x), _code(x.dtype), _ptr(router), _code(router.dtype), _ptr(r.expert),
          _ptr(r.weight), _ptr(counts), _ptr(r.offsets), _ptr(r.tile_first), _ptr(r.row_of_pair), _ptr(r.group_of_row),
          _ptr(r.rows), n, dim, experts, top, int(mode), _ptr(correction), float(route_scale), _stream())
    global launches
    launches += 2
    return r


def routed_linear(rows: torch.Tensor, weight: torch.Tensor, routing: Routing, glu: bool = False, limit: float = 0.0,
                  alpha: float = 1.0, relu_squared: bool = False) -> torch.Tensor:
    """Ragged groups: y[r] = rows[r] . weight[expert of r]^T; with ``glu`` weight[e] = [gate; up] and
    y = g * sigmoid(alpha g) * (u + 1) for g = min(gate, limit), u = clamp(up, -limit, limit); with ``relu_squared``
    y = max(y, 0)^2."""
    n, k = rows.shape
    n_out = weight.shape[1] // (2 if glu else 1)
    if weight.dtype != rows.dtype or weight.shape[0] != routing.experts or weight.shape[2] != k:
        raise KernelError(f"routed_linear: rows {rows.dtype} {tuple(rows.shape)}, weight {weight.dtype} {tuple(weight.shape)}")
    if (USE_LIBRARY_GROUPED and rows.dtype == torch.bfloat16 and n > GROUPED_FEW_ROWS and k % 8 == 0
            and weight.shape[1] % 8 == 0):
        # many bfloat16 rows: the library's grouped product (it takes the groups' ends from the device, as the
        # own kernels do), as the plain products of many rows take the library's; the gated unit is a kernel after it
        _ptr(rows), _ptr(weight)
        y = torch.nn.functional.grouped_mm(rows, weight.transpose(1, 2), offs=routing.offsets[1:])
        if relu_squared and not glu:
            _call("grouped", "fms_relu_squared", _ptr(y), _code(y.dtype), y.numel(), _stream())
        if not glu:
            return y
        out = torch.empty((n, n_out), dtype=rows.dtype, device=rows.device)
        _call("grouped", "fms_gated_clamped", _ptr(y), _ptr(out), _code(y.dtype), n, n_out, float(limit), float(alpha),
              _stream())
        return out
    y = torch.empty((n, n_out), dtype=rows.dtype, device=rows.device)
    _call("grouped", "fms_grouped_linear", _ptr(rows), _ptr(weight), _ptr(y), _code(rows.dtype), _ptr(routing.offsets),
          _ptr(routing.tile_first), _ptr(routing.group_of_row), routing.experts, n, n_out, k, k, 0, n_out, 0,
          1 if glu else (2 if relu_squared else 0), float(limit), float(alpha), 1 if n <= GROUPED_FEW_ROWS else 0, _stream())
    return y


def route_gather(ys: torch.Tensor, routing: Routing) -> torch.Tensor:
    """out[token] = the sum of its pairs' rows of ``ys`` (each times its weight where the routing left the weights for
    the experts' results), float32, in the order of its choices."""
    n = ys.shape[0] // routing.top
    out = torch.empty((n, ys.shape[1]), dtype=ys.dtype, device=ys.device)
    _call("grouped", "fms_route_gather", _ptr(ys), _code(ys.dtype), _ptr(routing.row_of_pair), _ptr(out), n, ys.shape[1],
          routing.top, _ptr(routing.weight) if routing.weights_on_output else None, _stream())
    return out


# ---- attention over cached latents -------------------------------------------------------------------
_latent_split = None
USE_LATENT_MMA = os.environ.get("FMS_B200_LATENT_MMA", "1") != "0"  # 0: a prompt's rows through the float32 kernel too


def latent_prepare(proj: torch.Tensor, q_full: torch.Tensor, c_gain: torch.Tensor, eps: float, inv_freq: torch.Tensor,
                   rot_dims: int, batch, view, heads: int, dim: int, rot: int, rank: int, writes_cache: bool = True,
                   halves: bool = False, rot_mult: float = 1.0, kv: Optional[torch.Tensor] = None) -> None:
    """From the fused projection [q heads (dim + rot each) | c (rank) | kr (rot) | ...] of a step's rows: norms c,
    rotates kr and every head's rot part by the row's position, writes [c | kr] into the cache at the row's place and
    the rotated query parts into q_full[:, h, rank:].  ``kv``: [c | kr] are the first columns of this matrix instead
    (queries that come from a projection of their own; ``proj`` then holds the query heads only).  ``halves``: value i
    of a rotated run turns with value i + rot_dims / 2 instead of its neighbour; ``rot_mult`` multiplies sines and cosines."""
    if kv is not None and (kv.dtype != proj.dtype or kv.shape[0] != proj.shape[0] or kv.shape[1] < rank + rot):
        raise KernelError("latent_prepare: the latent's matrix has the projection's dtype and rows, and rank + rot columns")
    if view.keys.dtype != proj.dtype or q_full.dtype != proj.dtype:
        raise KernelError(f"cache is {view.keys.dtype}, activations are {proj.dtype}")
    _call("latent_attention", "fms_latent_prepare", _ptr(proj), _code(proj.dtype), proj.shape[1], _ptr(q_full), _ptr(c_gain),
          _code(c_gain.dtype), float(eps), _ptr(inv_freq), int(rot_dims), _ptr(batch.positions),
          _ptr(getattr(batch, "position_ids", None)), _ptr(batch.token_seq), _ptr(batch.slots), _ptr(view.keys),
          _ptr(view.table), view.table.shape[1], view.block_tokens, proj.shape[0], heads, dim, rot, rank,
          1 if writes_cache else 0, batch.slots.shape[0], view.table.shape[0], view.keys.shape[0],
          _ptr(error_flag(proj.device)), 1 if halves else 0, float(rot_mult), _ptr(kv), 0 if kv is None else kv.shape[1],
          _stream())


def latent_query_norm(proj: torch.Tensor, offset: int, n: int, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """Columns ``offset .. offset + n`` of ``proj``, each row divided by its root mean square over them, times ``gain``
    [n]: the query's latent on its way to the projection that makes the heads' queries of it."""
    if proj.shape[1] < offset + n or gain.shape[0] != n:
        raise KernelError("latent_query_norm: the columns lie inside the rows and the gain has their number")
    out = torch.empty((proj.shape[0], n), dtype=proj.dtype, device=proj.device)
    _call("latent_attention", "fms_latent_query_norm", _ptr(proj) + offset * proj.element_size(), _code(proj.dtype),
          proj.shape[1], n, _ptr(gain), _code(gain.dtype), float(eps), _ptr(out), proj.shape[0], _stream())
    return out


def latent_attention(q_full: torch.Tensor, batch, view, gate: Optional[torch.Tensor], gate_offset: int,
                     sink: Optional[torch.Tensor], heads: int, rank: int, rot: int, scale: float,
                     window: int = 0) -> torch.Tensor:
    """Causal softmax attention of the step's rows over the cached latent rows [c | kr] (which already hold the step's
    own), with a per-head sink in the denominator and a per-head sigmoid gate on the result.  ``gate``: the matrix
    whose column ``gate_offset + h`` holds head h's gate logit of each row (None: no gate); ``sink`` None: no sink;
    ``window`` > 0: the row at position p sees the keys p - window + 1 .. p only.  Returns [tokens, heads, rank]."""
    global _latent_split, launches
    n = q_full.shape[0]
    out = torch.empty((n, heads, rank), dtype=q_full.dtype, device=q_full.device)
    if _latent_split is None:
        _latent_split = int(load_library("latent_attention").fms_latent_split_tokens())
    if (USE_LATENT_MMA and q_full.dtype == torch.bfloat16 and rank % 64 == 0 and rank <= 512
            and (rank + rot) % 32 == 0 and (gate is None or gate.dtype == torch.bfloat16)):
        # both products on the tensor cores, 32 rows a block: a prompt's rows as tokens x heads over all their keys; a
        # decode step's as one token's heads over one split of the keys, merged afterwards
        n_splits, part_o, part_ml = 1, None, None
        if batch.decode:
            heads_per_block = 32
            n_splits = max(1, (batch.max_len_after + _latent_split - 1) // _latent_split)
            if n_splits > 1:
                part_o = torch.empty((n, heads, n_splits, rank), dtype=torch.float32, device=q_full.device)
                part_ml = torch.empty((n, heads, n_splits, 2), dtype=torch.float32, device=q_full.device)
        else:
            heads_per_block = 1
            while heads_per_block < min(32, heads):
                heads_per_block *= 2
        tile_tokens = 32 // heads_per_block
        tiles = batch.query_tiles(tile_tokens)
        gate_ptr = None if gate is None else _ptr(gate) + gate_offset * gate.element_size()
        _call("latent_attention", "fms_latent_attention_prefill_bf16", _ptr(q_full), _ptr(out), _ptr(view.keys), gate_ptr,
              0 if gate is None else gate.shape[1], _ptr(sink), _code(sink.dtype) if sink is not None else F32,
              _ptr(view.table), view.table.shape[1], view.block_tokens, _ptr(batch.slots), _ptr(batch.first_row),
              _ptr(batch.positions), _ptr(tiles), tiles.shape[0], tile_tokens, heads_per_block, heads, rank, rot,
              float(scale), batch.slots.shape[0], view.table.shape[0], view.keys.shape[0], _ptr(batch.token_seq), n_splits,
              _ptr(part_o), _ptr(part_ml), int(window), _stream())
        if n_splits > 1:
            launches += 1
        return out
    n_splits, part_o, part_ml = 1, None, None
    if batch.decode:
        n_splits = max(1, (batch.max_len_after + _latent_split - 1) // _latent_split)
        if n_splits > 1:
            part_o = torch.empty((n, heads, n_splits, rank), dtype=torch.float32, device=q_full.device)
            part_ml = torch.empty((n, heads, n_splits, 2), dtype=torch.float32, device=q_full.device)
    gate_ptr = None if gate is None else _ptr(gate) + gate_offset * gate.element_size()
    _call("latent_attention", "fms_latent_attention", _ptr(q_full), _ptr(out), _code(q_full.dtype), _ptr(view.keys), gate_ptr,
          0 if gate is None else gate.shape[1], _ptr(sink), _code(sink.dtype) if sink is not None else F32,
          _ptr(view.table), view.table.shape[1], view.block_tokens, _ptr(batch.slots), _ptr(batch.token_seq),
          _ptr(batch.positions), n, n_splits, _ptr(part_o), _ptr(part_ml), heads, rank, rot, float(scale),
          batch.slots.shape[0], view.table.shape[0], view.keys.shape[0], int(window), _stream())
    if n_splits > 1:
        launches += 1
    return out


# ---- sampling ----------------------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, vocab = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("logits are float32")
    out = out if out is not None else torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _call("sampling", "fms_argmax", _ptr(logits), _ptr(out), rows, vocab, _stream())
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, seed: int, requests: torch.Tensor, step: int,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, vocab = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("logits are float32")
    out = out if out is not None else torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _call("sampling", "fms_sample", _ptr(logits), _ptr(out), rows, vocab, float(temperature), int(top_k),
          int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(requests), int(step), _stream())
    return out
