"""Figonex: a decoder whose sublayers read the residual stream as it is and whose outputs are normed on their way into
it, x = x + s1 * LN1(mixer(x)); x = x + s2 * LN2(mlp(x)) (a layer norm with a weight and no bias, then a scale per
channel).  A layer's mixer is one of

    mlstm      a matrix memory per head under exponential input and forget gates (capped logits, a running maximum)
    attention  grouped-query softmax attention whose values are its keys as projected, with a weighted rms norm of
               q and k per head before a rotation of the heads' first values in halves, one added to the softmax's
               denominator, and one sigmoid gate a head
    lightning  a matrix memory per head under one fixed decay a head, with silu on q, k and v

each followed by a dense gated feed-forward (or none).  A layer may run with the tensors of an earlier layer and a cache
entry or state of its own.  The embedded rows are multiplied by a number; the last norm is a layer norm as well.

This file is all that is specific to the architecture: its ``config.json`` (every size and constant is read from it:
``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and ``layers``, each entry with its ``type``, the sizes and
constants of its ``mixer``, its ``mlp`` or null, and ``weights_of`` where it has no tensors of its own), the
``DecoderSpec`` that configuration means, and the checkpoint's tensor names and layouts:

    embed [vocab, width]    final.norm [width]    head [vocab, width]
    l<i>.norm1, l<i>.ls1, l<i>.norm2, l<i>.ls2 [width]
    mlstm:      l<i>.mix.q, .k [heads dim, width], .v, .g [heads vdim, width], .i, .f [heads, width], .i.b, .f.b [heads],
                .norm [heads vdim], .o [width, heads vdim]
    attention:  l<i>.mix.q [heads dim, width], .k [kv_heads dim, width], .q.norm, .k.norm [dim], .g [heads, width],
                .o [width, heads dim]
    lightning:  l<i>.mix.q, .k [heads dim, width], .v, .g [heads vdim, width], .norm [heads vdim], .o [width, heads vdim]
    dense:      l<i>.mlp.gate, .up [ff, width], .down [width, ff]

Linear weights are stored [out, in].  The adapter puts everything that reads a mixer's input into one matrix
([q; k; g], [q; k; v; g; i; f], [q; k; v; g], rows filled up with zeros to a multiple of 8), the two gates' biases into
one vector, and [gate; up] into one matrix.
"""
from __future__ import annotations

import copy
import dataclasses
import re
from typing import Any, Dict, List, Optional

import torch

from ..config.model_config import ModelConfig
from ..config.specs import BlockSpec, DecoderSpec, FeedForwardSpec, LayerCall, MixerSpec, NormSpec, PositionSpec
from ..parts.attention import SinkAttention
from ..parts.linear_attention import LightningAttention, MatrixLSTM
from ..weights.adapters import register_adapter, register_adapter_step
from ..weights.sources import TensorLayout
from . import register_architecture, register_model
from .base import Model

LAYER_TYPES = ("mlstm", "attention", "lightning")


@dataclasses.dataclass
class FigonexConfig(ModelConfig):
    vocab: int = 1024
    width: int = 128
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    max_positions: int = 131072  # how long a sequence may get; nothing in the model depends on it

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ValueError(f"vocab {self.vocab}, width {self.width}")
        for i, layer in enumerate(self.layers):
            kind = layer.get("type")
            if kind not in LAYER_TYPES:
                raise ValueError(f"layer {i}: type {kind!r}; known: {', '.join(LAYER_TYPES)}")
            m = layer.get("mixer") or {}
            need = {"mlstm": ("heads", "dim", "vdim", "gate_cap"), "attention": ("heads", "kv_heads", "dim", "scale"),
                    "lightning": ("heads", "dim", "vdim", "decay")}[kind]
            absent = [k for k in need if k not in m]
            if absent:
                raise ValueError(f"layer {i} ({kind}): its mixer lacks {absent}")
            if kind == "attention":
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ValueError(f"layer {i}: {m['heads']} query heads over {m['kv_heads']} key heads")
                if int(m.get("vdim", m["dim"])) != int(m["dim"]):
                    raise ValueError(f"layer {i}: the values are the keys, so vdim {m['vdim']} has to be dim {m['dim']}")
            if kind == "lightning" and len(m["decay"]) != int(m["heads"]):
                raise ValueError(f"layer {i}: {len(m['decay'])} decays for {m['heads']} heads")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r}; known: dense, or null for none")
            j = layer.get("weights_of")
            if j is not None and not (0 <= int(j) < i and self.layers[int(j)]["type"] == kind):
                raise ValueError(f"layer {i}: weights_of {j} names no earlier layer of its type")

    def owner_of(self, i: int) -> int:
        """The layer whose tensors layer i runs with: itself, or where its chain of ``weights_of`` ends."""
        while self.layers[i].get("weights_of") is not None:
            i = int(self.layers[i]["weights_of"])
        return i


def _config_from_json(values: Dict[str, Any]) -> FigonexConfig:
    if values.get("architecture") != "Figonex":
        raise ValueError(f"config.json is of architecture {values.get('architecture')!r}, not Figonex")
    absent = [k for k in ("vocab", "width", "layers", "norm") if k not in values]
    if absent:
        raise ValueError(f"config.json lacks {absent}")
    return FigonexConfig(vocab=int(values["vocab"]), width=int(values["width"]), norm_eps=float(values["norm"]["eps"]),
                         embedding_scale=float((values.get("embedding") or {}).get("scale", 1.0)),
                         layers=copy.deepcopy(values["layers"]), max_positions=int(values.get("max_positions", 131072)))


# ---- layer entries as config.json has them -----------------------------------------------------------
def dense_mlp(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def _entry(kind: str, mixer: dict, mlp: Optional[dict], weights_of: Optional[int]) -> dict:
    out = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def mlstm_layer(heads: int, dim: int, vdim: int, gate_cap: float, mlp: Optional[dict],
                weights_of: Optional[int] = None) -> dict:
    return _entry("mlstm", {"dim": dim, "gate_cap": gate_cap, "heads": heads, "vdim": vdim}, mlp, weights_of)


def attention_layer(heads: int, kv_heads: int, dim: int, rot_dims: int, base: float, factor: Optional[float], scale: float,
                    mlp: Optional[dict], weights_of: Optional[int] = None) -> dict:
    rot = {"base": base, "dims": rot_dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return _entry("attention", {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot, "scale": scale, "vdim": dim},
                  mlp, weights_of)


def lightning_layer(heads: int, dim: int, vdim: int, decay, mlp: Optional[dict], weights_of: Optional[int] = None) -> dict:
    return _entry("lightning", {"decay": [float(d) for d in decay], "dim": dim, "heads": heads, "vdim": vdim}, mlp,
                  weights_of)


class Figonex(Model):
    architecture = "figonex"
    default_source = "native"

    def __init__(self, config: Optional[FigonexConfig] = None, **kwargs) -> None:
        config = config if config is not None else FigonexConfig()
        super().__init__(config.updated(**kwargs))

    @classmethod
    def config_from_json(cls, values: dict) -> FigonexConfig:
        return _config_from_json(values)

    def config_json(self) -> dict:
        c = self.config
        return {"architecture": "Figonex", "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps},
                "embedding": {"scale": c.embedding_scale}, "layers": copy.deepcopy(c.layers)}

    # ---- specs -------------------------------------------------------------------------------
    def _mixer_spec(self, layer: dict) -> MixerSpec:
        c, m = self.config, layer["mixer"]
        eps = float(c.norm_eps)
        if layer["type"] == "mlstm":
            return MixerSpec("mlstm", dim=c.width, nheads=int(m["heads"]), head_dim=int(m["dim"]),
                             options=(("vdim", int(m["vdim"])), ("gate_cap", float(m["gate_cap"])), ("eps", eps)))
        if layer["type"] == "lightning":
            return MixerSpec("lightning_attention", dim=c.width, nheads=int(m["heads"]), head_dim=int(m["dim"]),
                             options=(("vdim", int(m["vdim"])), ("decay", tuple(float(d) for d in m["decay"])), ("eps", eps)))
        rot = m.get("rot") or {}
        dims = int(rot.get("dims", 0))
        position = PositionSpec("none")
        if dims:
            factor = (rot.get("scaling") or {}).get("factor")
            position = PositionSpec("rope", head_dim=dims, theta=float(rot["base"]),
                                    scaling=() if factor is None else (("rope_type", "linear"), ("factor", float(factor))))
        return MixerSpec("sink_attention", dim=c.width, nheads=int(m["heads"]), kvheads=int(m["kv_heads"]),
                         head_dim=int(m["dim"]), scale=float(m["scale"]), position=position,
                         options=(("vdim", int(m["dim"])), ("values", "keys"), ("rot_dims", dims), ("pairing", "halves"),
                                  ("qk_norm", "before"), ("eps", eps), ("sink_logit", 0.0), ("gate", "head")))

    def decoder_spec(self) -> DecoderSpec:
        c = self.config
        scaled = NormSpec("layernorm", c.width, float(c.norm_eps), options=(("layer_scale", True),))
        blocks = []
        for layer in c.layers:
            ff = None
            if layer.get("mlp") is not None:
                ff = FeedForwardSpec("glu", dim=c.width, hidden=int(layer["mlp"]["ff"]), activation="silu")
            j = None if layer.get("weights_of") is None else c.owner_of(len(blocks))
            blocks.append(BlockSpec(mixer=self._mixer_spec(layer), feed_forward=ff, mixer_norm=scaled,
                                    feed_forward_norm=scaled if ff is not None else None, arrangement="output_norm",
                                    names=("norm1", "mix", "norm2", "mlp"), weights_of=None if j is None else int(j)))
        return DecoderSpec(vocab_size=c.vocab, dim=c.width, layers=tuple(blocks),
                           schedule=tuple(LayerCall(i) for i in range(len(blocks))),
                           final_norm=NormSpec("layernorm", c.width, float(c.norm_eps)), tie_head=False,
                           max_positions=int(c.max_positions), names=("embedding", "layers", "final_norm", "head"),
                           embedding_scale=float(c.embedding_scale))

    def checkpoint_layout(self) -> List[TensorLayout]:
        c = self.config
        d = c.width
        out = [TensorLayout("embed", (c.vocab, d), "embedding")]
        for i, layer in enumerate(c.layers):
            if layer.get("weights_of") is not None:
                continue
            p, m = f"l{i}.", layer["mixer"]
            out += [TensorLayout(p + "norm1", (d,), "gain"), TensorLayout(p + "ls1", (d,), "gain")]
            h, k = int(m["heads"]), int(m["dim"])
            q = p + "mix."
            if layer["type"] == "attention":
                g = int(m["kv_heads"])
                out += [TensorLayout(q + "q", (h * k, d), "matrix"), TensorLayout(q + "k", (g * k, d), "matrix"),
                        TensorLayout(q + "q.norm", (k,), "gain"), TensorLayout(q + "k.norm", (k,), "gain"),
                        TensorLayout(q + "g", (h, d), "matrix"), TensorLayout(q + "o", (d, h * k), "matrix")]
            else:
                v = int(m["vdim"])
                out += [TensorLayout(q + "q", (h * k, d), "matrix"), TensorLayout(q + "k", (h * k, d), "matrix"),
                        TensorLayout(q + "v", (h * v, d), "matrix"), TensorLayout(q + "g", (h * v, d), "matrix"),
                        TensorLayout(q + "norm", (h * v,), "gain"), TensorLayout(q + "o", (d, h * v), "matrix")]
                if layer["type"] == "mlstm":
                    out += [TensorLayout(q + "i", (h, d), "matrix"), TensorLayout(q + "i.b", (h,), "around_zero"),
                            TensorLayout(q + "f", (h, d), "matrix"), TensorLayout(q + "f.b", (h,), "around_zero")]
            if layer.get("mlp") is not None:
                f = int(layer["mlp"]["ff"])
                out += [TensorLayout(p + "norm2", (d,), "gain"), TensorLayout(p + "ls2", (d,), "gain"),
                        TensorLayout(p + "mlp.gate", (f, d), "matrix"), TensorLayout(p + "mlp.up", (f, d), "matrix"),
                        TensorLayout(p + "mlp.down", (d, f), "matrix")]
        out += [TensorLayout("final.norm", (d,), "gain"), TensorLayout("head", (c.vocab, d), "head")]
        return out


# ---- checkpoint adapter ------------------------------------------------------------------------------
_LAYER = re.compile(r"^l(\d+)\.(.*)$")
_RENAMED = {  # checkpoint name within a layer -> the engine's
    "norm1": "norm1.weight", "ls1": "norm1.scale", "norm2": "norm2.weight", "ls2": "norm2.scale",
    "mlp.down": "mlp.w2.weight", "mix.o": "mix.dense.weight", "mix.norm": "mix.norm",
    "mix.q.norm": "mix.q_norm", "mix.k.norm": "mix.k_norm",
}


def _fuse(held: Dict[str, torch.Tensor], names, out: Dict[str, torch.Tensor], target: str, rows: int = 0) -> bool:
    """Concatenates the tensors ``names`` of ``held`` along their rows into out[target] if all of them are there, with
    rows of zeros behind them up to ``rows``."""
    if not all(n in held for n in names):
        return False
    parts = [held.pop(n) for n in names]
    have = sum(p.shape[0] for p in parts)
    if rows > have:
        parts.append(torch.zeros((rows - have,) + tuple(parts[0].shape[1:]), dtype=parts[0].dtype, device=parts[0].device))
    out[target] = torch.cat(parts, dim=0)
    return True


def _native_to_engine(tensors: Dict[str, torch.Tensor], config: FigonexConfig = None, **_) -> Dict[str, torch.Tensor]:
    """Names and layouts of the checkpoint -> the engine's.  Incomplete sets (a projection without its partners) are
    passed on under their own names, so that the loader's one error lists them."""
    out: Dict[str, torch.Tensor] = {}
    layers: Dict[int, Dict[str, torch.Tensor]] = {}
    top = {"embed": "embedding.weight", "final.norm": "final_norm.weight", "head": "head.weight"}
    for name, t in tensors.items():
        m = _LAYER.match(name)
        if m:
            layers.setdefault(int(m.group(1)), {})[m.group(2)] = t
        else:
            out[top.get(name, name)] = t
    for i, held in layers.items():
        p = f"layers.{i}."
        entry = config.layers[i] if config is not None and i < len(config.layers) else None
        if entry is not None:
            m, kind = entry["mixer"], entry["type"]
            h, k = int(m["heads"]), int(m["dim"])
            if kind == "attention":
                rows = SinkAttention.fused_rows(h, int(m["kv_heads"]), k, k, True, "head")
                _fuse(held, ["mix.q", "mix.k", "mix.g"], out, p + "mix.in_proj.weight", rows)
            elif kind == "lightning":
                _fuse(held, ["mix.q", "mix.k", "mix.v", "mix.g"], out, p + "mix.in_proj.weight",
                      LightningAttention.fused_rows(h, k, int(m["vdim"])))
            elif all(n in held for n in ("mix.i.b", "mix.f.b")):
                if _fuse(held, ["mix.q", "mix.k", "mix.v", "mix.g", "mix.i", "mix.f"], out, p + "mix.in_proj.weight",
                         MatrixLSTM.fused_rows(h, k, int(m["vdim"]))):
                    _fuse(held, ["mix.i.b", "mix.f.b"], out, p + "mix.gate_bias")
        _fuse(held, ["mlp.gate", "mlp.up"], out, p + "mlp.wg1_fused.weight")
        for k in list(held):
            if k in _RENAMED:
                out[p + _RENAMED[k]] = held.pop(k)
        for k, t in held.items():  # whatever found no place keeps its name and is reported
            out[f"l{i}.{k}"] = t
    return out


register_architecture("figonex", Figonex, config_json_names=("Figonex",))
register_adapter_step("figonex", "native_to_engine", _native_to_engine)
register_adapter("figonex", "native", ["native_to_engine"])


# ---- variants ----------------------------------------------------------------------------------------
def rotating(n_layers: int, width: int, vocab: int, ff: int, heads: int, kv_heads: int, dim: int, rot_dims: int,
             memory_heads: int, memory_dim: int, memory_vdim: int, embedding_scale: float = 1.0, gate_cap: float = 15.0,
             base: float = 10000.0) -> FigonexConfig:
    """Layers that take turns: a gated matrix memory, attention, attention, a decaying matrix memory, each with a dense
    feed-forward.  The decays of the last kind are spread between 0.9 and 0.999 over its heads."""
    mlp = dense_mlp(ff)
    decays = [1.0 - 0.1 * 0.01 ** (i / max(1, memory_heads - 1)) for i in range(memory_heads)]
    kinds = [mlstm_layer(memory_heads, memory_dim, memory_vdim, gate_cap, mlp),
             attention_layer(heads, kv_heads, dim, rot_dims, base, None, dim ** -0.5, mlp),
             attention_layer(heads, kv_heads, dim, rot_dims, base, None, dim ** -0.5, mlp),
             lightning_layer(memory_heads, memory_dim, memory_vdim, decays, mlp)]
    return FigonexConfig(vocab=vocab, width=width, embedding_scale=embedding_scale,
                         layers=[copy.deepcopy(kinds[i % 4]) for i in range(n_layers)])


def _factory(config: FigonexConfig):
    def make(**kwargs) -> Figonex:
        return Figonex(copy.deepcopy(config), **kwargs)

    return make


# "tiny": for trying things out.  "8b-shape": layers of the width of the Llama-3-8B benchmark (4,096 wide; 32 heads of
# 128 over 8; matrix memories of 32 heads of 128 x 128; a feed-forward of 14,336), with which the two are measured side
# by side.
register_model("figonex", "tiny", _factory(rotating(4, 64, 256, 96, 4, 2, 16, 8, 2, 16, 24, embedding_scale=4.0)))
register_model("figonex", "8b-shape", _factory(rotating(32, 4096, 128256, 14336, 32, 8, 128, 64, 32, 128, 128,
                                                        embedding_scale=8.0)))
