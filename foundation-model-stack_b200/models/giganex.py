"""Giganex: a decoder whose layers run their mixer and their feed-forward side by side on the same stream,
x += mixer(norm1(x)) + mlp(norm2(x)), with norms taken in equal runs of the row.  A layer's mixer is one of

    "attention"          grouped-query attention whose queries and keys are rotated in their first ``rot.dims`` values (value
                         i with value i + dims / 2, frequencies stretched by a ramp, a constant on sines and cosines) and
                         then divided by their root mean square; a query sees the keys of its own run of ``mask.size``
                         positions (runs are counted from the sequence's position 0)
    "parallel"           two mixers on the same input: attention with biases, no rotation, scores capped by a tanh, all
                         earlier keys, a sigmoid gate on the heads' results and a bias on the output — beside a gated delta
                         rule with one decay a head and a silu gate after its norm; weighted by ``left_scale`` / ``right_scale``
    "latent_attention"   queries through a normed latent, keys and values from one cached latent row and one rotated key
                         part shared by the heads; the row at position p sees the last ``mask.size`` keys

and its feed-forward a dense gated unit ("dense"), routed experts ("moe": softmax scores, a correction on the choice
only, weights over their sum times ``router.scale``, experts Wdown relu(Wup h)^2), or none (null).

This file is all that is specific to the architecture: its ``config.json`` (every size and constant is read from it:
``vocab``, ``width``, ``norm.eps``, ``norm.groups``, and ``layers``, each entry with its ``type``, the sizes of its
``mixer`` and its ``mlp`` or null), the ``DecoderSpec`` that configuration means, and the checkpoint's tensor names:

    embed [vocab, width]    final.norm [width]    head [vocab, width]        l<i>.norm1, l<i>.norm2 [width]
    attention:  l<i>.mix.q, .k, .v, .o
    parallel:   l<i>.mix.left.q, .q.b, .k, .k.b, .v, .v.b, .g, .o, .o.b
                l<i>.mix.right.q, .q.conv, .k, .k.conv, .v, .v.conv, .b, .a [heads, width], .A_log, .dt_bias [heads],
                .norm [vdim], .g, .o
    latent:     l<i>.mix.dq, .dq.norm, .uq, .dkv, .dkv.norm, .uk, .uv, .o
    dense:      l<i>.mlp.gate, .up [ff, width], .down [width, ff]
    moe:        l<i>.mlp.router [experts, width], .correction [experts], .e<j>.up [ff, width], .e<j>.down [width, ff]

Linear weights are stored [out, in].  The adapter fuses what reads the same input into one matrix each ([q; k; v],
[q; k; v; g] with bias [q.b; k.b; v.b; 0], [q; k; v; b; a; zeros; g] with the three convolutions' taps, [dkv; dq],
[gate; up]) and stacks the experts.
"""
from __future__ import annotations

import copy
import dataclasses
import re
from typing import Any, Dict, List, Optional

import torch

from ..config.model_config import ModelConfig
from ..config.specs import BlockSpec, DecoderSpec, FeedForwardSpec, LayerCall, MixerSpec, NormSpec, PositionSpec
from ..parts.state_space import GatedDeltaRule
from ..weights.adapters import register_adapter, register_adapter_step
from ..weights.sources import TensorLayout
from . import register_architecture, register_model
from .base import Model

LAYER_TYPES = ("attention", "parallel", "latent_attention")
MLP_KINDS = ("dense", "moe")


@dataclasses.dataclass
class GiganexConfig(ModelConfig):
    vocab: int = 512
    width: int = 256
    norm_eps: float = 1e-6
    norm_groups: int = 1
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    max_positions: int = 131072  # how long a sequence may get; nothing in the model depends on it

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.norm_groups <= 0 or self.width % self.norm_groups:
            raise ValueError(f"vocab {self.vocab}, width {self.width}, norms in {self.norm_groups} runs")
        for i, layer in enumerate(self.layers):
            if layer.get("type") not in LAYER_TYPES:
                raise ValueError(f"layer {i}: type {layer.get('type')!r}; known: {', '.join(LAYER_TYPES)}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in MLP_KINDS:
                raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r}; known: {', '.join(MLP_KINDS)}, or null")


def _config_from_json(values: Dict[str, Any]) -> GiganexConfig:
    if values.get("architecture") != "Giganex":
        raise ValueError(f"config.json is of architecture {values.get('architecture')!r}, not Giganex")
    absent = [k for k in ("vocab", "width", "layers", "norm") if k not in values]
    if absent:
        raise ValueError(f"config.json lacks {absent}")
    return GiganexConfig(vocab=int(values["vocab"]), width=int(values["width"]), norm_eps=float(values["norm"]["eps"]),
                         norm_groups=int(values["norm"].get("groups", 1)), layers=copy.deepcopy(values["layers"]),
                         max_positions=int(values.get("max_positions", 131072)))


# ---- layer entries as config.json has them -----------------------------------------------------------
def dense_mlp(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts: int, top: int, ff: int, scale: float) -> dict:
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def rotation(dims: int, base: float, scaling: Optional[dict] = None) -> dict:
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(scaling)
    return out


def attention_layer(heads: int, kv_heads: int, dim: int, vdim: int, rot: dict, scale: float, chunk: int,
                    mlp: Optional[dict]) -> dict:
    return {"type": "attention", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": chunk}, "rot": rot, "scale": scale,
                      "vdim": vdim}}


def latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int, base: float,
                 scaling: Optional[dict], scale: float, window: int, mlp: Optional[dict]) -> dict:
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "mask": {"size": window}, "q_rank": q_rank,
                      "rot": rotation(rot_dim, base, scaling), "rot_dim": rot_dim, "scale": scale, "vdim": vdim}}


def parallel_layer(left: dict, right: dict, left_scale: float, right_scale: float, mlp: Optional[dict]) -> dict:
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "left_scale": left_scale, "right": right, "right_scale": right_scale}}


def capped_side(heads: int, kv_heads: int, dim: int, vdim: int, scale: float, softcap: float) -> dict:
    return {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "softcap": softcap, "vdim": vdim}


def delta_side(heads: int, kv_heads: int, dim: int, vdim: int, conv: int) -> dict:
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}


def _position(rot: Optional[dict]) -> PositionSpec:
    if not rot or not int(rot.get("dims", 0)):
        return PositionSpec("none")
    scaling = rot.get("scaling")
    return PositionSpec("rope", head_dim=int(rot["dims"]), theta=float(rot["base"]),
                        scaling=() if not scaling else (("rope_type", "yarn"), ("factor", float(scaling["factor"])),
                                                        ("original", float(scaling["original"])),
                                                        ("fast", float(scaling["fast"])), ("slow", float(scaling["slow"]))))


class Giganex(Model):
    architecture = "giganex"
    default_source = "native"

    def __init__(self, config: Optional[GiganexConfig] = None, **kwargs) -> None:
        config = config if config is not None else GiganexConfig()
        super().__init__(config.updated(**kwargs))

    @classmethod
    def config_from_json(cls, values: dict) -> GiganexConfig:
        return _config_from_json(values)

    def config_json(self) -> dict:
        c = self.config
        return {"architecture": "Giganex", "vocab": c.vocab, "width": c.width,
                "norm": {"eps": c.norm_eps, "groups": c.norm_groups}, "layers": copy.deepcopy(c.layers)}

    def load(self, source, adapter_source, device, dtype):
        # a size that config.json leaves out is read from the checkpoint's shapes
        shapes = {}

        def rows(name, axis=0):
            if name not in shapes:
                shapes[name] = tuple(source.spec(name)[1]) if name in names else None
            return None if shapes[name] is None else int(shapes[name][axis])

        names = set(source.keys())
        for i, layer in enumerate(self.config.layers):
            p, m = f"l{i}.", layer["mixer"]
            found = {}
            if layer["type"] == "latent_attention":
                found = {"q_rank": rows(p + "mix.dq"), "kv_rank": rows(p + "mix.dkv.norm")}
                target = m
            elif layer["type"] == "parallel":
                found = {"conv": rows(p + "mix.right.q.conv", 1)}
                target = m["right"]
            for key, value in found.items():
                if key not in target and value is not None:
                    target[key] = value
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") == "dense" and "ff" not in mlp and rows(p + "mlp.gate") is not None:
                mlp["ff"] = rows(p + "mlp.gate")
            if mlp is not None and mlp.get("kind") == "moe":
                if "ff" not in mlp.setdefault("expert", {}) and rows(p + "mlp.e0.up") is not None:
                    mlp["expert"]["ff"] = rows(p + "mlp.e0.up")
                if "experts" not in mlp.setdefault("router", {}) and rows(p + "mlp.router") is not None:
                    mlp["router"]["experts"] = rows(p + "mlp.router")
        return super().load(source, adapter_source, device, dtype)

    # ---- specs -------------------------------------------------------------------------------
    def _mixer_spec(self, layer: dict) -> MixerSpec:
        c, m = self.config, layer["mixer"]
        eps = float(c.norm_eps)
        if layer["type"] == "attention":
            rot = m.get("rot") or {}
            return MixerSpec("sink_attention", dim=c.width, nheads=int(m["heads"]), kvheads=int(m.get("kv_heads", m["heads"])),
                             head_dim=int(m["dim"]), bias=False, scale=float(m["scale"]), position=_position(rot),
                             options=(("vdim", int(m.get("vdim", m["dim"]))), ("rot_dims", int(rot.get("dims", 0))), ("pairing", "halves"),
                                      ("qk_norm", True), ("eps", eps), ("chunk", int((m.get("mask") or {}).get("size", 0)))))
        if layer["type"] == "latent_attention":
            rot = m.get("rot") or {}
            return MixerSpec("latent_attention", dim=c.width, nheads=int(m["heads"]), head_dim=int(m["dim"]),
                             scale=float(m["scale"]), window=int((m.get("mask") or {}).get("size", 0)), position=_position(rot),
                             options=(("rot", int(m["rot_dim"])), ("vdim", int(m["vdim"])), ("rank", int(m["kv_rank"])),
                                      ("rot_dims", int(rot.get("dims", m["rot_dim"]))), ("eps", eps),
                                      ("q_rank", int(m["q_rank"])), ("sink", False), ("gate", False), ("pairing", "halves")))
        left, right = m["left"], m["right"]
        left_spec = MixerSpec("sink_attention", dim=c.width, nheads=int(left["heads"]), kvheads=int(left.get("kv_heads", left["heads"])),
                              head_dim=int(left["dim"]), bias=True, scale=float(left["scale"]),
                              options=(("vdim", int(left.get("vdim", left["dim"]))), ("gate", True), ("out_bias", True),
                                       ("softcap", float(left.get("softcap", 0.0)))))
        right_spec = MixerSpec("gated_delta_rule", dim=c.width, nheads=int(right["heads"]), kvheads=int(right.get("kv_heads", right["heads"])),
                               head_dim=int(right["dim"]),
                               options=(("vdim", int(right["vdim"])), ("conv", int(right["conv"])), ("eps", eps),
                                        ("decay", "head")))
        return MixerSpec("parallel", dim=c.width,
                         options=(("left", left_spec), ("right", right_spec), ("left_factor", float(m["left_scale"])),
                                  ("right_factor", float(m["right_scale"]))))

    def _feed_forward_spec(self, mlp: Optional[dict]) -> Optional[FeedForwardSpec]:
        c = self.config
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return FeedForwardSpec("glu", dim=c.width, hidden=int(mlp["ff"]), activation="silu")
        r = mlp["router"]
        return FeedForwardSpec("routed_experts", dim=c.width, hidden=int(mlp["expert"]["ff"]),
                               options=(("experts", int(r["experts"])), ("top", int(r["top"])), ("scoring", "softmax"),
                                        ("correction", True), ("route_scale", float(r.get("scale", 1.0))),
                                        ("unit", "relu_squared")))

    def decoder_spec(self) -> DecoderSpec:
        c = self.config
        norm = NormSpec("group_rmsnorm", c.width, float(c.norm_eps), options=(("groups", int(c.norm_groups)),))
        blocks = []
        for layer in c.layers:
            ff = self._feed_forward_spec(layer.get("mlp"))
            blocks.append(BlockSpec(mixer=self._mixer_spec(layer), feed_forward=ff, mixer_norm=norm,
                                    feed_forward_norm=norm if ff is not None else None, arrangement="parallel_residual",
                                    names=("norm1", "mix", "norm2", "mlp")))
        return DecoderSpec(vocab_size=c.vocab, dim=c.width, layers=tuple(blocks),
                           schedule=tuple(LayerCall(i) for i in range(len(blocks))), final_norm=norm, tie_head=False,
                           max_positions=int(c.max_positions), names=("embedding", "layers", "final_norm", "head"))

    def checkpoint_layout(self) -> List[TensorLayout]:
        c = self.config
        d = c.width
        out = [TensorLayout("embed", (c.vocab, d), "embedding")]
        for i, layer in enumerate(c.layers):
            p, m = f"l{i}.", layer["mixer"]
            out.append(TensorLayout(p + "norm1", (d,), "gain"))
            if layer["type"] == "attention":
                h, g, k, v = (int(m[x]) for x in ("heads", "kv_heads", "dim", "vdim"))
                out += [TensorLayout(p + "mix.q", (h * k, d), "matrix"), TensorLayout(p + "mix.k", (g * k, d), "matrix"),
                        TensorLayout(p + "mix.v", (g * v, d), "matrix"), TensorLayout(p + "mix.o", (d, h * v), "matrix")]
            elif layer["type"] == "latent_attention":
                h, k, r, v, qr, kr = (int(m[x]) for x in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"))
                out += [TensorLayout(p + "mix.dq", (qr, d), "matrix"), TensorLayout(p + "mix.dq.norm", (qr,), "gain"),
                        TensorLayout(p + "mix.uq", (h * (k + r), qr), "matrix"),
                        TensorLayout(p + "mix.dkv", (kr + r, d), "matrix"), TensorLayout(p + "mix.dkv.norm", (kr,), "gain"),
                        TensorLayout(p + "mix.uk", (h * k, kr), "matrix"), TensorLayout(p + "mix.uv", (h * v, kr), "matrix"),
                        TensorLayout(p + "mix.o", (d, h * v), "matrix")]
            else:
                left, right = m["left"], m["right"]
                h, g, k, v = (int(left[x]) for x in ("heads", "kv_heads", "dim", "vdim"))
                q = p + "mix.left."
                out += [TensorLayout(q + "q", (h * k, d), "matrix"), TensorLayout(q + "q.b", (h * k,), "around_zero"),
                        TensorLayout(q + "k", (g * k, d), "matrix"), TensorLayout(q + "k.b", (g * k,), "around_zero"),
                        TensorLayout(q + "v", (g * v, d), "matrix"), TensorLayout(q + "v.b", (g * v,), "around_zero"),
                        TensorLayout(q + "g", (h * v, d), "matrix"), TensorLayout(q + "o", (d, h * v), "matrix"),
                        TensorLayout(q + "o.b", (d,), "around_zero")]
                h, g, k, v, taps = (int(right[x]) for x in ("heads", "kv_heads", "dim", "vdim", "conv"))
                q = p + "mix.right."
                out += [TensorLayout(q + "q", (g * k, d), "matrix"), TensorLayout(q + "q.conv", (g * k, taps), "taps"),
                        TensorLayout(q + "k", (g * k, d), "matrix"), TensorLayout(q + "k.conv", (g * k, taps), "taps"),
                        TensorLayout(q + "v", (h * v, d), "matrix"), TensorLayout(q + "v.conv", (h * v, taps), "taps"),
                        TensorLayout(q + "b", (h, d), "matrix"), TensorLayout(q + "A_log", (h,), "around_zero"),
                        TensorLayout(q + "norm", (v,), "gain"), TensorLayout(q + "a", (h, d), "matrix"),
                        TensorLayout(q + "dt_bias", (h,), "around_zero"), TensorLayout(q + "g", (h * v, d), "matrix"),
                        TensorLayout(q + "o", (d, h * v), "matrix")]
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            out.append(TensorLayout(p + "norm2", (d,), "gain"))
            if mlp["kind"] == "dense":
                f = int(mlp["ff"])
                out += [TensorLayout(p + "mlp.gate", (f, d), "matrix"), TensorLayout(p + "mlp.up", (f, d), "matrix"),
                        TensorLayout(p + "mlp.down", (d, f), "matrix")]
            else:
                f, n = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
                for j in range(n):
                    out += [TensorLayout(p + f"mlp.e{j}.up", (f, d), "matrix"), TensorLayout(p + f"mlp.e{j}.down", (d, f), "matrix")]
                out += [TensorLayout(p + "mlp.router", (n, d), "matrix"), TensorLayout(p + "mlp.correction", (n,), "around_zero")]
        out += [TensorLayout("final.norm", (d,), "gain"), TensorLayout("head", (c.vocab, d), "head")]
        return out


# ---- checkpoint adapter ------------------------------------------------------------------------------
_LAYER = re.compile(r"^l(\d+)\.(.*)$")
_EXPERT = re.compile(r"^mlp\.e(\d+)\.(up|down)$")
_RENAMED = {  # checkpoint name within a layer -> the engine's
    "norm1": "norm1.weight", "norm2": "norm2.weight", "mlp.down": "mlp.w2.weight",
    "mlp.router": "mlp.router.weight", "mlp.correction": "mlp.correction",
    "mix.o": "mix.dense.weight",
    "mix.dq.norm": "mix.q_norm", "mix.uq": "mix.q_up.weight", "mix.dkv.norm": "mix.latent_norm", "mix.uk": "mix.uk",
    "mix.uv": "mix.uv",
    "mix.left.o": "mix.left.dense.weight", "mix.left.o.b": "mix.left.dense.bias",
    "mix.right.A_log": "mix.right.A_log", "mix.right.norm": "mix.right.norm", "mix.right.dt_bias": "mix.right.dt_bias",
    "mix.right.o": "mix.right.dense.weight",
}


def _fuse(held: Dict[str, torch.Tensor], names, out: Dict[str, torch.Tensor], target: str) -> bool:
    """Concatenates the tensors ``names`` of ``held`` along their rows into out[target] if all of them are there."""
    if not all(n in held for n in names):
        return False
    out[target] = torch.cat([held.pop(n) for n in names], dim=0)
    return True


def _native_to_engine(tensors: Dict[str, torch.Tensor], config: GiganexConfig = None, **_) -> Dict[str, torch.Tensor]:
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
        entry = config.layers[i] if config is not None and i < len(config.layers) else {}
        _fuse(held, ["mix.q", "mix.k", "mix.v"], out, p + "mix.in_proj.weight")
        _fuse(held, ["mix.dkv", "mix.dq"], out, p + "mix.in_proj.weight")
        left = ["mix.left.q", "mix.left.k", "mix.left.v", "mix.left.g"]
        biases = ["mix.left.q.b", "mix.left.k.b", "mix.left.v.b"]
        if all(n in held for n in left + biases):
            gate_rows = held["mix.left.g"].shape[0]
            b = [held.pop(n) for n in biases]
            out[p + "mix.left.in_proj.bias"] = torch.cat(b + [torch.zeros(gate_rows, dtype=b[0].dtype, device=b[0].device)])
            _fuse(held, left, out, p + "mix.left.in_proj.weight")
        right = ["mix.right.q", "mix.right.k", "mix.right.v"]
        rest = ["mix.right.b", "mix.right.a", "mix.right.g"]
        if all(n in held for n in right + rest + [n + ".conv" for n in right]) and entry.get("type") == "parallel":
            r = entry["mixer"]["right"]
            gate_col = GatedDeltaRule.gate_column(int(r["kv_heads"]), int(r["dim"]), int(r["heads"]), int(r["vdim"]))
            _fuse(held, [n + ".conv" for n in right], out, p + "mix.right.conv")
            parts = [held.pop(n) for n in right + ["mix.right.b", "mix.right.a"]]
            used = sum(t.shape[0] for t in parts)
            if gate_col > used:  # the gates' rows begin at a multiple of 8
                parts.append(torch.zeros((gate_col - used, parts[0].shape[1]), dtype=parts[0].dtype, device=parts[0].device))
            out[p + "mix.right.in_proj.weight"] = torch.cat(parts + [held.pop("mix.right.g")], dim=0)
        _fuse(held, ["mlp.gate", "mlp.up"], out, p + "mlp.wg1_fused.weight")
        experts: Dict[int, Dict[str, torch.Tensor]] = {}
        for k in list(held):
            m = _EXPERT.match(k)
            if m:
                experts.setdefault(int(m.group(1)), {})[m.group(2)] = held[k]
        n = len(experts)
        if n and sorted(experts) == list(range(n)) and all(len(e) == 2 for e in experts.values()):
            out[p + "mlp.up"] = torch.stack([experts[j]["up"] for j in range(n)])
            out[p + "mlp.down"] = torch.stack([experts[j]["down"] for j in range(n)])
            for j in range(n):
                del held[f"mlp.e{j}.up"], held[f"mlp.e{j}.down"]
        for k in list(held):
            if k in _RENAMED:
                out[p + _RENAMED[k]] = held.pop(k)
        for k, t in held.items():  # whatever found no place keeps its name and is reported
            out[f"l{i}.{k}"] = t
    return out


register_architecture("giganex", Giganex, config_json_names=("Giganex",))
register_adapter_step("giganex", "native_to_engine", _native_to_engine)
register_adapter("giganex", "native", ["native_to_engine"])


# ---- variants ----------------------------------------------------------------------------------------
_STRETCH = {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}


def mixed(n_layers: int, width: int, vocab: int, groups: int, heads: int, kv_heads: int, dim: int, rot_dims: int,
          chunk: int, left_heads: int, left_kv_heads: int, left_dim: int, left_vdim: int, delta_heads: int,
          delta_kv_heads: int, delta_dim: int, delta_vdim: int, latent_heads: int, latent_dim: int, latent_rot: int,
          latent_vdim: int, q_rank: int, kv_rank: int, window: int, ff: int, experts: int, top: int, expert_ff: int) -> GiganexConfig:
    """Layers that take turns: the two mixers side by side, attention over cached latents, attention over runs of
    positions; the first with a dense feed-forward, the others with routed experts."""
    par = parallel_layer(capped_side(left_heads, left_kv_heads, left_dim, left_vdim, left_dim ** -0.5, 30.0),
                         delta_side(delta_heads, delta_kv_heads, delta_dim, delta_vdim, 4), 0.7, 0.6, dense_mlp(ff))
    moe = moe_mlp(experts, top, expert_ff, 2.0)
    lat = latent_layer(latent_heads, latent_dim, latent_rot, latent_vdim, q_rank, kv_rank, 10000.0, _STRETCH,
                       (latent_dim + latent_rot) ** -0.5, window, moe)
    att = attention_layer(heads, kv_heads, dim, dim, rotation(rot_dims, 500000.0, _STRETCH), dim ** -0.5, chunk, moe)
    kinds = [par, lat, att]
    return GiganexConfig(vocab=vocab, width=width, norm_groups=groups,
                         layers=[copy.deepcopy(kinds[i % 3]) for i in range(n_layers)])


def _factory(config: GiganexConfig):
    def make(**kwargs) -> Giganex:
        return Giganex(copy.deepcopy(config), **kwargs)

    return make


# "tiny": for trying things out.  "8b-shape": layers of the width of the Llama-3-8B benchmark (4,096 wide; 32 heads of
# 128 over 8; a delta rule of 16 heads of 128; a latent of 512 under 32 heads of 128 + 64; a dense feed-forward of
# 14,336, or 16 experts of 3,584 of which a token takes 4), with which the two are measured side by side.
register_model("giganex", "tiny", _factory(mixed(3, 64, 256, 2, 4, 2, 16, 8, 24, 4, 2, 16, 32, 2, 1, 16, 24, 4, 16, 16, 16, 24,
                                                 32, 20, 96, 8, 2, 48)))
register_model("giganex", "8b-shape", _factory(mixed(30, 4096, 128256, 8, 32, 8, 128, 128, 8192, 32, 8, 128, 128, 16, 16, 128,
                                                     128, 32, 128, 64, 128, 1536, 512, 4096, 14336, 16, 4, 3584)))
