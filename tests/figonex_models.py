"""Small Figonex configurations and random weights for the tests, written from scratch here (checkpoint names and
config.json keys as a user's folder has them).  The configurations differ from one another in everything a configuration
can say: order of the layers, layers that take an earlier layer's weights, widths, heads and key heads (one, some, as
many as query heads), key and value sizes of the matrix memories (equal, values wider, values narrower, no multiples of
8, more than one run of value columns), rotated sizes (none, a part, all of the head), frequency scaling or none,
attention scales, gate caps, decays (1.0, near 1, fast), the embedding's factor (1 and others), eps, layers without a
feed-forward."""
import json
import os

import torch


def dense(ff):
    return {"kind": "dense", "ff": ff}


def _entry(kind, mixer, mlp, weights_of):
    out = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def mlstm(heads, dim, vdim, cap, mlp, weights_of=None):
    return _entry("mlstm", {"dim": dim, "gate_cap": cap, "heads": heads, "vdim": vdim}, mlp, weights_of)


def attention(heads, kv_heads, dim, rot_dims, base, factor, scale, mlp, weights_of=None):
    rot = {"base": base, "dims": rot_dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return _entry("attention", {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot, "scale": scale, "vdim": dim},
                  mlp, weights_of)


def lightning(heads, dim, vdim, decay, mlp, weights_of=None):
    return _entry("lightning", {"decay": list(decay), "dim": dim, "heads": heads, "vdim": vdim}, mlp, weights_of)


def config(vocab, width, scale, layers, eps=1e-5):
    return {"architecture": "Figonex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


_P_ATT = attention(4, 1, 24, 6, 50.0, 4.0, 0.2, dense(40))
_P_MEM = mlstm(3, 12, 20, 8.0, dense(40))
_P_LIN = lightning(2, 12, 20, (0.5, 0.995), dense(40))
_S_ATT = attention(8, 2, 128, 64, 1000.0, None, 0.09, dense(72))
_W_ATT = attention(8, 2, 128, 128, 10000.0, None, 0.088, dense(1408))

CONFIGS = {
    # attention first; one key head; a fourth of the head rotated with scaled frequencies; values wider than keys in the
    # memories; the later layers run with the weights of the earlier ones, in another order, with states of their own
    "p": config(97, 48, 3.0, [_P_ATT, _P_MEM, _P_LIN, dict(_P_LIN, weights_of=2), dict(_P_ATT, weights_of=0),
                              dict(_P_MEM, weights_of=1)], eps=1e-4),
    # as many key heads as query heads, the whole head rotated, no scaling; one head in either memory, values narrower
    # than keys; a decay of exactly 1; a layer without a feed-forward; an embedding factor of 1
    "q": config(130, 64, 1.0, [lightning(1, 40, 8, (1.0,), None), attention(2, 2, 16, 16, 300.0, None, 0.3, dense(36)),
                               mlstm(1, 40, 8, 20.0, dense(36)), attention(2, 2, 16, 16, 300.0, None, 0.3, None)]),
    # no size a multiple of 8; nothing rotated in one attention layer, two values in the other; a small cap
    "r": config(75, 36, 0.5, [mlstm(5, 6, 7, 2.5, dense(22)), attention(3, 1, 10, 0, 20.0, None, 0.5, dense(22)),
                              lightning(3, 5, 9, (0.9, 0.3, 0.97), None), attention(6, 3, 6, 2, 20.0, 1.5, 0.5, dense(22))],
                eps=1e-6),
    # heads of 128 (the tensor-core attention kernels in bfloat16); memories of 96 x 40 and 128 x 64 (two runs of value
    # columns), the second attention layer with the first one's weights
    "s": config(101, 64, 2.0, [_S_ATT, mlstm(2, 96, 40, 10.0, dense(72)), lightning(2, 128, 64, (0.98, 0.9), dense(72)),
                               dict(_S_ATT, weights_of=0)]),
    # a width at which the products of a prompt run on the tensor-core kernels in bfloat16: memories of 128 x 128 and
    # 128 x 64 (sixteen state rows a thread), eight heads of 128 over two, a feed-forward of 1,408
    "w": config(2000, 512, 8.0, [mlstm(4, 128, 128, 15.0, dense(1408)), _W_ATT,
                                 lightning(4, 128, 64, (0.9, 0.99, 0.999, 0.6), dense(1408)), dict(_W_ATT, weights_of=1)]),
}


def tensors(cfg, seed, std=0.08, wide=4.0):
    """Matrices ~ N(0, std) with the projections of queries, keys and gates ``wide`` times wider (a tiny model with
    N(0, 0.02) has near-uniform attention rows in which a dropped key hardly shows), norm weights and layer scales around
    0.8 with some exact zeros, gains of the query and key norms around 1.4, forget-gate biases between 2 and 6 (a memory of
    tens of tokens) and input-gate biases around -0.5, all rounded to bfloat16 as a checkpoint stores them."""
    g = torch.Generator().manual_seed(seed)
    out = {}

    def mat(name, *shape, s=std):
        out[name] = (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    def around(name, n, centre, spread, zeros=0):
        t = centre + spread * (2 * torch.rand(n, generator=g) - 1)
        if zeros:
            t[torch.randperm(n, generator=g)[:zeros]] = 0.0
        out[name] = t.to(torch.bfloat16)

    d = cfg["width"]
    mat("embed", cfg["vocab"], d, s=0.06)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        h, k = m["heads"], m["dim"]
        around(p + "norm1", d, 0.8, 0.7, zeros=2), around(p + "ls1", d, 0.85, 0.4)
        q = p + "mix."
        if layer["type"] == "attention":
            kv = m["kv_heads"]
            mat(q + "q", h * k, d, s=wide * std), mat(q + "k", kv * k, d, s=wide * std)
            around(q + "q.norm", k, 1.4, 0.9), around(q + "k.norm", k, 1.4, 0.9)
            mat(q + "g", h, d, s=wide * std), mat(q + "o", d, h * k)
        else:
            v = m["vdim"]
            mat(q + "q", h * k, d, s=wide * std), mat(q + "k", h * k, d, s=wide * std), mat(q + "v", h * v, d, s=wide * std)
            mat(q + "g", h * v, d, s=wide * std), around(q + "norm", h * v, 1.0, 0.4), mat(q + "o", d, h * v)
            if layer["type"] == "mlstm":
                mat(q + "i", h, d, s=wide * std), mat(q + "f", h, d, s=wide * std)
                around(q + "i.b", h, -0.5, 0.7), around(q + "f.b", h, 4.0, 2.0)
        if layer["mlp"] is not None:
            f = layer["mlp"]["ff"]
            around(p + "norm2", d, 0.8, 0.7, zeros=2), around(p + "ls2", d, 0.85, 0.4)
            mat(p + "mlp.gate", f, d, s=wide * std), mat(p + "mlp.up", f, d, s=wide * std), mat(p + "mlp.down", d, f)
    around("final.norm", d, 0.8, 0.7, zeros=1)
    mat("head", cfg["vocab"], d)
    return out


def write_folder(path, cfg, weights):
    from fms_b200.weights.safetensors_io import write_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.contiguous() for k, v in weights.items()}, {})
    return path


def prompt(cfg, length, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, cfg["vocab"], (length,), generator=g).tolist()
