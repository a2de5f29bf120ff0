"""Small Giganex configurations and random weights for the tests, written from scratch here (checkpoint names and
config.json keys as a user's folder has them).  The configurations differ from one another in everything a configuration
can say: the order of the layers and which kinds occur, widths, the runs of the norms (one, some, many), heads and groups
(one, some, as many as heads), key and value sizes (equal, values wider, values narrower, no multiples of 8), rotated
sizes (none, a part, all of the head), stretched frequencies or plain ones, sizes of runs and windows (smaller than a
cache block, between, larger than a decode split), caps, the two mixers' weights, taps of the convolutions (one to five),
the ranks of both latents, experts (2 to 12, of which 1 to all are taken), router scales, layers with a dense
feed-forward, with experts and with none."""
import json
import os

import torch


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def rot(dims, base, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = scaling
    return out


def attention(heads, kv_heads, dim, vdim, r, scale, chunk, mlp):
    return {"type": "attention", "mlp": mlp, "mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": chunk},
                                                       "rot": r, "scale": scale, "vdim": vdim}}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, base, scaling, scale, window, mlp):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "mask": {"size": window}, "q_rank": q_rank,
                      "rot": rot(rot_dim, base, scaling), "rot_dim": rot_dim, "scale": scale, "vdim": vdim}}


def left(heads, kv_heads, dim, vdim, scale, softcap):
    return {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "softcap": softcap, "vdim": vdim}


def right(heads, kv_heads, dim, vdim, conv):
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}


def parallel(l, r, left_scale, right_scale, mlp):
    return {"type": "parallel", "mlp": mlp, "mixer": {"left": l, "left_scale": left_scale, "right": r, "right_scale": right_scale}}


def config(vocab, width, groups, layers, eps=1e-5):
    return {"architecture": "Giganex", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "layers": layers}


_STRETCH_A = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
_STRETCH_B = {"factor": 16.0, "original": 40, "fast": 4.0, "slow": 0.5}

CONFIGS = {
    # latent attention first; norms in three runs; a window of 20 (inside one cache block), a run of 50; values narrower
    # than keys; a fourth of the head rotated with stretched frequencies whose three ranges all occur; one group of keys
    "p": config(97, 48, 3, [latent(3, 10, 6, 12, 14, 18, 100.0, _STRETCH_A, 0.25, 20, moe(5, 2, 20, 1.5)),
                            parallel(left(4, 1, 24, 8, 0.2, 5.0), right(4, 2, 12, 20, 2), 0.7, 1.3, dense(40)),
                            attention(4, 1, 24, 8, rot(6, 50.0, _STRETCH_A), 0.2, 50, moe(5, 2, 20, 1.5)),
                            parallel(left(4, 1, 24, 8, 0.2, 5.0), right(4, 2, 12, 20, 2), 0.7, 1.3, None)], eps=1e-4),
    # norms in one run; values wider than keys, the whole head rotated, plain frequencies, as many key heads as query
    # heads everywhere, five taps, a layer without a feed-forward, every expert taken (top = experts), a run of 64 (a
    # cache block) and a window of 300 (more than a decode split), mixer weights of 1, a router scale of 1
    "q": config(130, 64, 1, [attention(2, 2, 16, 40, rot(16, 300.0), 0.3, 64, None),
                             parallel(left(2, 2, 16, 40, 0.3, 50.0), right(3, 3, 8, 8, 5), 1.0, 1.0, moe(3, 3, 24, 1.0)),
                             latent(2, 16, 16, 40, 24, 32, 300.0, None, 0.2, 300, dense(36)),
                             attention(2, 2, 16, 40, rot(16, 300.0), 0.3, 64, dense(36))]),
    # no size a multiple of 8; norms in as many runs as a row has pairs; nothing rotated in the attention layer; one tap
    # (no convolution at all); one expert of two; a window of one (a row sees itself only) and a run of one
    "r": config(75, 36, 18, [parallel(left(3, 1, 10, 6, 0.5, 2.0), right(2, 1, 6, 5, 1), 0.4, 0.9, dense(22)),
                             attention(6, 3, 6, 10, rot(0, 20.0), 0.5, 1, moe(2, 1, 9, 3.0)),
                             latent(5, 6, 2, 3, 5, 7, 20.0, _STRETCH_B, 0.4, 1, moe(2, 1, 9, 3.0)),
                             attention(3, 1, 10, 6, rot(2, 20.0, _STRETCH_B), 0.5, 7, None)], eps=1e-6),
    # heads of 128 keys and 64 values and of 64 and 64 (the tensor-core attention kernels in bfloat16), a latent of 64 with
    # 32 rotated values (the tensor-core kernel over latents), a delta rule with 96 key channels and 40 values, twelve
    # experts of which four; a run of 150 and a window of 210 (both over block edges)
    "s": config(101, 64, 4, [parallel(left(8, 2, 128, 64, 0.09, 30.0), right(2, 1, 96, 40, 4), 1.0, 0.25, moe(12, 4, 16, 2.5)),
                             attention(4, 4, 64, 64, rot(32, 10000.0, {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0}),
                                       0.125, 150, dense(72)),
                             latent(4, 32, 32, 48, 40, 64, 5000.0, {"factor": 2.0, "original": 256, "fast": 16.0, "slow": 2.0},
                                    0.125, 210, moe(12, 4, 16, 2.5))]),
}


def random_config(seed):
    """A configuration drawn from a seed: two to five layers of any kinds in any order, with sizes from small lists
    (widths 64 to 320, norms in 1 to 16 runs, 1 to 16 heads of 16 to 128, runs and windows from 1 to beyond the prompt,
    1 to 5 taps, 4 to 16 experts of which 1 to all)."""
    import random

    r = random.Random(seed)
    width = r.choice([64, 96, 128, 192, 256, 320])
    groups = r.choice([g for g in (1, 2, 4, 8, 16) if width % g == 0])

    def mlp():
        kind = r.choice(["dense", "moe", "moe", None])
        if kind == "dense":
            return dense(r.choice([48, 100, 360]))
        if kind == "moe":
            e = r.choice([4, 8, 16, 6])
            return moe(e, r.choice([1, 2, 4, e]), r.choice([32, 88, 40]), r.choice([1.0, 1.5, 2.5]))
        return None

    def scaling():
        return r.choice([None, {"factor": r.choice([2.0, 8.0, 32.0]), "original": r.choice([64, 500, 3000]),
                                "fast": r.choice([8.0, 32.0]), "slow": r.choice([1.0, 2.0])}])

    layers = []
    for _ in range(r.choice([2, 3, 4, 5])):
        kind = r.choice(["attention", "parallel", "latent_attention"])
        if kind == "attention":
            kv = r.choice([1, 2, 4])
            h, d = kv * r.choice([1, 2, 4]), r.choice([16, 32, 64, 128, 48])
            layers.append(attention(h, kv, d, r.choice([d, 32, 64, 128]), rot(r.choice([0, d, d // 2, 8]), r.choice([10000.0, 200000.0, 500.0]), scaling()),
                                    r.choice([d ** -0.5, 0.125, 0.3]), r.choice([1, 17, 64, 110, 200, 1000]), mlp()))
        elif kind == "parallel":
            kv, kv2 = r.choice([1, 2, 4]), r.choice([1, 2, 3])
            h, d = kv * r.choice([1, 2, 4]), r.choice([16, 32, 64, 128])
            layers.append(parallel(left(h, kv, d, r.choice([d, 32, 64, 128]), r.choice([d ** -0.5, 0.125]), r.choice([5.0, 25.0, 50.0])),
                                   right(kv2 * r.choice([1, 2]), kv2, r.choice([16, 32, 64, 40]), r.choice([16, 32, 64, 24]), r.choice([1, 2, 3, 4, 5])),
                                   r.choice([0.5, 0.8, 1.0]), r.choice([0.5, 1.0, 1.2]), mlp()))
        else:
            d, rd = r.choice([16, 32, 64]), r.choice([8, 16, 32, 64])
            layers.append(latent(r.choice([2, 4, 8, 3]), d, rd, r.choice([16, 32, 64, 128]), r.choice([24, 64, 96, 128]), r.choice([32, 64, 96, 128, 40]),
                                 r.choice([10000.0, 40000.0]), scaling(), (d + rd) ** -0.5, r.choice([1, 20, 64, 130, 300, 1000]), mlp()))
    return config(r.choice([77, 200, 450, 513]), width, groups, layers, eps=r.choice([1e-5, 1e-6]))


def tensors(cfg, seed, std=0.08):
    """Matrices ~ N(0, std) with the projections of queries, keys and gates four times wider (a tiny model with
    N(0, 0.02) has near-uniform attention rows in which a dropped key hardly shows), norm weights around one, taps
    around 1 / taps, all rounded to bfloat16 as a checkpoint stores them."""
    g = torch.Generator().manual_seed(seed)
    out = {}

    def mat(name, *shape, s=std):
        out[name] = (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    def around(name, n, centre, spread):
        out[name] = (centre + spread * (2 * torch.rand(n, generator=g) - 1)).to(torch.bfloat16)

    d = cfg["width"]
    mat("embed", cfg["vocab"], d, s=1.0)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        around(p + "norm1", d, 1.0, 0.4)
        if layer["type"] == "attention":
            h, kv, k, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mat(p + "mix.q", h * k, d, s=4 * std), mat(p + "mix.k", kv * k, d, s=4 * std), mat(p + "mix.v", kv * v, d, s=4 * std)
            mat(p + "mix.o", d, h * v)
        elif layer["type"] == "latent_attention":
            h, k, r, v, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            mat(p + "mix.dq", qr, d, s=4 * std), around(p + "mix.dq.norm", qr, 1.0, 0.4), mat(p + "mix.uq", h * (k + r), qr, s=6 * std)
            mat(p + "mix.dkv", kr + r, d, s=4 * std), around(p + "mix.dkv.norm", kr, 1.0, 0.4)
            mat(p + "mix.uk", h * k, kr, s=6 * std), mat(p + "mix.uv", h * v, kr, s=4 * std), mat(p + "mix.o", d, h * v)
        else:
            l, r = m["left"], m["right"]
            h, kv, k, v = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            q = p + "mix.left."
            mat(q + "q", h * k, d, s=4 * std), mat(q + "q.b", h * k, s=0.5)
            mat(q + "k", kv * k, d, s=4 * std), mat(q + "k.b", kv * k, s=0.5)
            mat(q + "v", kv * v, d, s=4 * std), mat(q + "v.b", kv * v, s=0.5)
            mat(q + "g", h * v, d, s=4 * std), mat(q + "o", d, h * v), mat(q + "o.b", d, s=0.3)
            h, kv, k, v, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            q = p + "mix.right."
            for n, rows in (("q", kv * k), ("k", kv * k), ("v", h * v)):
                mat(q + n, rows, d, s=4 * std)
                mat(q + n + ".conv", rows, taps, s=0.6)
            mat(q + "b", h, d, s=4 * std), mat(q + "a", h, d, s=4 * std)
            around(q + "A_log", h, -1.0, 1.0), around(q + "norm", v, 1.0, 0.4), mat(q + "dt_bias", h, s=1.0)
            mat(q + "g", h * v, d, s=4 * std), mat(q + "o", d, h * v)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        around(p + "norm2", d, 1.0, 0.4)
        if mlp["kind"] == "dense":
            f = mlp["ff"]
            mat(p + "mlp.gate", f, d, s=4 * std), mat(p + "mlp.up", f, d, s=4 * std), mat(p + "mlp.down", d, f)
        else:
            f, n = mlp["expert"]["ff"], mlp["router"]["experts"]
            for j in range(n):
                mat(p + f"mlp.e{j}.up", f, d, s=4 * std), mat(p + f"mlp.e{j}.down", d, f)
            mat(p + "mlp.router", n, d, s=6 * std), mat(p + "mlp.correction", n, s=0.2)
    around("final.norm", d, 1.0, 0.4)
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
