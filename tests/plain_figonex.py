"""A plain, slow restatement of the Figonex design: whole sequences, no cache, no batching, one function per
mechanism, float64 by default.  It reads a configuration (the config.json dictionary) and the checkpoint's tensors by
their checkpoint names and shares no code with the library.

    embedding        x = embed[token] * embedding.scale
    layer            x = x + ls1 * LN1(mixer(x));  x = x + ls2 * LN2(mlp(x)) where the layer has a feed-forward;
                     LN(y) = (y - mean y) / sqrt(var y + eps) * w; the sublayers read x as it is
    mlstm            q = Wq h / sqrt(dim), k = Wk h, v = Wv h; a = cap tanh((Wi h + bi) / cap),
                     f = logsigmoid(cap tanh((Wf h + bf) / cap)); m' = max(f + m, a) with m = 0 before the first token;
                     S' = exp(f + m - m') S + exp(a - m') k v^T; n' likewise with k; o = S'^T q / (max(|n'.q|, exp(-m')) + 1e-6)
                     out = Wo (o / rms(o) per head * w * sigmoid(Wg h))
    attention        q = Wq h, k = Wk h, v = k as projected; q, k: rms norm per head with a weight, then the first
                     rot.dims values rotated, value i with value i + dims / 2, by p * base^(-2i / dims) / factor;
                     s = q.k * scale, causal; p = exp(s) / (1 + sum exp(s)); out = Wo (sum p v * sigmoid(Wg h) per head)
    lightning        q, k, v = silu(Wq h), silu(Wk h), silu(Wv h); S' = decay_h S + k v^T; o = S'^T q
                     out = Wo (rms norm of all heads together * w * sigmoid(Wg h))
    dense            Wdown (silu(Wgate h) * Wup h)
    output           logits = head LN_final(x)
"""
import math

import torch


def silu(x):
    return x * torch.sigmoid(x)


def layer_norm(x, w, eps):
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate_halves(v, positions, dims, base, factor):
    """v [n, heads, width]: of the first ``dims`` values of every head, value i and value i + dims / 2 turn by the
    angle p * base^(-2i / dims) / factor."""
    if dims == 0:
        return v
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(half)], dtype=v.dtype)
    ang = positions.to(v.dtype)[:, None] * f[None]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = a * cs - b * sn
    out[..., half:dims] = b * cs + a * sn
    return out


def attention(h, m, eps, t, p, first_position=0):
    """t: the checkpoint's tensors, p: the prefix of this mixer's names ('l1.mix.')."""
    n = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ t[p + "q"].T).view(n, H, d)
    k = (h @ t[p + "k"].T).view(n, G, d)
    v = k  # the values are the keys as projected
    q, k = rms_norm(q, t[p + "q.norm"], eps), rms_norm(k, t[p + "k.norm"], eps)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if dims:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        pos = torch.arange(first_position, first_position + n)
        q = rotate_halves(q, pos, dims, float(rot["base"]), factor)
        k = rotate_halves(k, pos, dims, float(rot["base"]), factor)
    out = torch.zeros(n, H, d, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * float(m["scale"])
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), -math.inf)
        top = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - top)
        w = e / (e.sum(-1, keepdim=True) + torch.exp(-top))
        out[:, head] = w @ v[:, kv]
    gate = torch.sigmoid(h @ t[p + "g"].T)  # [n, H]
    return (out * gate[:, :, None]).reshape(n, H * d) @ t[p + "o"].T


def mlstm(h, m, eps, t, p, state=None):
    """``state``: None, or a dictionary that holds S, n, m of every head from an earlier call and is updated."""
    n = h.shape[0]
    H, d, dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (h @ t[p + "q"].T).view(n, H, d) * d ** -0.5
    k = (h @ t[p + "k"].T).view(n, H, d)
    v = (h @ t[p + "v"].T).view(n, H, dv)
    gi = cap * torch.tanh((h @ t[p + "i"].T + t[p + "i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ t[p + "f"].T + t[p + "f.b"]) / cap))
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for head in range(H):
        if state is not None and head in state:
            S, nn, mm = state[head]
        else:
            S, nn, mm = torch.zeros(d, dv, dtype=h.dtype), torch.zeros(d, dtype=h.dtype), torch.zeros((), dtype=h.dtype)
        for i in range(n):
            new = torch.maximum(gf[i, head] + mm, gi[i, head])
            keep, take = torch.exp(gf[i, head] + mm - new), torch.exp(gi[i, head] - new)
            S = keep * S + take * torch.outer(k[i, head], v[i, head])
            nn = keep * nn + take * k[i, head]
            mm = new
            den = torch.maximum(torch.abs(nn @ q[i, head]), torch.exp(-mm)) + 1e-6
            out[i, head] = S.T @ q[i, head] / den
        if state is not None:
            state[head] = (S, nn, mm)
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps)
    out = out.reshape(n, H * dv) * t[p + "norm"] * torch.sigmoid(h @ t[p + "g"].T)
    return out @ t[p + "o"].T


def lightning(h, m, eps, t, p, state=None):
    n = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ t[p + "q"].T).view(n, H, d)
    k = silu(h @ t[p + "k"].T).view(n, H, d)
    v = silu(h @ t[p + "v"].T).view(n, H, dv)
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for head in range(H):
        S = state[head] if state is not None and head in state else torch.zeros(d, dv, dtype=h.dtype)
        decay = float(m["decay"][head])
        for i in range(n):
            S = decay * S + torch.outer(k[i, head], v[i, head])
            out[i, head] = S.T @ q[i, head]
        if state is not None:
            state[head] = S
    out = rms_norm(out.reshape(n, H * dv), t[p + "norm"], eps) * torch.sigmoid(h @ t[p + "g"].T)
    return out @ t[p + "o"].T


def dense(h, t, p):
    return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


MIXERS = {"mlstm": mlstm, "attention": attention, "lightning": lightning}


def logits(cfg, tensors, tokens, dtype=torch.float64, first_position=0, layers_out=None):
    """Logits [len(tokens), vocab] of one whole sequence.  ``layers_out``: a list that receives the stream after every
    layer."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = t["embed"][torch.tensor(list(tokens))] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        j = i
        while cfg["layers"][j].get("weights_of") is not None:
            j = int(cfg["layers"][j]["weights_of"])
        p = f"l{j}."
        if layer["type"] not in MIXERS:
            raise ValueError(layer["type"])
        kwargs = {"first_position": first_position} if layer["type"] == "attention" else {}
        a = MIXERS[layer["type"]](x, layer["mixer"], eps, t, p + "mix.", **kwargs)
        x = x + layer_norm(a, t[p + "norm1"], eps) * t[p + "ls1"]
        if layer.get("mlp") is not None:
            x = x + layer_norm(dense(x, t, p + "mlp."), t[p + "norm2"], eps) * t[p + "ls2"]
        if layers_out is not None:
            layers_out.append(x)
    return layer_norm(x, t["final.norm"], eps) @ t["head"].T
