"""A plain, slow restatement of the Giganex design: whole sequences, no cache, no batching, one function per
mechanism, float64 by default.  It reads a configuration (the config.json dictionary) and the checkpoint's tensors by
their checkpoint names and shares no code with the library.

    norm             the row in ``groups`` equal runs, each run r / sqrt(mean(r^2) + eps); the whole times w
    layer            x = x + mixer(n1(x)) + mlp(n2(x))          both norms read the same x; a layer may have no mlp
    attention        q, k, v = Wq h, Wk h, Wv h; value i of the first rot.dims of a head turns with value i + dims/2 by
                     p * f_i (f_i stretched for long wavelengths, cos and sin times a constant of the stretch); q, k
                     divided by their root mean square; s = q.k * scale; key j counts for query i when j <= i and both
                     lie in the same run of mask.size positions; softmax; Wo
    parallel         left_scale * capped_attention(h) + right_scale * delta_rule(h)
    capped attention q, k, v = Wq h + bq, ...; s = cap * tanh(q.k * scale / cap), causal; softmax;
                     out = Wo (sum p v * sigmoid(Wg h)) + bo
    delta rule       q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h)); q, k unit vectors, q / sqrt(dim)
                     beta = sigmoid(Wb h); g = exp(-exp(A_log_h) softplus(Wa h + dt_bias_h))       (one number a head)
                     S = g S; u = beta (v - S^T k); S = S + k u^T; o = S^T q
                     out = Wo (o / rms(o) * w * silu(Wg h))
    latent attention cq = n(Wdq h) * w_dq; q = Wuq cq, per head [dim | rot_dim]; [c' | kr] = Wdkv h; c = n(c') * w_dkv
                     s = (q_nope . Wuk,h c + rot(q_rot) . rot(kr)) * scale; key j counts when 0 <= i - j < mask.size;
                     softmax; v = Wuv,h c; Wo
    dense            Wdown (silu(Wgate h) * Wup h)
    experts          s = softmax(Wr h); the ``top`` largest of s + correction are the token's; weights s over their sum
                     (+ 1e-20), times router.scale; expert: Wdown relu(Wup h)^2; the weighted sum of the chosen experts
    output           logits = head n_final(x)
"""
import math

import torch


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def group_norm(x, w, eps, groups):
    """Rows of x cut into ``groups`` equal consecutive runs, each divided by its own root mean square; then times w."""
    n, d = x.shape
    r = x.reshape(n, groups, d // groups)
    r = r / torch.sqrt((r * r).mean(-1, keepdim=True) + eps)
    return r.reshape(n, d) * w


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(x, taps_w, before=None):
    """x [n, channels]; taps_w [channels, taps], its last column multiplies the current row; rows before the start
    are zeros (or ``before`` [taps - 1, channels])."""
    n, c = x.shape
    taps = taps_w.shape[1]
    pad = torch.zeros(taps - 1, c, dtype=x.dtype) if before is None else before
    xp = torch.cat([pad, x], 0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + xp[j:j + n] * taps_w[:, j][None]
    return out


def stretched_frequencies(dims, base, scaling=None):
    """(frequencies [dims / 2], the constant that multiplies cos and sin)."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn(t):  # the dimension whose wave makes t turns over the original length
        return dims * math.log(orig / (2 * math.pi * t)) / (2 * math.log(base))

    lo = max(math.floor(turn(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
    out = []
    for i, v in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(v / factor * ramp + v * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_halves(v, positions, dims, freqs, mult):
    """v [n, heads, width]: value i of the first ``dims`` of every head turns with value i + dims / 2 by p * f_i."""
    if dims == 0:
        return v
    ang = positions.to(v.dtype)[:, None] * torch.tensor(freqs, dtype=v.dtype)[None]
    cs, sn = torch.cos(ang)[:, None, :] * mult, torch.sin(ang)[:, None, :] * mult
    h = dims // 2
    a, b = v[..., :h], v[..., h:dims]
    out = v.clone()
    out[..., :h] = a * cs - b * sn
    out[..., h:dims] = b * cs + a * sn
    return out


def visible(n, kind, size):
    """[n, n] bool: may query i (row) see key j (column)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if kind == "window":
        ok = ok & (i - j < size)
    elif kind == "chunk":
        ok = ok & (i // size == j // size)
    return ok


def softmax_heads(s, ok):
    """s [heads, n, n] scores, ok [n, n]: ordinary softmax over the visible keys."""
    s = s.masked_fill(~ok[None], float("-inf"))
    return torch.softmax(s, dim=-1)


def attention(h, w, p, m, eps, first_position=0):
    """The mixer 'attention' (rotated, normed queries and keys; chunked)."""
    n = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).reshape(n, H, D)
    k = (h @ w[p + "k"].T).reshape(n, G, D)
    v = (h @ w[p + "v"].T).reshape(n, G, V)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    pos = torch.arange(first_position, first_position + n)
    if dims:
        f, mult = stretched_frequencies(dims, float(rot["base"]), rot.get("scaling"))
        q, k = rotate_halves(q, pos, dims, f, mult), rotate_halves(k, pos, dims, f, mult)
    q, k = rms(q, eps), rms(k, eps)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    pr = softmax_heads(s, visible(n, "chunk", int(m["mask"]["size"])))
    o = torch.einsum("hij,jhv->ihv", pr, v).reshape(n, H * V)
    return o @ w[p + "o"].T


def capped_attention(h, w, p, m):
    """The left side of the mixer 'parallel': biases, no rotation, capped scores, causal, a sigmoid gate."""
    n = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(n, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(n, G, D).repeat_interleave(H // G, dim=1)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(n, G, V).repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    cap = float(m["softcap"])
    s = cap * torch.tanh(s / cap)
    pr = softmax_heads(s, visible(n, "causal", 0))
    o = torch.einsum("hij,jhv->ihv", pr, v).reshape(n, H * V)
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T + w[p + "o.b"]


def delta_rule(h, w, p, m, eps, state=None, before=None):
    """The right side of the mixer 'parallel'.  Returns (output, state [heads, dim, vdim], last inputs of the
    convolutions); ``state`` and ``before`` continue a sequence."""
    n = h.shape[0]
    H, G, D, V, taps = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"])
    raw = torch.cat([h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T], dim=1)
    taps_w = torch.cat([w[p + "q.conv"], w[p + "k.conv"], w[p + "v.conv"]], dim=0)
    x = silu(causal_conv(raw, taps_w, before))
    tail = torch.cat([torch.zeros(taps - 1, raw.shape[1], dtype=raw.dtype) if before is None else before, raw], 0)[-(taps - 1):] \
        if taps > 1 else raw[:0]
    q = x[:, :G * D].reshape(n, G, D)
    k = x[:, G * D:2 * G * D].reshape(n, G, D)
    v = x[:, 2 * G * D:].reshape(n, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q = q.repeat_interleave(H // G, dim=1)
    k = k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None] * softplus(h @ w[p + "a"].T + w[p + "dt_bias"][None]))
    S = torch.zeros(H, D, V, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(n, H, V, dtype=h.dtype)
    for t in range(n):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + torch.einsum("hd,hv->hdv", k[t], u)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * w[p + "norm"][None, None]
    o = o.reshape(n, H * V) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T, S, tail


def latent_attention(h, w, p, m, eps, first_position=0):
    """The mixer 'latent_attention': queries through a latent, keys and values from one cached latent row and one
    rotated key part shared by the heads; a sliding window."""
    n = h.shape[0]
    H, D, R, V, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(n, H, D + R)
    dkv = h @ w[p + "dkv"].T
    c = rms(dkv[:, :rank], eps) * w[p + "dkv.norm"]
    kr = dkv[:, rank:].reshape(n, 1, R)
    rot = m["rot"]
    pos = torch.arange(first_position, first_position + n)
    f, mult = stretched_frequencies(R, float(rot["base"]), rot.get("scaling"))
    q_rot = rotate_halves(q[..., D:].contiguous(), pos, R, f, mult)
    kr = rotate_halves(kr, pos, R, f, mult)
    k_nope = (c @ w[p + "uk"].T).reshape(n, H, D)
    v = (c @ w[p + "uv"].T).reshape(n, H, V)
    s = (torch.einsum("ihd,jhd->hij", q[..., :D], k_nope) + torch.einsum("ihd,jd->hij", q_rot, kr[:, 0])) * float(m["scale"])
    pr = softmax_heads(s, visible(n, "window", int(m["mask"]["size"])))
    o = torch.einsum("hij,jhv->ihv", pr, v).reshape(n, H * V)
    return o @ w[p + "o"].T


def dense_mlp(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, mlp):
    """(chosen experts [n, top], their weights [n, top], all scores [n, experts])."""
    r = mlp["router"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    chosen = torch.topk(s + w[p + "correction"][None], int(r["top"]), dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20) * float(r["scale"]), s


def experts_mlp(h, w, p, mlp):
    chosen, weights, _ = route(h, w, p, mlp)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            mid = torch.relu(h[t] @ w[p + f"e{e}.up"].T) ** 2
            out[t] = out[t] + a * (mid @ w[p + f"e{e}.down"].T)
    return out


def mixer(h, w, p, layer, eps):
    m = layer["mixer"]
    if layer["type"] == "attention":
        return attention(h, w, p, m, eps)
    if layer["type"] == "latent_attention":
        return latent_attention(h, w, p, m, eps)
    if layer["type"] == "parallel":
        left = capped_attention(h, w, p + "left.", m["left"])
        right = delta_rule(h, w, p + "right.", m["right"], eps)[0]
        return float(m["left_scale"]) * left + float(m["right_scale"]) * right
    raise ValueError(layer["type"])


def forward(config, weights, tokens, dtype=torch.float64, streams=None):
    """Logits [n, vocab] of one sequence.  ``streams``: a list that receives the stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, groups = float(config["norm"]["eps"]), int(config["norm"].get("groups", 1))
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        y = mixer(group_norm(x, w[p + "norm1"], eps, groups), w, p + "mix.", layer, eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h2 = group_norm(x, w[p + "norm2"], eps, groups)
            y = y + (dense_mlp(h2, w, p + "mlp.") if mlp["kind"] == "dense" else experts_mlp(h2, w, p + "mlp.", mlp))
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    return group_norm(x, w["final.norm"], eps, groups) @ w["head"].T
