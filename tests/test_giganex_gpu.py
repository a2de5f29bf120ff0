"""The Giganex design on the GPU against its plain restatement (tests/plain_giganex.py): every mechanism alone, then
whole models of several shapes through the engine — prompts, token-by-token decoding (graphs included), prompts cut
into portions down to two tokens, unequal batches, slots, blocks and states that are used again, long decoding over
the edges of cache blocks, of the decode kernels' key splits, of runs and of windows, greedy generation and the trace
program."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import giganex_models as gm
import plain_giganex as pg

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16}


def _weights(which, mild):
    """Sharp weights for the float32 comparisons (peaked attention rows, saturated gates), mild ones for bfloat16,
    where 16-bit rounding of large scores would itself move the softmax by several percent."""
    i = list(gm.CONFIGS).index(which)
    return gm.tensors(gm.CONFIGS[which], seed=31 + i, std=0.03) if mild else gm.tensors(gm.CONFIGS[which], seed=11 + i)


def K(which, dtype):
    return which + ("_mild" if dtype == "bf16" else "")


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("giganex")
    out = {}
    for which, cfg in gm.CONFIGS.items():
        out[which] = gm.write_folder(str(root / which), cfg, _weights(which, False))
        out[which + "_mild"] = gm.write_folder(str(root / (which + "_mild")), cfg, _weights(which, True))
    return out


class Oracle:
    def __init__(self, cfg, weights):
        self.cfg, self.weights, self._memo = cfg, weights, {}

    def logits(self, ids):
        key = tuple(ids)
        if key not in self._memo:
            self._memo[key] = pg.forward(self.cfg, self.weights, ids)
        return self._memo[key]

    def close_calls(self, ids, margin=0.02):
        """Rows of a sequence whose choice of experts in some layer hangs on less than ``margin`` (16-bit rounding may
        then choose otherwise): what bfloat16 comparisons leave out."""
        w = {k: v.double() if v.is_floating_point() else v for k, v in self.weights.items()}
        streams = []
        pg.forward(self.cfg, self.weights, ids, streams=streams)
        eps, groups = float(self.cfg["norm"]["eps"]), int(self.cfg["norm"]["groups"])
        x = [w["embed"][torch.as_tensor(ids)]] + streams
        bad = torch.zeros(len(ids), dtype=torch.bool)
        for i, layer in enumerate(self.cfg["layers"]):
            mlp = layer.get("mlp")
            if mlp is None or mlp["kind"] != "moe":
                continue
            p = f"l{i}.mlp."
            h = pg.group_norm(x[i], w[f"l{i}.norm2"], eps, groups)
            s = torch.softmax(h @ w[p + "router"].T, -1) + w[p + "correction"][None]
            top = int(mlp["router"]["top"])
            if top < s.shape[1]:
                v = s.sort(-1, descending=True).values
                bad |= (v[:, top - 1] - v[:, top]) < margin
        return bad


@pytest.fixture(scope="module")
def oracles():
    out = {}
    for which, cfg in gm.CONFIGS.items():
        out[which] = Oracle(cfg, _weights(which, False))
        out[which + "_mild"] = Oracle(cfg, _weights(which, True))
    return out


_models = {}


def model_of(folders, which, dtype):
    from fms_b200.models import get_model

    key = (which, dtype)
    if key not in _models:
        _models[key] = get_model("hf_pretrained", model_path=folders[K(which, dtype)], device_type="cuda", data_type=dtype)
    return _models[key]


def close(got, want, dtype, loose=1.0, keep=None):
    want = want.to(torch.float64)
    got = got.detach().cpu().to(torch.float64)
    assert got.shape == want.shape and torch.isfinite(got).all()
    if keep is not None:
        got, want = got[keep], want[keep]
    top = want.abs().max().item() if want.numel() else 1.0
    if dtype == "fp32":
        torch.testing.assert_close(got, want, atol=3e-5 * loose * max(1.0, top), rtol=1e-4 * loose)
    else:
        torch.testing.assert_close(got, want, atol=0.03 * loose * top, rtol=0.03 * loose)


def check_rows(oracle, ids, got, dtype, rows=None):
    """Logits of rows ``rows`` (all by default) of the sequence ``ids`` against the oracle; bfloat16 leaves out rows whose
    routing is a close call."""
    want = oracle.logits(ids)
    rows = list(range(len(ids))) if rows is None else list(rows)
    keep = None
    if dtype == "bf16":
        bad = oracle.close_calls(ids)
        keep = ~bad[rows]
        assert len(rows) < 8 or keep.float().mean() > 0.5
    close(got, want[rows], dtype, keep=keep)


def part_with(part, tensors, dtype):
    for q, owner, local, decl in part.named_decls():
        owner.set_tensor(local, tensors[q].to(device="cuda", dtype=dtype).contiguous())
    part.finalize(torch.device("cuda"), dtype)
    return part


def step_through(mixer, x, cuts, dtype, lanes=1):
    """Runs x [n, dim] through a mixer as ``lanes`` equal sequences side by side, each cut into steps of the given sizes;
    returns the first sequence's rows (the others must equal them)."""
    from fms_b200.cache import Cache
    from fms_b200.engine.batch import Batch

    cache = Cache([mixer.cache_request()], max_tokens=1024 * lanes, max_positions=1024, dtype=dtype, device="cuda")
    slots = cache.begin(lanes)
    out, at = [], 0
    for n in cuts:
        before = cache.prepare(slots, [n] * lanes)
        batch = Batch.from_lists(slots, before, [[0] * n] * lanes, [[]] * lanes, "cuda")
        piece = x[at:at + n].contiguous()
        y = mixer.forward(piece.repeat(lanes, 1) if lanes > 1 else piece, batch, cache.layer_view(0), True)
        if hasattr(y, "parts"):
            y = sum(f * t.float() for t, f in y.parts).to(y.parts[0][0].dtype)
        for lane in range(1, lanes):
            assert torch.equal(y[:n], y[lane * n:(lane + 1) * n])
        out.append(y[:n])
        cache.commit(slots, [n] * lanes)
        at += n
    assert at == x.shape[0]
    return torch.cat(out)


def mk(g, *s, sd=0.3):
    return (torch.randn(*s, generator=g) * sd).to(torch.bfloat16)


def position_spec(r):
    from fms_b200.config import PositionSpec

    if not r or not r["dims"]:
        return PositionSpec("none")
    sc = r.get("scaling")
    return PositionSpec("rope", head_dim=r["dims"], theta=r["base"], scaling=() if sc is None else (
        ("rope_type", "yarn"), ("factor", sc["factor"]), ("original", sc["original"]), ("fast", sc["fast"]), ("slow", sc["slow"])))


# ---- mechanisms alone ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("dim,groups", [(36, 18), (256, 4), (1000, 1), (4096, 2), (5000, 5), (6, 3)])
def test_norm_in_runs_with_pending_parts(dtype, dim, groups):
    """One to four pending outputs with their factors, one or two gains, the stream written or (with rows) only read."""
    from fms_b200.kernels import ops

    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(dim)
    res = torch.randn(7, dim, generator=g) * 3
    deltas = [(torch.randn(7, dim, generator=g) * 5).to(dt) for _ in range(4)]
    gains = [1 + 0.5 * torch.randn(dim, generator=g) for _ in range(2)]
    for factors in ((), (1.0,), (0.6, 0.5), (-2.0, 1.0, 0.25), (0.5, 0.5, 1.0, 3.0)):
        parts = list(zip(deltas, factors))
        x = res.double() + sum(f * t.double() for t, f in parts)
        want = [pg.group_norm(x, w.double(), 1e-5, groups) for w in gains]
        for n_out in (1, 2):
            r = res.clone().cuda()
            outs = ops.parts_group_rmsnorm(r, [(t.cuda(), f) for t, f in parts], [w.cuda() for w in gains[:n_out]], 1e-5, groups, dt)
            close(r, x, "fp32")
            for o, w in zip(outs, want):
                close(o, w, dtype, loose=0.5)
        rows = torch.tensor([5, 0, 5], dtype=torch.int32)
        r = res.clone().cuda()
        (o,) = ops.parts_group_rmsnorm(r, [(t.cuda(), f) for t, f in parts], [gains[0].cuda()], 1e-5, groups, dt, rows.cuda())
        assert torch.equal(r.cpu(), res)
        close(o, want[0][rows.long()], dtype, loose=0.5)


def plain_masked_attention(q, batch, view, nheads, kvheads, hd, scale, chunk, softcap):
    """The step's queries over the cache, row by row in float32: keys of the query's own run of ``chunk`` positions
    (0: all earlier keys), scores capped by ``softcap`` (0: as they are)."""
    import plain_ops as P

    out = torch.zeros_like(q)
    first, lens, slots = batch.first_row.tolist(), batch.len_after.tolist(), batch.slots.tolist()
    group = nheads // kvheads
    for i in range(batch.n_seqs):
        n_new = first[i + 1] - first[i]
        for j in range(n_new):
            p = lens[i] - n_new + j
            lo = p - p % chunk if chunk else 0
            k, v = P.gather_cache(view, slots[i], lo, p + 1)
            s = torch.einsum("hd,thd->ht", q[first[i] + j].float().view(nheads, hd), k.repeat_interleave(group, dim=1)) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            out[first[i] + j] = torch.einsum("ht,thd->hd", torch.softmax(s, -1), v.repeat_interleave(group, dim=1)).reshape(-1).to(q.dtype)
    return out


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("nheads,kvheads,hd,lens_before,num_new,chunk,softcap", [
    (4, 2, 16, [0, 0, 0], [5, 70, 17], 16, 0.0),          # prompts from an empty cache, runs shorter than a block
    (3, 1, 32, [100, 3, 64], [1, 1, 1], 64, 2.0),         # decode: a run that began at a block's edge, one that begins now
    (5, 5, 48, [130, 0], [40, 129], 100, 1.0),            # continuation onto a cached prefix over a run's edge, capped
    (12, 1, 64, [300], [1], 0, 0.5),                      # decode with 12 query heads on one kv head, cap alone
    (2, 2, 128, [513], [1], 257, 0.0),                    # decode over three splits of which the run touches two
    (8, 2, 128, [0, 100], [200, 77], 150, 3.0),           # prefill on the tcgen05 kernel, head size 128
    (4, 4, 64, [64, 0], [130, 1], 64, 4.0),               # prefill, head size 64, runs of one block
    (4, 2, 80, [10], [70], 33, 0.0),                      # prefill on mma.sync
    (2, 1, 64, [33000], [1], 5000, 1.5),                  # decode over more splits than the merge stages in shared memory
    (8, 8, 128, [33000, 100, 5000, 64], [1, 1, 1, 1], 4000, 2.5),  # enough to read for the streaming kernel
])
def test_attention_kernels_in_runs_and_with_a_cap(dtype, nheads, kvheads, hd, lens_before, num_new, chunk, softcap):
    """The attention kernels themselves over a poisoned cache with scrambled blocks: every kernel (float32 and the
    tensor-core ones for prompts, split keys and the streamed cache for decode steps) with runs, a cap, and both."""
    from test_kernels_gpu import make_cache_case, tol

    from fms_b200.kernels import ops

    dt = DTYPES[dtype]
    cache, view, batch = make_cache_case(dt, nheads, kvheads, hd, lens_before, num_new, 9)
    g = torch.Generator().manual_seed(hd + chunk)
    qkv = (torch.randn(sum(num_new), (nheads + 2 * kvheads) * hd, generator=g) * 1.5).to(dt).cuda()
    q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
    scale = 1.0 / math.sqrt(hd)
    want = plain_masked_attention(q, batch, view, nheads, kvheads, hd, scale, chunk, softcap)
    got = ops.attention(q, batch, view, nheads, kvheads, hd, scale, 0, None, chunk=chunk, softcap=softcap)
    ops.check_error_flag("cuda")
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got.float(), want.float(), **tol(dt))


def test_streamed_decode_attention_in_runs_with_a_cap():
    """Seventy sequences of 32 heads over 8: decode attention is the persistent kernel that streams the cache by TMA;
    with runs of 300 positions and a cap of 3, and one marked key inside the first sequence's run and one just before it."""
    from test_kernels_gpu import make_cache_case, tol

    from fms_b200.kernels import ops

    dt, nheads, kvheads, hd, chunk, softcap = torch.bfloat16, 32, 8, 128, 300, 3.0
    g = torch.Generator().manual_seed(23)
    lens = [int(v) for v in torch.randint(1, 700, (70,), generator=g)]
    lens[0], lens[1], lens[2] = 699, 256, 1
    cache, view, batch = make_cache_case(dt, nheads, kvheads, hd, lens, [1] * 70, 16)
    qkv = torch.randn(70, (nheads + 2 * kvheads) * hd, generator=g).to(dt).cuda()
    q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
    table = cache.groups[0].table_host
    head, group = nheads - 1, nheads // kvheads
    for far, value in ((600, 2.0), (599, -5.0)):  # the query at position 699 sees 600..699
        blk = int(table[int(batch.slots[0]), far // 64])
        view.keys[blk, head // group, far % 64] = (q[0, head * hd:(head + 1) * hd].float() * 6).to(dt)
        view.values[blk, head // group, far % 64] = torch.full((hd,), value).to(dt).cuda()
    scale = 1.0 / math.sqrt(hd)
    before = ops.attention_stream_launches(hd)
    got = ops.attention(q, batch, view, nheads, kvheads, hd, scale, 0, None, chunk=chunk, softcap=softcap)
    ops.check_error_flag("cuda")
    assert ops.attention_stream_launches(hd) == before + 1  # it was this kernel that ran
    want = plain_masked_attention(q, batch, view, nheads, kvheads, hd, scale, chunk, softcap)
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got.float(), want.float(), **tol(dt))
    # the cap bounds the marked key's score at 3, so it shares the weight with the run's other 99 keys instead of taking all
    assert float(want[0, head * hd].float()) < 1.0 and float(got[0, head * hd].float()) < 1.0


def chunked_tensors(g, dim_in, m):
    h, kv, k, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {"q": mk(g, h * k, dim_in), "k": mk(g, kv * k, dim_in), "v": mk(g, kv * v, dim_in), "o": mk(g, dim_in, h * v)}


def chunked_mixer(m, dim_in, w, eps, dt):
    from fms_b200.config import MixerSpec
    from fms_b200.parts import build_mixer

    r = m["rot"]
    spec = MixerSpec("sink_attention", dim=dim_in, nheads=m["heads"], kvheads=m["kv_heads"], head_dim=m["dim"], bias=False,
                     scale=m["scale"], position=position_spec(r),
                     options=(("vdim", m["vdim"]), ("rot_dims", r["dims"]), ("pairing", "halves"), ("qk_norm", True),
                              ("eps", eps), ("chunk", m["mask"]["size"])))
    return part_with(build_mixer(spec), {"in_proj.weight": torch.cat([w["q"], w["k"], w["v"]]), "dense.weight": w["o"]}, dt)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(4, 2, 16, 16, 8, 1, 50), (6, 1, 24, 8, 24, 0, 64), (2, 2, 10, 40, 0, 0, 7), (3, 3, 64, 64, 32, 1, 150),
                                   (8, 2, 128, 64, 64, 1, 300), (5, 5, 6, 10, 2, 0, 1), (2, 1, 48, 33, 48, 1, 1000), (4, 4, 64, 64, 64, 0, 65)])
def test_attention_in_runs_alone(dtype, shape):
    heads, kv, dim, vdim, rd, scaled, chunk = shape
    sc = {"factor": 8.0, "original": 96, "fast": 4.0, "slow": 1.0} if scaled else None
    m = gm.attention(heads, kv, dim, vdim, gm.rot(rd, 300.0, sc), 2.0 * dim ** -0.5 * (1 if dtype == "bf16" else 3), chunk, None)["mixer"]
    dt, dim_in, n = DTYPES[dtype], 40, 331
    g = torch.Generator().manual_seed(sum(shape))
    w = chunked_tensors(g, dim_in, m)
    mixer = chunked_mixer(m, dim_in, w, 1e-5, dt)
    x = torch.randn(n, dim_in, generator=g).to(dt)
    want = pg.attention(x.double(), {k: v.double() for k, v in w.items()}, "", m, 1e-5)
    # whole; portions whose edges fall on and beside the cache's blocks of 64; the last rows one by one (the decode
    # kernels, over the edge of their first split of 256 keys)
    for cuts in ([n], [63, 1, 1, 63, 2, 128, 73], [250] + [1] * 81):
        close(step_through(mixer, x.cuda(), cuts, dt), want, dtype)


def capped_tensors(g, dim_in, m):
    h, kv, k, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {"q": mk(g, h * k, dim_in), "q.b": mk(g, h * k), "k": mk(g, kv * k, dim_in), "k.b": mk(g, kv * k), "v": mk(g, kv * v, dim_in),
            "v.b": mk(g, kv * v), "g": mk(g, h * v, dim_in), "o": mk(g, dim_in, h * v), "o.b": mk(g, dim_in)}


def capped_mixer(m, dim_in, w, dt):
    from fms_b200.config import MixerSpec
    from fms_b200.parts import build_mixer

    spec = MixerSpec("sink_attention", dim=dim_in, nheads=m["heads"], kvheads=m["kv_heads"], head_dim=m["dim"], bias=True,
                     scale=m["scale"], options=(("vdim", m["vdim"]), ("gate", True), ("out_bias", True), ("softcap", m["softcap"])))
    zeros = torch.zeros(m["heads"] * m["vdim"], dtype=torch.bfloat16)
    return part_with(build_mixer(spec), {
        "in_proj.weight": torch.cat([w["q"], w["k"], w["v"], w["g"]]), "in_proj.bias": torch.cat([w["q.b"], w["k.b"], w["v.b"], zeros]),
        "dense.weight": w["o"], "dense.bias": w["o.b"]}, dt)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(4, 2, 16, 16, 3.0), (6, 1, 24, 8, 50.0), (2, 2, 10, 40, 1.0), (8, 2, 128, 64, 10.0), (4, 1, 64, 128, 2.0),
                                   (5, 5, 6, 10, 0.5), (4, 4, 64, 64, 4.0)])
def test_capped_attention_alone(dtype, shape):
    """Scores several times their cap (the cap decides the weights) down to scores far below it (it does nothing)."""
    heads, kv, dim, vdim, cap = shape
    m = gm.left(heads, kv, dim, vdim, 0.7 * dim ** -0.5 * (1 if dtype == "bf16" else 3), cap)
    dt, dim_in, n = DTYPES[dtype], 40, 331
    g = torch.Generator().manual_seed(int(sum(shape)))
    w = capped_tensors(g, dim_in, m)
    mixer = capped_mixer(m, dim_in, w, dt)
    x = torch.randn(n, dim_in, generator=g).to(dt)
    want = pg.capped_attention(x.double(), {k: v.double() for k, v in w.items()}, "", m)
    for cuts in ([n], [63, 1, 1, 63, 2, 128, 73], [250] + [1] * 81):
        close(step_through(mixer, x.cuda(), cuts, dt), want, dtype)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_one_key_just_inside_and_just_outside_a_run(dtype):
    """Weights and inputs made so that a fault shows.  Queries read the first half of the input and keys the second
    half through the same matrix, and the first half of some rows is the second half of ONE earlier row, so that this
    key's score stands out among hundreds: for rows whose marked key is the first of their own run (it counts: the
    result is nearly its value) and for rows whose marked key is the last of the run before (it does not: the result
    has nothing of it), in prompts, in portions and when decoding."""
    chunk, dim_in, n = 100, 32, 520
    # normed queries and keys have length 4: the marked key scores 16 times the scale (milder in bfloat16, where the
    # rounding of a large score would itself move the softmax)
    m = gm.attention(2, 1, 16, 16, gm.rot(0, 10.0), 3.0 if dtype == "fp32" else 1.0, chunk, None)["mixer"]
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(78)
    a = mk(g, 16, 16, sd=0.6)
    w = {"q": torch.cat([torch.cat([a, torch.zeros_like(a)], 1)] * 2), "k": torch.cat([torch.zeros_like(a), a], 1),
         "v": mk(g, 16, dim_in), "o": mk(g, dim_in, 32)}
    x = torch.randn(n, dim_in, generator=g)
    inside, outside = [], []
    for run in range(1, 5):
        first = run * chunk
        for t in (first, first + 1, first + 57, first + chunk - 1):  # sees the first key of its own run
            x[t, :16] = x[first, 16:]
            inside.append(t)
        for t in (first + 2, first + 58):  # asks for the last key of the run before
            x[t, :16] = x[first - 1, 16:]
            outside.append(t)
    x = x.to(dt)
    d = {k: v.double() for k, v in w.items()}
    want = pg.attention(x.double(), d, "", m, 1e-5)
    # the oracle itself says that the edge matters: with runs one position longer the marked rows come out otherwise
    moved = pg.attention(x.double(), d, "", dict(m, mask={"size": chunk + 1}), 1e-5)
    assert (want[outside] - moved[outside]).abs().max() > 0.2 * want.abs().max()
    mixer = chunked_mixer(m, dim_in, w, 1e-5, dt)
    for cuts in ([n], [99, 1, 1, 99, 2, 198, 120], [95] + [1] * 425, [2] * 260):
        close(step_through(mixer, x.cuda(), cuts, dt), want, dtype)


def latent_tensors(g, dim_in, m):
    h, k, r, v, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
    return {"dq": mk(g, qr, dim_in), "dq.norm": 1 + mk(g, qr), "uq": mk(g, h * (k + r), qr, sd=0.5), "dkv": mk(g, kr + r, dim_in),
            "dkv.norm": 1 + mk(g, kr), "uk": mk(g, h * k, kr, sd=0.5), "uv": mk(g, h * v, kr), "o": mk(g, dim_in, h * v)}


def latent_mixer(m, dim_in, w, eps, dt):
    from fms_b200.config import MixerSpec
    from fms_b200.parts import build_mixer

    spec = MixerSpec("latent_attention", dim=dim_in, nheads=m["heads"], head_dim=m["dim"], scale=m["scale"], window=m["mask"]["size"],
                     position=position_spec(m["rot"]),
                     options=(("rot", m["rot_dim"]), ("vdim", m["vdim"]), ("rank", m["kv_rank"]), ("rot_dims", m["rot_dim"]),
                              ("eps", eps), ("q_rank", m["q_rank"]), ("sink", False), ("gate", False), ("pairing", "halves")))
    return part_with(build_mixer(spec), {"in_proj.weight": torch.cat([w["dkv"], w["dq"]]), "q_norm": w["dq.norm"], "q_up.weight": w["uq"],
                                         "latent_norm": w["dkv.norm"], "uk": w["uk"], "uv": w["uv"], "dense.weight": w["o"]}, dt)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(3, 10, 6, 12, 14, 18, 1, 20), (2, 16, 16, 40, 24, 32, 0, 300), (5, 6, 2, 3, 5, 7, 1, 1), (4, 32, 32, 48, 40, 64, 1, 210),
                                   (40, 8, 8, 8, 16, 128, 0, 64), (2, 64, 32, 64, 96, 192, 1, 257), (3, 0, 16, 8, 8, 16, 1, 33)])
def test_windowed_latent_attention_alone(dtype, shape):
    """Windows inside one cache block, over block edges, over the edge of a decode split, of one key; latents that take
    the float32 kernel and ones that take the tensor-core kernel; more heads than a block takes; heads without an
    unrotated part."""
    heads, dim, rd, vdim, qr, kr, scaled, window = shape
    sc = {"factor": 8.0, "original": 96, "fast": 4.0, "slow": 1.0} if scaled else None
    m = gm.latent(heads, dim, rd, vdim, qr, kr, 300.0, sc, 0.7 * (dim + rd) ** -0.5 * (1 if dtype == "bf16" else 2), window, None)["mixer"]
    dt, dim_in, n = DTYPES[dtype], 40, 331
    g = torch.Generator().manual_seed(sum(shape))
    w = latent_tensors(g, dim_in, m)
    mixer = latent_mixer(m, dim_in, w, 1e-5, dt)
    x = torch.randn(n, dim_in, generator=g).to(dt)
    want = pg.latent_attention(x.double(), {k: v.double() for k, v in w.items()}, "", m, 1e-5)
    for cuts in ([n], [63, 1, 1, 63, 2, 128, 73], [250] + [1] * 81):
        close(step_through(mixer, x.cuda(), cuts, dt), want, dtype, loose=2)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("rank", [24, 64])
def test_one_key_just_inside_and_just_outside_a_window(dtype, rank):
    """The rotated key part is switched off (its rows of the projection are zeros).  The query's latent and the first 16
    values of the key's latent read the first half of the input through the same matrix, and every head's two
    up-projections are one orthogonal matrix, so that a row whose first half repeats an earlier row's scores that row's
    key (and its own) far above all others; the rest of the latent reads the second half of the input, so that the two
    rows' values differ.  Rows that repeat the row window - 1 back (the last key the window keeps) against rows that
    repeat the row window back (the first one it has dropped), through the float32 kernel (rank 24) and the tensor-core
    kernel (rank 64)."""
    window, dim_in, n = 130, 32, 560
    # a marked key scores about 16 times the scale: 40 in float32, 12 in bfloat16
    m = gm.latent(2, 16, 16, 8, 16, rank, 100.0, None, 2.5 if dtype == "fp32" else 0.75, window, None)["mixer"]
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(79 + rank)
    w = latent_tensors(g, dim_in, m)
    w["dkv"][rank:] = 0
    w["dkv"][:16, 16:] = 0
    w["dkv"][16:rank, :16] = 0
    w["dq"] = w["dkv"][:16].clone()
    a = torch.linalg.qr(torch.randn(16, 16, generator=g)).Q
    w["uq"] = torch.cat([torch.cat([a, torch.zeros(16, 16)]).to(torch.bfloat16)] * 2)
    w["uk"] = torch.cat([torch.cat([a, torch.zeros(16, rank - 16)], 1).to(torch.bfloat16)] * 2)
    w["dq.norm"] = torch.ones(16, dtype=torch.bfloat16)
    w["dkv.norm"] = torch.ones(rank, dtype=torch.bfloat16)
    x = torch.randn(n, dim_in, generator=g)
    inside, outside = [], []
    for t in range(140, n, 9):
        back = window - 1 if (t // 9) % 2 else window
        x[t, :16] = x[t - back, :16]
        (inside if back == window - 1 else outside).append(t)
    x = x.to(dt)
    d = {k: v.double() for k, v in w.items()}
    want = pg.latent_attention(x.double(), d, "", m, 1e-5)
    moved = pg.latent_attention(x.double(), d, "", dict(m, mask={"size": window + 1}), 1e-5)
    assert (want[outside] - moved[outside]).abs().max() > 0.2 * want.abs().max()
    shrunk = pg.latent_attention(x.double(), d, "", dict(m, mask={"size": window - 1}), 1e-5)
    assert (want[inside] - shrunk[inside]).abs().max() > 0.2 * want.abs().max()
    mixer = latent_mixer(m, dim_in, w, 1e-5, dt)
    for cuts in ([n], [129, 1, 1, 129, 2, 128, 170], [135] + [1] * 425, [2] * 280):
        close(step_through(mixer, x.cuda(), cuts, dt), want, dtype, loose=2)


def delta_tensors(g, dim_in, m):
    h, kv, k, v, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    out = {"b": mk(g, h, dim_in), "a": mk(g, h, dim_in), "A_log": mk(g, h, sd=1.0) - 1, "norm": 1 + mk(g, v), "dt_bias": mk(g, h, sd=1.0),
           "g": mk(g, h * v, dim_in), "o": mk(g, dim_in, h * v)}
    for n, rows in (("q", kv * k), ("k", kv * k), ("v", h * v)):
        out[n], out[n + ".conv"] = mk(g, rows, dim_in), mk(g, rows, taps, sd=0.6)
    return out


def delta_mixer(m, dim_in, w, eps, dt):
    from fms_b200.config import MixerSpec
    from fms_b200.parts import build_mixer
    from fms_b200.parts.state_space import GatedDeltaRule

    spec = MixerSpec("gated_delta_rule", dim=dim_in, nheads=m["heads"], kvheads=m["kv_heads"], head_dim=m["dim"],
                     options=(("vdim", m["vdim"]), ("conv", m["conv"]), ("eps", eps), ("decay", "head")))
    rows = [w["q"], w["k"], w["v"], w["b"], w["a"]]
    gate_col = GatedDeltaRule.gate_column(m["kv_heads"], m["dim"], m["heads"], m["vdim"])
    rows.append(torch.zeros(gate_col - sum(r.shape[0] for r in rows), dim_in, dtype=torch.bfloat16))
    return part_with(build_mixer(spec), {
        "in_proj.weight": torch.cat(rows + [w["g"]]), "conv": torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]]),
        "dt_bias": w["dt_bias"], "A_log": w["A_log"], "norm": w["norm"], "dense.weight": w["o"]}, dt)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(2, 2, 32, 32, 4), (4, 1, 12, 20, 2), (3, 3, 5, 3, 1), (2, 1, 96, 40, 4), (1, 1, 256, 33, 3), (6, 2, 64, 128, 4),
                                   (4, 2, 8, 8, 5)])
def test_delta_rule_with_one_decay_a_head_alone(dtype, shape):
    heads, kv, dim, vdim, taps = shape
    m = gm.right(heads, kv, dim, vdim, taps)
    dt, dim_in, n = DTYPES[dtype], 40, 150
    g = torch.Generator().manual_seed(sum(shape))
    w = delta_tensors(g, dim_in, m)
    mixer = delta_mixer(m, dim_in, w, 1e-5, dt)
    x = torch.randn(n, dim_in, generator=g).to(dt)
    want = pg.delta_rule(x.double(), {k: v.double() for k, v in w.items()}, "", m, 1e-5)[0]
    for cuts, lanes in (([n], 1), ([15, 1, 1, 17, 2, 16, 98], 3), ([100] + [1] * 50, 2), ([2] * 75, 1)):
        close(step_through(mixer, x.cuda(), cuts, dt, lanes), want, dtype, loose=2)


def test_state_that_decays_slowly_keeps_the_first_tokens():
    """A delta rule whose decay is close to 1 (A_log very negative): the output hundreds of tokens later still carries
    the first tokens' writes; a state that was lost or reset on the way shows."""
    m = gm.right(2, 1, 16, 8, 2)
    g = torch.Generator().manual_seed(5)
    w = delta_tensors(g, 24, m)
    w["A_log"] = torch.full_like(w["A_log"], -9.0)
    w["b"] = torch.zeros_like(w["b"])
    x = torch.randn(400, 24, generator=g) * 0.2
    x[:3] *= 40
    d = {k: v.double() for k, v in w.items()}
    want = pg.delta_rule(x.double(), d, "", m, 1e-5)[0]
    lost = pg.delta_rule(x.double()[3:], d, "", m, 1e-5)[0]
    assert (want[300:] - lost[297:]).abs().max() > 0.05 * want.abs().max()
    mixer = delta_mixer(m, 24, w, 1e-5, torch.float32)
    for cuts in ([400], [1] + [3] * 133, [330] + [1] * 70):
        close(step_through(mixer, x.cuda(), cuts, torch.float32), want, "fp32", loose=2)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("experts,top,hidden,rows", [(4, 1, 16, 70), (5, 2, 20, 3), (16, 4, 24, 200), (3, 3, 8, 33), (12, 4, 16, 1), (2, 1, 9, 40)])
def test_softmax_routed_experts_alone(dtype, experts, top, hidden, rows):
    """Few rows (the kernel that walks each expert's rows) and many (tiles, or the library's grouped product); a
    correction large enough to move the choice away from the largest scores; every expert taken; one of two."""
    from fms_b200.config import FeedForwardSpec
    from fms_b200.parts import build_feed_forward

    dt, dim = DTYPES[dtype], 40
    g = torch.Generator().manual_seed(experts * 100 + top)
    mlp = gm.moe(experts, top, hidden, 1.7)
    w = {"router": mk(g, experts, dim, sd=0.5), "correction": mk(g, experts, sd=0.4)}
    for e in range(experts):
        w[f"e{e}.up"], w[f"e{e}.down"] = mk(g, hidden, dim), mk(g, dim, hidden)
    spec = FeedForwardSpec("routed_experts", dim=dim, hidden=hidden,
                           options=(("experts", experts), ("top", top), ("scoring", "softmax"), ("correction", True),
                                    ("route_scale", 1.7), ("unit", "relu_squared")))
    part = part_with(build_feed_forward(spec), {"router.weight": w["router"], "correction": w["correction"],
                                                "up": torch.stack([w[f"e{e}.up"] for e in range(experts)]),
                                                "down": torch.stack([w[f"e{e}.down"] for e in range(experts)])}, dt)
    x = torch.randn(rows, dim, generator=g).to(dt)
    d = {k: v.double() for k, v in w.items()}
    want = pg.experts_mlp(x.double(), d, "", mlp)
    chosen, _, s = pg.route(x.double(), d, "", mlp)
    if top < experts:  # the correction does move choices in this test
        assert (chosen.sort(-1).values != s.topk(top, -1).indices.sort(-1).values).any() or rows < 3
    got = part.forward(x.cuda())
    keep = None
    if top < experts:
        v = (s + d["correction"][None]).sort(-1, descending=True).values
        keep = (v[:, top - 1] - v[:, top]) > (1e-4 if dtype == "fp32" else 0.02)
    close(got, want, dtype, loose=2, keep=keep)
    # a row's result does not depend on the other rows of the step
    alone = part.forward(x[:1].cuda())
    if keep is None or keep[0]:
        close(alone, want[:1], dtype, loose=2)


# ---- whole models -------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("which", ["p", "q", "r", "s"])
def test_whole_prompts_alone(folders, oracles, which, dtype):
    model = model_of(folders, which, dtype)
    engine = model.new_engine(max_tokens=1024, sampling=False)
    for i, n in enumerate((1, 2, 63, 64, 65, 300)):
        ids = gm.prompt(gm.CONFIGS[which], n, i)
        (slot,) = engine.begin(1)
        got = engine.step([slot], [ids], [list(range(n))])
        engine.release([slot])
        check_rows(oracles[K(which, dtype)], ids, got, dtype)
    engine.check()
    assert engine.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in engine.cache.groups if hasattr(g, "pool"))


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "fp32"), ("r", "bf16"), ("s", "fp32")])
def test_token_by_token_from_the_first_token(folders, oracles, which, dtype):
    """Decode steps from a sequence's very first token (the first plain, the second captured, the rest replayed), over
    the edge of a cache block, twice in the same slot."""
    engine = model_of(folders, which, dtype).new_engine(max_tokens=256, sampling=False)
    for rep in range(2):
        ids = gm.prompt(gm.CONFIGS[which], 70, 20 + rep)
        (slot,) = engine.begin(1)
        got = torch.cat([engine.step([slot], [[t]], [[0]]) for t in ids])
        engine.release([slot])
        check_rows(oracles[K(which, dtype)], ids, got, dtype)
    assert engine.graphs_captured >= 1
    engine.check()


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "bf16"), ("r", "fp32"), ("s", "bf16"), ("s", "fp32"), ("q", "fp32")])
def test_prompt_then_long_decoding_over_split_edges(folders, oracles, which, dtype):
    """A prompt of 250 tokens, then 290 tokens one by one: the decode kernels go from one split of 256 keys to two and
    to three, the cache from its fourth block to its ninth; runs begin and windows pass over decoded tokens."""
    engine = model_of(folders, which, dtype).new_engine(max_tokens=1024, sampling=False)
    ids = gm.prompt(gm.CONFIGS[which], 540, 31)
    (slot,) = engine.begin(1)
    got = [engine.step([slot], [ids[:250]], [list(range(250))])]
    got += [engine.step([slot], [[t]], [[0]]) for t in ids[250:]]
    engine.release([slot])
    check_rows(oracles[K(which, dtype)], ids, torch.cat(got), dtype)
    engine.check()


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "fp32"), ("r", "fp32"), ("s", "fp32"), ("p", "bf16"), ("s", "bf16")])
def test_prompts_cut_into_portions(folders, oracles, which, dtype):
    engine = model_of(folders, which, dtype).new_engine(max_tokens=1024, sampling=False)
    ids = gm.prompt(gm.CONFIGS[which], 420, 41)
    for cuts in ([2, 3, 59, 1, 64, 65, 6, 220], [193, 2, 225], [1, 1, 2, 416], [2] * 40 + [340]):
        (slot,) = engine.begin(1)
        got, at = [], 0
        for n in cuts:
            got.append(engine.step([slot], [ids[at:at + n]], [list(range(n))]))
            at += n
        engine.release([slot])
        check_rows(oracles[K(which, dtype)], ids, torch.cat(got), dtype)
    engine.check()


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "fp32"), ("r", "fp32"), ("s", "fp32"), ("q", "bf16"), ("s", "bf16")])
def test_unequal_batches_freed_slots_and_poisoned_blocks(folders, oracles, which, dtype):
    """Requests of unequal lengths start together and go on one token at a time while the shorter ones end; then
    everything the cache holds is filled with NaN (keys, values, latents, state matrices, the convolutions' tails) and
    new requests take the freed slots and blocks.  Every request against the oracle, alone."""
    cfg = gm.CONFIGS[which]
    engine = model_of(folders, which, dtype).new_engine(max_tokens=64 * 12, max_slots=5, sampling=False)
    for round_ in range(2):
        lengths, extra = ((1, 70, 5, 131, 64), (3, 9, 0, 12, 12)) if round_ == 0 else ((210, 2, 33), (5, 5, 1))
        full = [gm.prompt(cfg, n + e, 50 + 10 * round_ + i) for i, (n, e) in enumerate(zip(lengths, extra))]
        slots = engine.begin(len(lengths))
        got = [[] for _ in lengths]
        first = engine.step(slots, [f[:n] for f, n in zip(full, lengths)], [list(range(n)) for n in lengths])
        for i, piece in enumerate(torch.split(first, list(lengths))):
            got[i].append(piece)
        for t in range(max(extra)):
            live = [i for i in range(len(lengths)) if t < extra[i]]
            out = engine.step([slots[i] for i in live], [[full[i][lengths[i] + t]] for i in live])
            for i, row in zip(live, out):
                got[i].append(row[None])
            done = [i for i in live if t + 1 == extra[i]]
            engine.release([slots[i] for i in done])
        engine.release([slots[i] for i in range(len(lengths)) if extra[i] == 0])
        for i, f in enumerate(full):
            check_rows(oracles[K(which, dtype)], f, torch.cat(got[i]), dtype)
        assert engine.cache.slots.n_held == 0
        for g in engine.cache.groups:
            g.storage.fill_(float("nan") if g.storage.is_floating_point() else 12345)
    engine.check()


@pytest.mark.parametrize("seed", [0, 4, 5, 7, 12, 16])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Layers of any kinds in any order with sizes drawn from a seed, float32: a prompt whole, its last 30 tokens one by
    one, and three unequal requests started together and decoded together, every row against the oracle."""
    from fms_b200.models import get_model

    cfg = gm.random_config(seed)
    weights = gm.tensors(cfg, 100 + seed, std=0.05)
    folder = gm.write_folder(str(tmp_path / "m"), cfg, weights)
    model = get_model("hf_pretrained", model_path=folder, device_type="cuda", data_type="fp32")
    engine = model.new_engine(max_tokens=1024, max_slots=4, sampling=False)
    reqs = [gm.prompt(cfg, n, seed + i) for i, n in enumerate((170, 37, 90))]
    want = [pg.forward(cfg, weights, ids) for ids in reqs]
    (slot,) = engine.begin(1)
    close(engine.step([slot], [reqs[0]], [list(range(170))]), want[0], "fp32", loose=2)
    engine.release([slot])
    (slot,) = engine.begin(1)
    got = [engine.step([slot], [reqs[0][:140]], [list(range(140))])] + [engine.step([slot], [[t]], [[0]]) for t in reqs[0][140:]]
    close(torch.cat(got), want[0], "fp32", loose=2)
    engine.release([slot])
    slots = engine.begin(3)
    first = engine.step(slots, [q[:-8] for q in reqs], [list(range(len(q) - 8)) for q in reqs])
    outs = [[p] for p in torch.split(first, [len(q) - 8 for q in reqs])]
    for t in range(8):
        rows = engine.step(slots, [[q[len(q) - 8 + t]] for q in reqs])
        for i in range(3):
            outs[i].append(rows[i][None])
    engine.release(slots)
    for i in range(3):
        close(torch.cat(outs[i]), want[i], "fp32", loose=2)
    engine.check()


def test_many_sequences_in_one_decode_step_fill_rows_and_graphs(folders, oracles):
    """Eleven sequences decode together (filled up to twelve rows with rows in the spare slot), then nine of them."""
    which, cfg, dtype = "p", gm.CONFIGS["p"], "fp32"
    engine = model_of(folders, which, "fp32").new_engine(max_tokens=64 * 24, sampling=False)
    full = [gm.prompt(cfg, 3 + 5 * i + 6, 70 + i) for i in range(11)]
    slots = engine.begin(11)
    engine.step(slots, [f[:-6] for f in full], [[] for _ in full])
    got = [[] for _ in full]
    for t in range(6):
        live = list(range(11)) if t < 3 else list(range(2, 11))
        out = engine.step([slots[i] for i in live], [[full[i][len(full[i]) - 6 + t]] for i in live])
        for i, row in zip(live, out):
            got[i].append(row[None])
    engine.release(slots)
    for i, f in enumerate(full):
        want = oracles[K(which, dtype)].logits(f)
        close(torch.cat(got[i]), want[len(f) - 6: len(f) - 6 + len(got[i])], "fp32")
    engine.check()


def test_greedy_generation_through_generate(folders, oracles):
    from fms_b200.utils.generation import generate

    which, cfg, dtype = "q", gm.CONFIGS["q"], "fp32"
    model = model_of(folders, which, "fp32")
    prompts = [gm.prompt(cfg, n, 80 + i) for i, n in enumerate((5, 1, 40))]
    out = generate(model, [torch.tensor(p) for p in prompts], max_new_tokens=10, do_sample=False)
    for p, o in zip(prompts, out):
        o = o.tolist()
        assert o[: len(p)] == p and len(o) == len(p) + 10
        for k in range(len(p), len(o)):  # every new token is the oracle's choice given what came before
            row = oracles[K(which, dtype)].logits(o[:k])[-1]
            best = row.topk(2).values
            if best[0] - best[1] > 1e-3:
                assert o[k] == int(row.argmax())


def test_trace_program_replays_a_batch(folders, oracles, tmp_path):
    which, cfg, dtype = "r", gm.CONFIGS["r"], "fp32"
    a, b = gm.prompt(cfg, 70, 90), gm.prompt(cfg, 9, 91)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for t in range(4):
        steps.append({"step": t + 1, "entries": [{"id": "a", "tokens": [a[66 + t]], "want": [0]},
                                                  {"id": "b", "tokens": [b[5 + t]], "want": [0] if t % 2 else []}],
                      "end": ["a", "b"] if t == 3 else []})
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[which], "--dtype",
                           "float32", "--out", str(tmp_path), "--max-tokens", "256"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    wa, wb = oracles[K(which, dtype)].logits(a), oracles[K(which, dtype)].logits(b)
    read = lambda i: torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))
    close(read(0), torch.stack([wa[0], wa[65], wb[4]]), "fp32")
    for t in range(4):
        want = [wa[66 + t]] + ([wb[5 + t]] if t % 2 else [])
        close(read(t + 1), torch.stack(want), "fp32")


def test_command_line_and_sampling(folders, oracles):
    """The framework's command line finds the design through config.json: greedy tokens equal the oracle's choices; with
    sampling (temperature, top-k) every token is among the oracle's k best given what came before."""
    from fms_b200.utils.generation import generate

    which, cfg = "p", gm.CONFIGS["p"]
    prompts = [gm.prompt(cfg, n, 95 + i) for i, n in enumerate((4, 9))]
    args = [sys.executable, os.path.join(ROOT, "bin", "fms_inference"), "--architecture", "hf_pretrained", "--model_path", folders[which],
            "--default_dtype", "fp32",
            "--batch_input", "--max_new_tokens", "6", "--deterministic"]
    for p in prompts:
        args += ["--prompt_ids", ",".join(str(t) for t in p)]
    proc = subprocess.run(args, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [[int(x) for x in l.split(",")] for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 2
    for p, o in zip(prompts, lines):
        assert o[: len(p)] == p and len(o) == len(p) + 6
        for k in range(len(p), len(o)):
            row = oracles[which].logits(o[:k])[-1]
            best = row.topk(2).values
            if best[0] - best[1] > 1e-3:
                assert o[k] == int(row.argmax())
    out = generate(model_of(folders, which, "fp32"), [torch.tensor(p) for p in prompts], max_new_tokens=8, do_sample=True,
                   temperature=0.8, top_k=3, seed=5)
    for p, o in zip(prompts, out):
        o = o.tolist()
        for k in range(len(p), len(o)):
            row = oracles[which].logits(o[:k])[-1]
            kth = row.topk(4).values
            assert row[o[k]] >= kth[2] - 1e-4 or kth[2] - kth[3] < 1e-3
