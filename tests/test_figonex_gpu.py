"""The Figonex design on the GPU against its plain restatement (tests/plain_figonex.py): every mechanism alone, then
whole models of several shapes through the engine: prompts, token-by-token decoding (graphs included), prompts cut
into portions, unequal batches, slots and blocks that are used again, long decoding over the edges of cache blocks and
of the decode kernels' key splits, greedy generation, the trace program and the command line."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import figonex_models as fm
import plain_figonex as pf

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16}


def _weights(which, mild):
    """Sharp weights for the float32 comparisons (peaked attention rows, saturated gates: a dropped key or a lost state
    shows), mild ones for bfloat16, where 16-bit rounding of scores of magnitude ten would itself move the softmax by
    several percent."""
    i = list(fm.CONFIGS).index(which)
    if mild:
        return fm.tensors(fm.CONFIGS[which], seed=31 + i, std=0.04, wide=1.5)
    return fm.tensors(fm.CONFIGS[which], seed=11 + i)


def K(which, dtype):
    return which + ("_mild" if dtype == "bf16" else "")


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("figonex")
    out = {}
    for which, cfg in fm.CONFIGS.items():
        out[which] = fm.write_folder(str(root / which), cfg, _weights(which, False))
        out[which + "_mild"] = fm.write_folder(str(root / (which + "_mild")), cfg, _weights(which, True))
    return out


class Oracle:
    def __init__(self, cfg, weights):
        self.cfg, self.weights, self._memo = cfg, weights, {}

    def logits(self, ids):
        key = tuple(ids)
        if key not in self._memo:
            self._memo[key] = pf.logits(self.cfg, self.weights, ids)
        return self._memo[key]

    def moved_by_rounding(self, ids):
        """Per position, how far 32-bit arithmetic moves the plain implementation's own logits (largest difference over
        the vocabulary between its float32 and its float64 run)."""
        key = ("moved",) + tuple(ids)
        if key not in self._memo:
            single = pf.logits(self.cfg, self.weights, ids, dtype=torch.float32).double()
            self._memo[key] = (single - self.logits(ids)).abs().max(-1).values
        return self._memo[key]


@pytest.fixture(scope="module")
def oracles():
    out = {}
    for which, cfg in fm.CONFIGS.items():
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


def close(got, want, dtype, loose=1.0):
    want = want.to(torch.float64)
    got = got.detach().cpu().to(torch.float64)
    assert got.shape == want.shape and torch.isfinite(got).all()
    top = want.abs().max().item()
    if dtype == "fp32":
        torch.testing.assert_close(got, want, atol=3e-5 * loose * max(1.0, top), rtol=1e-4 * loose)
    else:
        torch.testing.assert_close(got, want, atol=0.03 * loose * top, rtol=0.03 * loose)


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

    cache = Cache([mixer.cache_request()], max_tokens=1280 * lanes, max_positions=1280, dtype=dtype, device="cuda")
    slots = cache.begin(lanes)
    out, at = [], 0
    for n in cuts:
        before = cache.prepare(slots, [n] * lanes)
        batch = Batch.from_lists(slots, before, [[0] * n] * lanes, [[]] * lanes, "cuda")
        piece = x[at:at + n].contiguous()
        y = mixer.forward(piece.repeat(lanes, 1) if lanes > 1 else piece, batch, cache.layer_view(0), True)
        for lane in range(1, lanes):
            assert torch.equal(y[:n], y[lane * n:(lane + 1) * n])
        out.append(y[:n])
        cache.commit(slots, [n] * lanes)
        at += n
    assert at == x.shape[0]
    return torch.cat(out)


def pad_rows(t, rows):
    return torch.cat([t, torch.zeros(rows - t.shape[0], t.shape[1], dtype=t.dtype)]) if rows > t.shape[0] else t


# ---- mechanisms alone ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("dim", [36, 256, 1000, 5000])
def test_layer_norm_of_an_output_on_its_way_into_the_stream(dtype, dim):
    """stream += LN(delta) * w * s, and the norm of the sum; the rows have a large common offset, which a norm that
    forgot to take the mean off (or took the variance around zero) would show."""
    from fms_b200.config import NormSpec
    from fms_b200.parts import build_norm
    from fms_b200.parts.norm import NormedDelta

    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(dim)
    res = torch.randn(7, dim, generator=g) * 3 + 2.0
    delta = (torch.randn(7, dim, generator=g) * 5 + 9.0).to(dt)
    w = {k: (0.5 + torch.rand(dim, generator=g)).to(torch.bfloat16) for k in ("w1", "s1", "w2")}
    scaled = part_with(build_norm(NormSpec("layernorm", dim, 1e-3, options=(("layer_scale", True),))),
                       {"weight": w["w1"], "scale": w["s1"]}, dt)
    last = part_with(build_norm(NormSpec("layernorm", dim, 1e-5)), {"weight": w["w2"]}, dt)
    want_res = res.double() + pf.layer_norm(delta.double(), w["w1"].double(), 1e-3) * w["s1"].double()
    r = res.clone().cuda()
    h = scaled.add(r, delta.cuda(), dt)  # the sum, handed to the next sublayer in the compute dtype
    close(r, want_res, "fp32")
    close(h, want_res, dtype)
    r = res.clone().cuda()
    out = last.apply(r, NormedDelta(delta.cuda(), scaled), dt)  # the pending output added and the sum normed at once
    close(r, want_res, "fp32")
    close(out, pf.layer_norm(want_res, w["w2"].double(), 1e-5), dtype)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32).cuda()
    r2 = res.clone().cuda()
    out = last.apply(r2, NormedDelta(delta.cuda(), scaled), dt, rows)
    assert torch.equal(r2.cpu(), res)  # with rows the stream stays as it is
    close(out, pf.layer_norm(want_res, w["w2"].double(), 1e-5)[[5, 0, 5]], dtype)


def attention_tensors(g, dim_in, m, std=0.3):
    h, kv, k = m["heads"], m["kv_heads"], m["dim"]
    mk = lambda *s, sd=std: (torch.randn(*s, generator=g) * sd).to(torch.bfloat16)
    gain = lambda: (0.4 + 2.0 * torch.rand(k, generator=g)).to(torch.bfloat16)
    return {"q": mk(h * k, dim_in), "k": mk(kv * k, dim_in), "q.norm": gain(), "k.norm": gain(), "g": mk(h, dim_in),
            "o": mk(dim_in, h * k)}


def attention_mixer(m, dim_in, w, eps, dt):
    from fms_b200.config import MixerSpec, PositionSpec
    from fms_b200.parts import build_mixer
    from fms_b200.parts.attention import SinkAttention

    rot = m["rot"]
    factor = (rot.get("scaling") or {}).get("factor")
    position = PositionSpec("rope", head_dim=rot["dims"], theta=rot["base"], scaling=() if factor is None else (
        ("rope_type", "linear"), ("factor", factor))) if rot["dims"] else PositionSpec("none")
    spec = MixerSpec("sink_attention", dim=dim_in, nheads=m["heads"], kvheads=m["kv_heads"], head_dim=m["dim"],
                     scale=m["scale"], position=position,
                     options=(("vdim", m["dim"]), ("values", "keys"), ("rot_dims", rot["dims"]), ("pairing", "halves"),
                              ("qk_norm", "before"), ("eps", eps), ("sink_logit", 0.0), ("gate", "head")))
    rows = SinkAttention.fused_rows(m["heads"], m["kv_heads"], m["dim"], m["dim"], True, "head")
    return part_with(build_mixer(spec), {"in_proj.weight": pad_rows(torch.cat([w["q"], w["k"], w["g"]]), rows),
                                         "q_norm": w["q.norm"], "k_norm": w["k.norm"], "dense.weight": w["o"]}, dt)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(4, 2, 16, 8, None), (6, 1, 24, 24, 3.0), (2, 2, 10, 0, None), (3, 3, 64, 32, 1.5),
                                   (8, 2, 128, 64, None), (5, 5, 6, 2, None), (9, 3, 48, 48, 4.0), (2, 1, 250, 100, None)])
def test_attention_whose_values_are_its_keys_alone(dtype, shape):
    heads, kv, dim, rot, factor = shape
    m = fm.attention(heads, kv, dim, rot, 300.0, factor, (0.25 if dtype == "bf16" else 0.6) * dim ** -0.5 * 3, None)["mixer"]
    dt, dim_in, n = DTYPES[dtype], 40, 331
    g = torch.Generator().manual_seed(sum(int(x or 0) for x in shape))
    w = attention_tensors(g, dim_in, m)
    mixer = attention_mixer(m, dim_in, w, 1e-5, dt)
    x = torch.randn(n, dim_in, generator=g).to(dt)
    want = pf.attention(x.double(), m, 1e-5, {k: v.double() for k, v in w.items()}, "")
    # whole; portions whose edges fall on and beside the cache's blocks of 64; the last rows one by one (the decode
    # kernels, over the edge of their first split of 256 keys)
    for cuts in ([n], [63, 1, 1, 63, 2, 128, 73], [250] + [1] * 81):
        close(step_through(mixer, x.cuda(), cuts, dt), want, dtype)


def test_the_one_in_the_denominator_on_the_first_token_and_a_key_far_back():
    """Weights and inputs made so that a fault shows.  The first token of a sequence sees one key, so its weight is
    exp(s) / (1 + exp(s)), by hand below: a softmax without the one would give 1.  Queries read the first half of
    the input and keys the second half through the same matrix, and every seventh row's first half is the second half
    of ONE row far back (hundreds of positions: another cache block and, when decoding, another split), so that this
    key's score stands out among hundreds."""
    m = fm.attention(2, 1, 64, 8, 50.0, 2.0, 0.35, None)["mixer"]
    g = torch.Generator().manual_seed(77)
    dim_in, n = 32, 600
    w = attention_tensors(g, dim_in, m)
    a = w["k"][:, :16].clone()
    w["k"] = torch.cat([torch.zeros_like(a), a], 1)
    w["q"] = torch.cat([torch.cat([a, torch.zeros_like(a)], 1)] * 2)
    w["q.norm"] = w["k.norm"] = (0.8 + 0.4 * torch.rand(64, generator=g)).to(torch.bfloat16)
    x = torch.randn(n, dim_in, generator=g)
    for t in range(300, n, 7):
        x[t, :16] = x[t - 290 + (t % 50), 16:]
    d = {k: v.double() for k, v in w.items()}
    want = pf.attention(x.double(), m, 1e-5, d, "")
    # the oracle itself says that the far keys matter: without the first 200 keys the result is another
    near = pf.attention(x.double()[200:], m, 1e-5, d, "", first_position=200)
    assert (want[300:] - near[100:]).abs().max() > 0.3 * want.abs().max()
    # row 0 by hand (position 0: nothing turns): weight sigmoid(s) on the one value, which is the key as projected
    x0 = x[0].double()
    k0 = d["k"] @ x0
    kn = pf.rms_norm(k0, d["k.norm"], 1e-5)
    heads = []
    for h in range(2):
        qn = pf.rms_norm(d["q"][64 * h:64 * h + 64] @ x0, d["q.norm"], 1e-5)
        s = float(qn @ kn) * 0.35
        assert abs(s) < 6  # neither weight is all or nothing
        heads.append(k0 / (1 + math.exp(-s)) * torch.sigmoid(d["g"][h] @ x0))
    torch.testing.assert_close(want[0], d["o"] @ torch.cat(heads), atol=1e-9, rtol=1e-9)
    mixer = attention_mixer(m, dim_in, w, 1e-5, torch.float32)
    for cuts in ([n], [520] + [1] * 80, [2] * 300):
        close(step_through(mixer, x.cuda(), cuts, torch.float32), want, "fp32")
    # sequences of one and of two tokens, each in a slot of its own
    for t in (0, 1):
        close(step_through(mixer, x[:t + 1].cuda(), [t + 1], torch.float32), want[:t + 1], "fp32")


def memory_tensors(g, dim_in, m, gated, std=0.3, i_bias=0.0, f_bias=4.0):
    h, k, v = m["heads"], m["dim"], m["vdim"]
    mk = lambda *s, sd=std: (torch.randn(*s, generator=g) * sd).to(torch.bfloat16)
    w = {"q": mk(h * k, dim_in), "k": mk(h * k, dim_in), "v": mk(h * v, dim_in), "g": mk(h * v, dim_in),
         "norm": (0.5 + torch.rand(h * v, generator=g)).to(torch.bfloat16), "o": mk(dim_in, h * v)}
    if gated:
        w.update({"i": mk(h, dim_in), "f": mk(h, dim_in), "i.b": (i_bias + torch.randn(h, generator=g)).to(torch.bfloat16),
                  "f.b": (f_bias + torch.randn(h, generator=g)).to(torch.bfloat16)})
    return w


def memory_mixer(m, dim_in, w, eps, dt):
    from fms_b200.config import MixerSpec
    from fms_b200.parts import build_mixer
    from fms_b200.parts.linear_attention import LightningAttention, MatrixLSTM

    common = (("vdim", m["vdim"]), ("eps", eps))
    if "decay" in m:
        spec = MixerSpec("lightning_attention", dim=dim_in, nheads=m["heads"], head_dim=m["dim"],
                         options=common + (("decay", tuple(m["decay"])),))
        rows = LightningAttention.fused_rows(m["heads"], m["dim"], m["vdim"])
        fused = {"in_proj.weight": pad_rows(torch.cat([w["q"], w["k"], w["v"], w["g"]]), rows)}
    else:
        spec = MixerSpec("mlstm", dim=dim_in, nheads=m["heads"], head_dim=m["dim"], options=common + (("gate_cap", m["gate_cap"]),))
        rows = MatrixLSTM.fused_rows(m["heads"], m["dim"], m["vdim"])
        fused = {"in_proj.weight": pad_rows(torch.cat([w["q"], w["k"], w["v"], w["g"], w["i"], w["f"]]), rows),
                 "gate_bias": torch.cat([w["i.b"], w["f.b"]])}
    return part_with(build_mixer(spec), dict(fused, norm=w["norm"], **{"dense.weight": w["o"]}), dt)


MEMORY_SHAPES = [(2, 24, 56), (3, 12, 20), (1, 40, 8), (5, 6, 7), (2, 96, 40), (2, 128, 64), (1, 256, 24), (4, 64, 128)]


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", MEMORY_SHAPES)
def test_matrix_memory_under_exponential_gates_alone(dtype, shape):
    """Gates of every kind: input gates far below, around and far above the forget gates' sums (the running maximum
    follows the one or the other; with large input gates exp(-m) and the 1e-6 in the denominator are of one size),
    caps that cut the logits and caps that do not."""
    heads, dim, vdim = shape
    dt, dim_in, n = DTYPES[dtype], 40, 331
    # the norm that follows divides a head's values by their size, so the read-out's denominator shows only where eps
    # counts beside them: the second and third case have an eps of the values' own size and above
    for case, (cap, i_bias, f_bias, eps) in enumerate(((15.0, 7.0, 5.0, 1e-5), (2.5, -1.0, 1.0, 0.5), (8.0, -6.0, 3.0, 8.0))):
        m = fm.mlstm(heads, dim, vdim, cap, None)["mixer"]
        g = torch.Generator().manual_seed(sum(shape) + case)
        w = memory_tensors(g, dim_in, m, True, i_bias=i_bias, f_bias=f_bias)
        mixer = memory_mixer(m, dim_in, w, eps, dt)
        x = torch.randn(n, dim_in, generator=g).to(dt)
        d = {k: v.double() for k, v in w.items()}
        want = pf.mlstm(x.double(), m, eps, d, "")
        if case:  # the oracle itself says that the denominators show: with no eps the result is another
            assert (want - pf.mlstm(x.double(), m, 1e-9, d, "")).abs().max() > 0.15 * want.abs().max()
        # whole; portions of one, two, fifteen, sixteen, seventeen rows (the scans bring sixteen rows at a time) and
        # more; a prompt and then row by row
        for cuts in ([n], [1, 2, 15, 16, 17, 1, 33, 246], [250] + [1] * 81):
            close(step_through(mixer, x.cuda(), cuts, dt), want, dtype, loose=2.0)
    close(step_through(mixer, x.cuda(), [2, 329], dt, lanes=3), want, dtype, loose=2.0)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", MEMORY_SHAPES)
def test_matrix_memory_under_fixed_decays_alone(dtype, shape):
    heads, dim, vdim = shape
    dt, dim_in, n = DTYPES[dtype], 40, 331
    decays = [(1.0, 0.97, 0.3, 0.999, 0.9)[i % 5] for i in range(heads)]
    m = fm.lightning(heads, dim, vdim, decays, None)["mixer"]
    g = torch.Generator().manual_seed(sum(shape))
    w = memory_tensors(g, dim_in, m, False)
    mixer = memory_mixer(m, dim_in, w, 1e-5, dt)
    x = torch.randn(n, dim_in, generator=g).to(dt)
    want = pf.lightning(x.double(), m, 1e-5, {k: v.double() for k, v in w.items()}, "")
    for cuts in ([n], [1, 2, 15, 16, 17, 1, 33, 246], [250] + [1] * 81):
        close(step_through(mixer, x.cuda(), cuts, dt), want, dtype, loose=2.0)
    close(step_through(mixer, x.cuda(), [2, 329], dt, lanes=3), want, dtype, loose=2.0)


def test_memories_that_keep_the_first_tokens_for_a_thousand_steps():
    """A decay of exactly 1 and one of 0.999, and forget gates that stay open: what the first tokens wrote is still read
    1,100 tokens later (the oracle without the first 200 tokens gives another result), in a prompt, in portions and
    token by token."""
    dim_in, n = 24, 1100
    g = torch.Generator().manual_seed(9)
    x = torch.randn(n, dim_in, generator=g)
    x[:200] *= 3.0
    for m in (fm.lightning(3, 16, 24, (1.0, 0.999, 0.5), None)["mixer"], fm.mlstm(2, 16, 24, 9.0, None)["mixer"]):
        gated = "gate_cap" in m
        w = memory_tensors(g, dim_in, m, gated, i_bias=-1.0, f_bias=9.0)
        if gated:
            w["f"] = w["f"] * 0.1
        d = {k: v.double() for k, v in w.items()}
        plain = pf.mlstm if gated else pf.lightning
        eps = 0.3 if gated else 1e-5  # with the gates: large enough for the read-out's denominator to show
        want = plain(x.double(), m, eps, d, "")
        late = plain(x.double()[200:], m, eps, d, "")
        assert (want[1000:] - late[800:]).abs().max() > 0.1 * want.abs().max()
        mixer = memory_mixer(m, dim_in, w, eps, torch.float32)
        for cuts in ([n], [1000] + [1] * 100, [7] * 100 + [400]):
            close(step_through(mixer, x.cuda(), cuts, torch.float32), want, "fp32", loose=3.0)


# ---- whole models -------------------------------------------------------------------------------------
def close_logits(got, oracle, ids, dtype, rows=None):
    """float32: as sharp as for a mechanism alone.  Where that fails, a position is allowed four times what 32-bit
    rounding does to the plain implementation itself there: a sublayer's output is normed to unit size whatever it was,
    so where a read-out nearly cancels (a query across the keys a memory holds) its rounding comes back at full
    size, in any 32-bit implementation; such positions are one in hundreds and the allowance is theirs alone.
    bfloat16: every sublayer reads the stream rounded to 16 bits, and the roundings of up to a dozen sublayers reach
    the logits at full weight; the bound is three times a single mechanism's, one value in a thousand may lie up to
    twice as far (the positions above again), none farther."""
    want = oracle.logits(ids)
    want = want if rows is None else want[rows]
    if dtype == "fp32":
        try:
            close(got, want, dtype)
        except AssertionError:
            moved = oracle.moved_by_rounding(ids)
            moved = moved if rows is None else moved[rows]
            diff = (got.detach().cpu().double() - want.double()).abs()
            bound = 3e-5 * max(1.0, want.abs().max().item()) + 1e-4 * want.abs() + 4.0 * moved[:, None]
            assert got.shape == want.shape and bool((diff <= bound).all()), f"{int((diff > bound).sum())} values differ, by up to {diff.max():.3g}"
        return
    got = got.detach().cpu().double()
    assert got.shape == want.shape and torch.isfinite(got).all()
    diff = (got - want.double()).abs()
    bound = 0.09 * want.abs().max().item() + 0.09 * want.abs()
    assert int((diff > bound).sum()) <= want.numel() // 1000 and bool((diff <= 2 * bound).all()), \
        f"{int((diff > bound).sum())} of {want.numel()} values differ, by up to {diff.max():.3g} (bound {bound.min():.3g})"


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("which", ["p", "q", "r", "s"])
def test_whole_prompts_alone(folders, oracles, which, dtype):
    model = model_of(folders, which, dtype)
    engine = model.new_engine(max_tokens=1024, sampling=False)
    for i, n in enumerate((1, 2, 63, 64, 65, 300)):
        ids = fm.prompt(fm.CONFIGS[which], n, i)
        (slot,) = engine.begin(1)
        got = engine.step([slot], [ids], [list(range(n))])
        engine.release([slot])
        close_logits(got, oracles[K(which, dtype)], ids, dtype)
    engine.check()
    assert engine.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in engine.cache.groups if hasattr(g, "pool"))


def test_the_stream_after_every_layer(folders):
    """The residual stream after each layer, float32, against the oracle's, layers that run with an earlier layer's
    weights included.  The engine keeps a layer's last output pending for the kernel that adds it, so the stream after
    layer i is the stream the next layer sees plus that output's norm, taken here with the oracle's layer norm."""
    which = "p"
    cfg, weights = fm.CONFIGS[which], _weights(which, False)
    model = model_of(folders, which, "fp32")
    ids = fm.prompt(cfg, 90, 7)
    want, got = [], []
    pf.logits(cfg, weights, ids, layers_out=want)
    blocks = model.decoder.blocks
    calls = iter(range(len(blocks)))
    originals = {id(b): b.forward for b in blocks}

    def recording(block):
        def forward(residual, pending, batch, view, writes_cache, dtype):
            i = next(calls)
            out = originals[id(block)](residual, pending, batch, view, writes_cache, dtype)
            j = i
            while cfg["layers"][j].get("weights_of") is not None:
                j = cfg["layers"][j]["weights_of"]
            last = "2" if cfg["layers"][i]["mlp"] is not None else "1"
            w, s = weights[f"l{j}.norm{last}"].double(), weights[f"l{j}.ls{last}"].double()
            got.append(residual.double().cpu() + pf.layer_norm(out.delta.double().cpu(), w, cfg["norm"]["eps"]) * s)
            return out
        return forward

    try:
        for b in set(blocks):
            b.forward = recording(b)
        engine = model.new_engine(max_tokens=256, sampling=False)
        (slot,) = engine.begin(1)
        engine.step([slot], [ids], [[0]])
        engine.release([slot])
    finally:
        for b in set(blocks):
            del b.forward
    assert len(got) == len(cfg["layers"])
    for have, ref in zip(got, want):
        close(have, ref, "fp32")


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "fp32"), ("r", "bf16"), ("s", "fp32")])
def test_token_by_token_from_the_first_token(folders, oracles, which, dtype):
    """Decode steps from a sequence's very first token (the first plain, the second captured, the rest replayed), over
    the edge of a cache block, twice in the same slot."""
    engine = model_of(folders, which, dtype).new_engine(max_tokens=256, sampling=False)
    for rep in range(2):
        ids = fm.prompt(fm.CONFIGS[which], 70, 20 + rep)
        (slot,) = engine.begin(1)
        got = torch.cat([engine.step([slot], [[t]], [[0]]) for t in ids])
        engine.release([slot])
        close_logits(got, oracles[K(which, dtype)], ids, dtype)
    assert engine.graphs_captured >= 1
    engine.check()


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "bf16"), ("r", "fp32"), ("s", "bf16")])
def test_prompt_then_long_decoding_over_split_edges(folders, oracles, which, dtype):
    """A prompt of 250 tokens, then 290 tokens one by one: the decode kernels go from one split of 256 keys to two and
    to three, the cache from its fourth block to its ninth, and the memories carry their states for 290 steps."""
    engine = model_of(folders, which, dtype).new_engine(max_tokens=1024, sampling=False)
    ids = fm.prompt(fm.CONFIGS[which], 540, 31)
    (slot,) = engine.begin(1)
    got = [engine.step([slot], [ids[:250]], [list(range(250))])]
    got += [engine.step([slot], [[t]], [[0]]) for t in ids[250:]]
    engine.release([slot])
    close_logits(torch.cat(got), oracles[K(which, dtype)], ids, dtype)
    engine.check()


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "fp32"), ("r", "fp32"), ("s", "fp32"), ("p", "bf16"), ("s", "bf16")])
def test_prompts_cut_into_portions(folders, oracles, which, dtype):
    engine = model_of(folders, which, dtype).new_engine(max_tokens=1024, sampling=False)
    ids = fm.prompt(fm.CONFIGS[which], 420, 41)
    for cuts in ([2, 3, 59, 1, 64, 65, 6, 220], [193, 2, 225], [1, 1, 2, 416], [2] * 40 + [340]):
        (slot,) = engine.begin(1)
        got, at = [], 0
        for n in cuts:
            got.append(engine.step([slot], [ids[at:at + n]], [list(range(n))]))
            at += n
        engine.release([slot])
        close_logits(torch.cat(got), oracles[K(which, dtype)], ids, dtype)
    engine.check()


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_a_wider_model_whole_in_portions_and_decoding(folders, oracles, dtype):
    """Width 512 with heads and memories of 128: the kernels that larger models run (tensor-core products and
    attention of a prompt in bfloat16, sixteen state rows a thread in the scans)."""
    which = "w"
    engine = model_of(folders, which, dtype).new_engine(max_tokens=1024, sampling=False)
    ids = fm.prompt(fm.CONFIGS[which], 300, 43)
    for cuts in ([300], [180, 2, 118], [258] + [1] * 42):
        (slot,) = engine.begin(1)
        got, at = [], 0
        for n in cuts:
            got.append(engine.step([slot], [ids[at:at + n]], [list(range(n))]))
            at += n
        engine.release([slot])
        close_logits(torch.cat(got), oracles[K(which, dtype)], ids, dtype)
    engine.check()


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "fp32"), ("r", "fp32"), ("s", "fp32"), ("q", "bf16"), ("s", "bf16")])
def test_unequal_batches_freed_slots_and_poisoned_blocks(folders, oracles, which, dtype):
    """Requests of unequal lengths start together and go on one token at a time while the shorter ones end; then
    everything the cache holds is filled with NaN (keys, state matrices, normalizers and maxima) and new requests take
    the freed slots and blocks.  Every request against the oracle, alone."""
    cfg = fm.CONFIGS[which]
    engine = model_of(folders, which, dtype).new_engine(max_tokens=64 * 12, max_slots=5, sampling=False)
    for round_ in range(2):
        lengths, extra = ((1, 70, 5, 131, 64), (3, 9, 0, 12, 12)) if round_ == 0 else ((210, 2, 33), (5, 5, 1))
        full = [fm.prompt(cfg, n + e, 50 + 10 * round_ + i) for i, (n, e) in enumerate(zip(lengths, extra))]
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
            close_logits(torch.cat(got[i]), oracles[K(which, dtype)], f, dtype)
        assert engine.cache.slots.n_held == 0
        for g in engine.cache.groups:
            g.storage.fill_(float("nan") if g.storage.is_floating_point() else 12345)
    engine.check()


def test_many_sequences_in_one_decode_step_fill_rows_and_graphs(folders, oracles):
    """Eleven sequences decode together (filled up to twelve rows with rows in the spare slot), then nine of them."""
    which, cfg = "p", fm.CONFIGS["p"]
    engine = model_of(folders, which, "fp32").new_engine(max_tokens=64 * 24, sampling=False)
    full = [fm.prompt(cfg, 3 + 5 * i + 6, 70 + i) for i in range(11)]
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
        want = oracles[which].logits(f)
        close(torch.cat(got[i]), want[len(f) - 6: len(f) - 6 + len(got[i])], "fp32")
    engine.check()


def test_greedy_generation_through_generate(folders, oracles):
    from fms_b200.utils.generation import generate

    which, cfg = "q", fm.CONFIGS["q"]
    model = model_of(folders, which, "fp32")
    prompts = [fm.prompt(cfg, n, 80 + i) for i, n in enumerate((5, 1, 40))]
    out = generate(model, [torch.tensor(p) for p in prompts], max_new_tokens=10, do_sample=False)
    for p, o in zip(prompts, out):
        o = o.tolist()
        assert o[: len(p)] == p and len(o) == len(p) + 10
        for k in range(len(p), len(o)):  # every new token is the oracle's choice given what came before
            row = oracles[which].logits(o[:k])[-1]
            best = row.topk(2).values
            if best[0] - best[1] > 1e-3:
                assert o[k] == int(row.argmax())


def _trace(folder, dtype, steps, out_dir, max_tokens):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]


def test_trace_program_replays_a_batch(folders, oracles, tmp_path):
    which, cfg = "r", fm.CONFIGS["r"]
    a, b = fm.prompt(cfg, 70, 90), fm.prompt(cfg, 9, 91)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for t in range(4):
        steps.append({"step": t + 1, "entries": [{"id": "a", "tokens": [a[66 + t]], "want": [0]},
                                                  {"id": "b", "tokens": [b[5 + t]], "want": [0] if t % 2 else []}],
                      "end": ["a", "b"] if t == 3 else []})
    _trace(folders[which], "float32", steps, tmp_path, 256)
    wa, wb = oracles[which].logits(a), oracles[which].logits(b)
    read = lambda i: torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))
    close(read(0), torch.stack([wa[0], wa[65], wb[4]]), "fp32")
    for t in range(4):
        want = [wa[66 + t]] + ([wb[5 + t]] if t % 2 else [])
        close(read(t + 1), torch.stack(want), "fp32")


def test_trace_program_with_many_short_requests_and_no_room_to_spare(folders, oracles, tmp_path):
    """Six requests of three tokens in one batch with --max-tokens 18, the tokens they hold and not one more, in
    bfloat16; a step in which nothing is wanted still reports that it is done."""
    which, cfg = "q_mild", fm.CONFIGS["q"]
    reqs = [fm.prompt(cfg, 3, 120 + i) for i in range(6)]
    steps = [{"step": 0, "entries": [{"id": str(i), "tokens": r[:2], "want": []} for i, r in enumerate(reqs)], "end": []},
             {"step": 1, "entries": [{"id": str(i), "tokens": r[2:], "want": [0]} for i, r in enumerate(reqs)],
              "end": [str(i) for i in range(6)]}]
    _trace(folders[which], "bfloat16", steps, tmp_path, 18)
    assert not os.path.exists(os.path.join(str(tmp_path), "0.f32"))
    got = torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), "1.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))
    for i, r in enumerate(reqs):
        close_logits(got[i:i + 1], oracles[which], r, "bf16", rows=[2])


def test_command_line_and_sampling(folders, oracles):
    """The framework's command line finds the design through config.json: greedy tokens equal the oracle's choices; with
    sampling (temperature, top-k) every token is among the oracle's k best given what came before."""
    from fms_b200.utils.generation import generate

    which, cfg = "p", fm.CONFIGS["p"]
    prompts = [fm.prompt(cfg, n, 95 + i) for i, n in enumerate((4, 9))]
    args = [sys.executable, os.path.join(ROOT, "bin", "fms_inference"), "--architecture", "hf_pretrained", "--model_path", folders[which],
            "--default_dtype", "fp32", "--batch_input", "--max_new_tokens", "6", "--deterministic"]
    for p in prompts:
        args += ["--prompt_ids", ",".join(str(t) for t in p)]
    proc = subprocess.run(args, capture_output=True, text=True, timeout=900)
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
