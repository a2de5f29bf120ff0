"""Figonex on the CPU: configuration, registry, checkpoint adapter, layers that share weights, the cache entries its
mixers ask for, and the one error for a checkpoint that does not fit; and the plain restatement against itself (the
recurrences carried over a cut, the one in the softmax's denominator, the rotation in halves, the running maximum)."""
import json
import math

import pytest
import torch

import figonex_models as fm
import plain_figonex as pf


def test_config_json_round_trip_registry_and_shared_layers(tmp_path):
    from fms_b200 import models
    from fms_b200.cache.requests import KVRequest, StateRequest
    from fms_b200.models import get_model
    from fms_b200.models.figonex import Figonex

    assert "figonex" in models.list_models() and "tiny" in models.list_variants("figonex")
    cfg = fm.CONFIGS["p"]
    folder = fm.write_folder(str(tmp_path / "p"), cfg, fm.tensors(cfg, 1))
    model = get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")  # found by "architecture"
    assert isinstance(model, Figonex)
    spec = model.decoder_spec()
    assert [b.mixer.kind for b in spec.layers] == ["sink_attention", "mlstm", "lightning_attention", "lightning_attention",
                                                   "sink_attention", "mlstm"]
    assert [b.weights_of for b in spec.layers] == [None, None, None, 2, 0, 1]
    assert all(b.arrangement == "output_norm" and b.mixer_norm.kind == "layernorm" for b in spec.layers)
    assert spec.embedding_scale == 3.0 and spec.final_norm.kind == "layernorm" and spec.final_norm.eps == 1e-4
    att = dict(spec.layers[0].mixer.options)
    assert att["values"] == "keys" and att["pairing"] == "halves" and att["sink_logit"] == 0.0 and att["gate"] == "head"
    assert spec.layers[0].mixer.position.scaling_dict() == {"rope_type": "linear", "factor": 4.0}
    assert dict(spec.layers[2].mixer.options)["decay"] == (0.5, 0.995) and dict(spec.layers[1].mixer.options)["gate_cap"] == 8.0
    blocks = model.decoder.blocks
    assert blocks[3] is blocks[2] and blocks[4] is blocks[0] and blocks[5] is blocks[1] and blocks[0] is not blocks[1]
    sd = model.state_dict()
    assert not any(k.startswith(("layers.3.", "layers.4.", "layers.5.")) for k in sd)
    # [q; k; g] with the four gate rows filled up to a multiple of 8; [q; k; v; g; i; f]; [q; k; v; g]
    assert sd["layers.0.mix.in_proj.weight"].shape == (4 * 24 + 24 + 8, 48)
    assert sd["layers.0.mix.in_proj.weight"][4 * 24 + 24 + 4:].abs().max() == 0
    assert sd["layers.1.mix.in_proj.weight"].shape == (2 * 3 * 12 + 2 * 3 * 20 + 6 + 2, 48)
    assert sd["layers.1.mix.gate_bias"].shape == (6,)
    assert sd["layers.2.mix.in_proj.weight"].shape == (2 * 2 * 12 + 2 * 2 * 20, 48)
    assert sd["layers.0.mlp.wg1_fused.weight"].shape == (80, 48) and sd["layers.0.norm1.scale"].shape == (48,)
    # every layer has cache entries of its own, also those that share weights
    requests = model.decoder.cache_requests()
    assert len(requests) == 6
    assert isinstance(requests[0], KVRequest) and requests[0].head_dim == 32 and requests[0].kvheads == 1 and requests[4] == requests[0]
    matrix, rest = requests[1]
    assert isinstance(matrix, StateRequest) and matrix.shape == (3, 20, 12) and rest.shape == (3, 13) and requests[5] == requests[1]
    assert requests[2].shape == (2, 20, 12) and requests[3] == requests[2]
    assert model.cache_bytes_per_token() == 2 * (2 * 1 * 32 * 4)  # two attention layers, keys and values, float32
    assert json.loads(json.dumps(model.config_json())) == cfg


def test_a_checkpoint_that_does_not_fit_is_refused_with_one_error(tmp_path):
    from fms_b200.models import get_model
    from fms_b200.weights import WeightError

    cfg = fm.CONFIGS["q"]
    weights = fm.tensors(cfg, 2)
    del weights["l1.mix.q.norm"], weights["l2.mix.f.b"], weights["l0.ls1"]
    weights["l3.mix.o"] = weights["l3.mix.o"][:, :-1]
    weights["stray"] = torch.zeros(3, dtype=torch.bfloat16)
    folder = fm.write_folder(str(tmp_path / "q"), cfg, weights)
    with pytest.raises(WeightError) as e:
        get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")
    assert {"layers.1.mix.q_norm", "layers.2.mix.gate_bias", "layers.2.mix.in_proj.weight", "layers.0.norm1.scale"} <= set(e.value.missing)
    assert "stray" in e.value.unexpected and any(n == "layers.3.mix.dense.weight" for n, _, _ in e.value.wrong_shapes)


def test_config_json_of_another_design_or_with_unknown_layers_is_refused():
    from fms_b200.models.figonex import Figonex

    with pytest.raises(ValueError):
        Figonex.config_from_json({"architecture": "Other"})
    bad = json.loads(json.dumps(fm.CONFIGS["r"]))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError, match="convolution"):
        Figonex.config_from_json(bad)
    chained = json.loads(json.dumps(fm.CONFIGS["p"]))
    chained["layers"].append(dict(chained["layers"][3], weights_of=3))  # the weights of a layer that takes another's
    spec = Figonex(Figonex.config_from_json(chained)).decoder_spec()
    assert [b.weights_of for b in spec.layers] == [None, None, None, 2, 0, 1, 2]
    bad = json.loads(json.dumps(fm.CONFIGS["p"]))
    bad["layers"][3]["weights_of"] = 0  # a layer of another type
    with pytest.raises(ValueError, match="weights_of"):
        Figonex.config_from_json(bad)
    bad = json.loads(json.dumps(fm.CONFIGS["q"]))
    bad["layers"][0]["mixer"]["decay"] = [0.5, 0.5]  # two decays for one head
    with pytest.raises(ValueError, match="decays"):
        Figonex.config_from_json(bad)
    bad = json.loads(json.dumps(fm.CONFIGS["q"]))
    bad["layers"][1]["mlp"]["kind"] = "routed"
    with pytest.raises(ValueError, match="routed"):
        Figonex.config_from_json(bad)


def test_random_weights_of_a_registered_variant():
    from fms_b200.models import get_model

    model = get_model("figonex", "tiny", device_type="cpu", data_type="fp32", seed=4)
    names = {t.name for t in model.checkpoint_layout()}
    assert {"embed", "final.norm", "head", "l0.mix.i.b", "l0.ls2", "l1.mix.q.norm", "l3.mix.norm", "l1.mlp.down"} <= names
    assert not any(n.startswith("l1.mix.v") for n in names)  # attention has no value projection
    assert abs(float(model.state_dict()["layers.0.norm1.scale"].mean()) - 1.0) < 0.1


# ---- the plain restatement against itself -------------------------------------------------------------
def _r(g, *s):
    return torch.randn(*s, generator=g, dtype=torch.float64)


def test_plain_recurrences_carried_over_a_cut():
    """Restarted from the middle with the state of the first half, the restatement's recurrences give the second half:
    what a step function must carry is exactly that (S for one, S, n and m for the other)."""
    g = torch.Generator().manual_seed(0)
    h = _r(g, 13, 7)
    m = fm.lightning(2, 3, 4, (0.8, 0.99), None)["mixer"]
    t = {"q": _r(g, 6, 7), "k": _r(g, 6, 7), "v": _r(g, 8, 7), "g": _r(g, 8, 7), "norm": _r(g, 8), "o": _r(g, 7, 8)}
    whole, state = pf.lightning(h, m, 1e-5, t, ""), {}
    parts = [pf.lightning(h[:5], m, 1e-5, t, "", state), pf.lightning(h[5:], m, 1e-5, t, "", state)]
    torch.testing.assert_close(torch.cat(parts), whole)
    m = fm.mlstm(2, 3, 4, 6.0, None)["mixer"]
    t.update({"i": _r(g, 2, 7), "f": _r(g, 2, 7), "i.b": _r(g, 2), "f.b": _r(g, 2) + 3})
    whole, state = pf.mlstm(h, m, 1e-5, t, ""), {}
    parts = [pf.mlstm(h[:1], m, 1e-5, t, "", state), pf.mlstm(h[1:6], m, 1e-5, t, "", state), pf.mlstm(h[6:], m, 1e-5, t, "", state)]
    torch.testing.assert_close(torch.cat(parts), whole)


def test_plain_memory_with_a_running_maximum_that_starts_at_zero():
    """One head, keys and values of one number, gates fixed by their biases alone: the first token's output by hand.
    With i = -3 the maximum stays at its start, 0 (not at i, as it would from minus infinity): m1 = max(f + 0, i)."""
    m = fm.mlstm(1, 1, 1, 50.0, None)["mixer"]
    z = torch.zeros(1, 2, dtype=torch.float64)
    t = {"q": torch.tensor([[1.0, 0.0]], dtype=torch.float64), "k": torch.tensor([[0.0, 1.0]], dtype=torch.float64),
         "v": torch.tensor([[0.0, 1.0]], dtype=torch.float64), "g": z, "i": z, "f": z, "norm": torch.ones(1, dtype=torch.float64),
         "o": torch.ones(1, 1, dtype=torch.float64), "i.b": torch.tensor([-3.0], dtype=torch.float64),
         "f.b": torch.tensor([-0.2], dtype=torch.float64)}
    h = torch.tensor([[2.0, 0.5]], dtype=torch.float64)  # q = 2, k = v = 0.5
    i = 50 * math.tanh(-3 / 50)
    f = -math.log1p(math.exp(-50 * math.tanh(-0.2 / 50)))
    m1 = max(f, i)
    assert m1 == f  # the forget gate's logarithm is above the input gate's: from minus infinity it would have been i
    S = math.exp(i - m1) * 0.25
    n = math.exp(i - m1) * 0.5
    o = S * 2 / (max(abs(n * 2), math.exp(-m1)) + 1e-6)
    want = o / math.sqrt(o * o + 1e-5) * 0.5  # the head's rms, then sigmoid(0)
    assert abs(float(pf.mlstm(h, m, 1e-5, t, "")) - want) < 1e-12


def test_plain_attention_by_hand():
    """Two tokens, one head: the first sees itself only, and with the one in the denominator its weight is
    e^s / (1 + e^s); the value is the key as projected, not the normed and rotated one."""
    g = torch.Generator().manual_seed(2)
    m = fm.attention(1, 1, 4, 2, 10.0, 2.0, 0.7, None)["mixer"]
    t = {"q": _r(g, 4, 5), "k": _r(g, 4, 5), "q.norm": _r(g, 4), "k.norm": _r(g, 4), "g": torch.zeros(1, 5, dtype=torch.float64),
         "o": torch.eye(4, dtype=torch.float64)}
    h = _r(g, 2, 5)
    out = pf.attention(h, m, 1e-5, t, "")
    q0, k0 = h[0] @ t["q"].T, h[0] @ t["k"].T
    nq = q0 / torch.sqrt((q0 * q0).mean() + 1e-5) * t["q.norm"]
    nk = k0 / torch.sqrt((k0 * k0).mean() + 1e-5) * t["k.norm"]
    s = float(nq @ nk) * 0.7  # position 0: nothing turns
    torch.testing.assert_close(out[0], 0.5 * math.exp(s) / (1 + math.exp(s)) * k0)
    # the rotation: values 0 and 1 of a head of four are a pair (halves of the first two), angle p * 10^0 / 2
    v = torch.tensor([[[1.0, 0.0, 5.0, 7.0]]], dtype=torch.float64)
    turned = pf.rotate_halves(v, torch.tensor([3]), 2, 10.0, 2.0)
    torch.testing.assert_close(turned[0, 0], torch.tensor([math.cos(1.5), math.sin(1.5), 5.0, 7.0], dtype=torch.float64))
    # four rotated values: (0, 2) and (1, 3) are the pairs, the second with the frequency 10^(-1/2) / 2
    v = torch.tensor([[[1.0, 1.0, 0.0, 0.0]]], dtype=torch.float64)
    turned = pf.rotate_halves(v, torch.tensor([2]), 4, 10.0, 2.0)
    a = 2 * 10 ** -0.5 / 2
    torch.testing.assert_close(turned[0, 0], torch.tensor([math.cos(1.0), math.cos(a), math.sin(1.0), math.sin(a)], dtype=torch.float64))


def test_plain_whole_model_runs_with_shared_layers():
    cfg = fm.CONFIGS["p"]
    w = fm.tensors(cfg, 3)
    ids = fm.prompt(cfg, 9, 0)
    layers = []
    out = pf.logits(cfg, w, ids, layers_out=layers)
    assert out.shape == (9, cfg["vocab"]) and len(layers) == 6 and torch.isfinite(out).all()
    # causal: a later token changes nothing before it
    other = pf.logits(cfg, w, ids[:5] + [(ids[5] + 1) % cfg["vocab"]] + ids[6:])
    torch.testing.assert_close(other[:5], out[:5])
    assert (other[5:] - out[5:]).abs().max() > 1e-6
