"""Giganex on the CPU: configuration, registry, checkpoint adapter, the cache's entries, the one error for a checkpoint
that does not fit; and the plain restatement against itself (what a run, a window and a cap do at their edges, the
recurrence carried over a cut, the stretched frequencies, the routing's weights)."""
import json
import math

import pytest
import torch

import giganex_models as gm
import plain_giganex as pg


def test_config_json_round_trip_registry_and_fused_tensors(tmp_path):
    from fms_b200 import models
    from fms_b200.cache.requests import KVRequest, StateRequest
    from fms_b200.models import get_model
    from fms_b200.models.giganex import Giganex

    assert "giganex" in models.list_models() and "tiny" in models.list_variants("giganex")
    cfg = gm.CONFIGS["p"]
    folder = gm.write_folder(str(tmp_path / "p"), cfg, gm.tensors(cfg, 1))
    model = get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")  # found by "architecture"
    assert isinstance(model, Giganex)
    spec = model.decoder_spec()
    assert [b.mixer.kind for b in spec.layers] == ["latent_attention", "parallel", "sink_attention", "parallel"]
    assert all(b.arrangement == "parallel_residual" for b in spec.layers)
    assert [None if b.feed_forward is None else b.feed_forward.kind for b in spec.layers] == ["routed_experts", "glu", "routed_experts", None]
    assert dict(spec.final_norm.options)["groups"] == 3 and spec.final_norm.kind == "group_rmsnorm"
    assert spec.layers[0].mixer.window == 20 and dict(spec.layers[2].mixer.options)["chunk"] == 50
    sd = model.state_dict()
    assert sd["layers.0.mix.in_proj.weight"].shape == (18 + 6 + 14, 48)  # [dkv; dq]
    assert sd["layers.0.mix.q_up.weight"].shape == (3 * 16, 14) and sd["layers.0.mlp.up"].shape == (5, 20, 48)
    assert sd["layers.0.mlp.down"].shape == (5, 48, 20) and sd["layers.0.mlp.correction"].shape == (5,)
    assert sd["layers.1.mix.left.in_proj.weight"].shape == (4 * 24 + 24 + 8 + 4 * 8, 48)
    assert sd["layers.1.mix.left.in_proj.bias"][-32:].abs().max() == 0 and sd["layers.1.mix.left.dense.bias"].shape == (48,)
    # [q; k; v; b; a; zeros up to a multiple of 8; g]: 128 channels + 8 -> the gates begin at row 136
    w = sd["layers.1.mix.right.in_proj.weight"]
    assert w.shape == (136 + 80, 48) and sd["layers.1.mix.right.conv"].shape == (128, 2)
    raw = gm.tensors(cfg, 1)
    assert torch.equal(w[128:132], raw["l1.mix.right.b"].float()) and torch.equal(w[132:136], raw["l1.mix.right.a"].float())
    assert torch.equal(w[136:], raw["l1.mix.right.g"].float())
    assert sd["layers.2.mix.in_proj.weight"].shape == (4 * 24 + 24 + 8, 48) and "layers.2.mix.in_proj.bias" not in sd
    requests = model.decoder.cache_requests()
    assert isinstance(requests[0], KVRequest) and requests[0].head_dim == 24 and requests[0].planes == 1
    kv, matrix, tail = requests[1]
    assert isinstance(kv, KVRequest) and kv.head_dim == 32 and kv.kvheads == 1  # heads of 24 and 8, padded to 32
    assert isinstance(matrix, StateRequest) and matrix.shape == (4, 20, 12) and tail.shape == (1, 128)
    assert json.loads(json.dumps(model.config_json())) == cfg


def test_a_checkpoint_that_does_not_fit_is_refused_with_one_error(tmp_path):
    from fms_b200.models import get_model
    from fms_b200.weights import WeightError

    cfg = gm.CONFIGS["q"]
    weights = gm.tensors(cfg, 2)
    del weights["l1.mix.left.o.b"], weights["l1.mix.right.k.conv"], weights["l1.mlp.e2.down"]
    weights["l0.mix.o"] = weights["l0.mix.o"][:, :-1]
    weights["stray"] = torch.zeros(3, dtype=torch.bfloat16)
    folder = gm.write_folder(str(tmp_path / "q"), cfg, weights)
    with pytest.raises(WeightError) as e:
        get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")
    assert "layers.1.mix.left.dense.bias" in e.value.missing and "layers.1.mix.right.conv" in e.value.missing
    assert "layers.1.mlp.down" in e.value.missing
    assert "stray" in e.value.unexpected and any(n == "layers.0.mix.dense.weight" for n, _, _ in e.value.wrong_shapes)


def test_config_json_of_another_design_or_with_unknown_layers_is_refused():
    from fms_b200.models.giganex import Giganex

    with pytest.raises(ValueError):
        Giganex.config_from_json({"architecture": "Other"})
    bad = json.loads(json.dumps(gm.CONFIGS["r"]))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError, match="convolution"):
        Giganex.config_from_json(bad)
    bad = json.loads(json.dumps(gm.CONFIGS["r"]))
    bad["layers"][1]["mlp"]["kind"] = "sparse"
    with pytest.raises(ValueError, match="sparse"):
        Giganex.config_from_json(bad)
    bad = json.loads(json.dumps(gm.CONFIGS["r"]))
    bad["norm"]["groups"] = 5  # 36 values do not go into five runs
    with pytest.raises(ValueError):
        Giganex.config_from_json(bad)


def test_sizes_that_config_json_leaves_out_come_from_the_shapes(tmp_path):
    from fms_b200.models import get_model

    cfg = json.loads(json.dumps(gm.CONFIGS["p"]))
    weights = gm.tensors(cfg, 3)
    del cfg["layers"][0]["mixer"]["q_rank"], cfg["layers"][0]["mixer"]["kv_rank"], cfg["layers"][1]["mixer"]["right"]["conv"]
    del cfg["layers"][1]["mlp"]["ff"], cfg["layers"][0]["mlp"]["expert"]["ff"], cfg["layers"][0]["mlp"]["router"]["experts"]
    del cfg["layers"][2]["mixer"]["kv_heads"]  # as many key heads as heads would be read; the checkpoint has one: refused
    folder = gm.write_folder(str(tmp_path / "p"), cfg, weights)
    from fms_b200.weights import WeightError

    with pytest.raises(WeightError):
        get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")
    cfg["layers"][2]["mixer"]["kv_heads"] = 1
    folder = gm.write_folder(str(tmp_path / "p2"), cfg, weights)
    model = get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")
    assert model.config_json() == gm.CONFIGS["p"]


def test_random_weights_of_a_registered_variant():
    from fms_b200.models import get_model

    model = get_model("giganex", "tiny", device_type="cpu", data_type="fp32", seed=4)
    names = {t.name for t in model.checkpoint_layout()}
    assert {"embed", "final.norm", "head", "l0.mix.left.o.b", "l0.mix.right.a", "l1.mix.dq.norm", "l1.mlp.e7.down",
            "l1.mlp.correction", "l2.mix.k"} <= names
    assert abs(float(model.state_dict()["layers.0.norm1.weight"].mean()) - 1) < 0.1


def test_plain_masks_at_their_edges():
    ok = pg.visible(9, "window", 3)
    assert ok[5].tolist() == [False, False, False, True, True, True, False, False, False]
    assert ok[1].tolist() == [True, True] + [False] * 7
    ok = pg.visible(9, "chunk", 4)
    assert ok[3].tolist() == [True] * 4 + [False] * 5 and ok[4].tolist() == [False] * 4 + [True] + [False] * 4
    assert ok[7].tolist() == [False] * 4 + [True] * 4 + [False] and ok[8].tolist() == [False] * 8 + [True]
    assert pg.visible(3, "causal", 0).tolist() == [[True, False, False], [True, True, False], [True, True, True]]


def test_plain_group_norm_and_capped_scores():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 12, generator=g, dtype=torch.float64)
    w = torch.randn(12, generator=g, dtype=torch.float64)
    out = pg.group_norm(x, w, 1e-5, 3)
    for r in range(3):
        part = x[:, 4 * r:4 * r + 4]
        torch.testing.assert_close(out[:, 4 * r:4 * r + 4], part / torch.sqrt((part * part).mean(-1, keepdim=True) + 1e-5) * w[4 * r:4 * r + 4])
    # a cap far above the scores changes nothing; a small one bounds them, so that two keys whose scores differ hugely
    # still share the weight
    m = gm.left(1, 1, 2, 2, 1.0, 1e6)
    t = {"q": torch.eye(2, dtype=torch.float64) * 30, "q.b": torch.zeros(2, dtype=torch.float64), "k": torch.eye(2, dtype=torch.float64),
         "k.b": torch.zeros(2, dtype=torch.float64), "v": torch.eye(2, dtype=torch.float64), "v.b": torch.zeros(2, dtype=torch.float64),
         "g": torch.zeros(2, 2, dtype=torch.float64), "o": torch.eye(2, dtype=torch.float64), "o.b": torch.tensor([0.0, 7.0], dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 0.0]], dtype=torch.float64)
    sharp = pg.capped_attention(h, t, "", m)
    torch.testing.assert_close(sharp[2], torch.tensor([0.5, 7.0], dtype=torch.float64), atol=1e-9, rtol=0)  # two equal keys of three hold all
    soft = pg.capped_attention(h, t, "", dict(m, softcap=1.0))
    e = math.exp(math.tanh(30.0)), math.exp(0.0)
    torch.testing.assert_close(soft[2, 0], torch.tensor(0.5 * 2 * e[0] / (2 * e[0] + e[1]), dtype=torch.float64))


def test_plain_delta_rule_carried_over_a_cut():
    """The restatement's recurrence restarted from the middle with the state and the convolutions' inputs of the first
    half gives the second half: what a step function must carry is exactly that."""
    g = torch.Generator().manual_seed(3)
    m = gm.right(4, 2, 6, 5, 3)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    t = {"q": r(12, 9), "k": r(12, 9), "v": r(20, 9), "q.conv": r(12, 3), "k.conv": r(12, 3), "v.conv": r(20, 3), "b": r(4, 9), "a": r(4, 9),
         "A_log": r(4), "dt_bias": r(4), "norm": r(5), "g": r(20, 9), "o": r(9, 20)}
    h = r(17, 9)
    whole, state, tail = pg.delta_rule(h, t, "", m, 1e-5)
    first, s1, t1 = pg.delta_rule(h[:7], t, "", m, 1e-5)
    second, s2, _ = pg.delta_rule(h[7:], t, "", m, 1e-5, state=s1, before=t1)
    torch.testing.assert_close(torch.cat([first, second]), whole)
    torch.testing.assert_close(s2, state)
    assert t1.shape == (2, 44)


def test_plain_stretched_frequencies_and_routing():
    f, mult = pg.stretched_frequencies(8, 10000.0, {"factor": 4.0, "original": 100, "fast": 4.0, "slow": 1.0})
    plain = [10000.0 ** (-2 * i / 8) for i in range(4)]
    # the pairs whose waves make 4 turns and 1 turn over 100 positions: 8 ln(100 / 8 pi) / (2 ln 10000) = 0.6 -> 0 and
    # 8 ln(100 / 2 pi) / (2 ln 10000) = 1.2 -> 2
    assert f[0] == plain[0] and abs(f[1] - (plain[1] / 4 * 0.5 + plain[1] * 0.5)) < 1e-15 and f[2] == plain[2] / 4 and f[3] == plain[3] / 4
    assert abs(mult - (0.1 * math.log(4.0) + 1)) < 1e-15
    assert pg.stretched_frequencies(8, 10000.0, None) == (plain, 1.0)
    # the correction moves the choice, not the weights; the weights of the chosen sum to the router's scale
    w = {"router": torch.tensor([[1.0], [0.0], [-1.0]], dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 5.0], dtype=torch.float64)}
    mlp = gm.moe(3, 2, 4, 2.5)
    chosen, weights, s = pg.route(torch.tensor([[2.0]], dtype=torch.float64), w, "", mlp)
    assert sorted(chosen[0].tolist()) == [0, 2]
    torch.testing.assert_close(weights.sum(), torch.tensor(2.5, dtype=torch.float64))
    a, b = s[0, chosen[0, 0]], s[0, chosen[0, 1]]
    torch.testing.assert_close(weights[0, 0] / weights[0, 1], a / b)
