"""Losorax on the CPU: the configuration reader and the spec it builds, the random-weights
folder, and the plain implementation's mechanisms against properties they must have."""
import copy
import json
import math

import pytest
import torch

import losorax_tiny as tiny
import plain_losorax as plain


def test_config_to_spec_and_manifest(tmp_path):
    from cretif_b200.config import load_config
    from cretif_b200.engine.model import manifest
    from cretif_b200.weights.random_model import write_random_model
    d = str(tmp_path / "m")
    write_random_model(d, tiny.L_A, seed=3)
    with open(d + "/config.json") as f:
        assert json.load(f)["architecture"] == "Losorax"
    arch, cfg, spec = load_config(d)
    assert arch.name == "Losorax"
    # every layer has tensors; the third reads the keys and values the first stores
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, None), (1, None), (2, 0)]
    names, _ = manifest(spec)
    assert names["l0.mix.q"].shape == (64, 64) and names["l0.mix.k"].shape == (32, 64)
    assert names["l0.mix.v"].shape == (48, 64) and names["l0.mix.o"].shape == (64, 96)
    assert names["l0.mix.v.conv"].shape == (48, 3) and names["l0.mix.rel"].shape == (12, 4)
    assert "l2.mix.k" not in names and "l2.mix.v.conv" not in names and "l2.mix.q.conv" in names
    assert names["l1.mix.w1"].shape == (8, 64) and names["l1.mix.w2"].shape == (32, 8)
    assert names["l1.mix.a.b"].shape == (32,) and names["l1.mix.norm"].shape == (32,)
    assert names["l1.mlp.router"].shape == (6, 64) and names["l1.mlp.e5.down"].shape == (64, 32)
    assert names["l0.norm1.alpha"].shape == () and names["l0.norm1b.b"].shape == (64,)
    assert names["l0.ls1"].shape == (64,) and names["l0.shift"].shape == (64,)
    assert names["head"].shape == (96, 64) and names["final.norm.alpha"].shape == ()
    for layer in spec.layers:
        b = layer.branches[0]
        assert b.norm.kind == b.post_norm.kind == "dynamic_tanh" and b.shift.kind == "token_shift"
        assert b.post_norm.params["gain"] == "ls1" and "gain" not in b.norm.params
    assert all(b.shift is None for l in spec.layers for b in l.branches[1:])
    cfg_b, w = plain.read_model_folder(d)
    assert set(w) == set(names)


def test_sizes_that_only_the_tensors_know(tmp_path):
    """The rows of the distance-bias table and the decay's low rank are whatever the file has."""
    from cretif_b200.config import load_config
    from cretif_b200.engine.model import manifest
    from cretif_b200.weights import load_weights
    from cretif_b200.weights.loader import random_weights, write_model_folder
    from cretif_b200.weights.safetensors_io import CheckpointError
    cfg = copy.deepcopy(tiny.L_A)
    from cretif_b200.config import build_losorax_spec, losorax_config_from_dict
    names, _ = manifest(build_losorax_spec(losorax_config_from_dict(cfg)))
    tensors = random_weights(names, 5, torch.bfloat16)
    tensors["l0.mix.rel"] = torch.zeros(20, 4, dtype=torch.bfloat16)
    tensors["l1.mix.w1"] = torch.zeros(3, 64, dtype=torch.bfloat16)
    tensors["l1.mix.w2"] = torch.zeros(32, 3, dtype=torch.bfloat16)
    for key in ("bias_rows", "decay_rank"):            # a checkpoint's config.json has neither
        for layer in cfg["layers"]:
            layer["mixer"].pop(key, None)
    d = str(tmp_path / "m")
    write_model_folder(d, cfg, tensors)
    _, _, spec = load_config(d)
    got = load_weights(d, *manifest(spec))
    assert got["l0.mix.rel"].shape == (20, 4) and got["l1.mix.w1"].shape == (3, 64)
    tensors["l0.norm1.alpha"] = tensors["l0.norm1.alpha"].reshape(1)     # a scalar as [1]
    write_model_folder(d, cfg, tensors)
    assert load_weights(d, *manifest(spec))["l0.norm1.alpha"].numel() == 1
    tensors["l0.mix.rel"] = torch.zeros(20, 5, dtype=torch.bfloat16)     # heads are not free
    write_model_folder(d, cfg, tensors)
    with pytest.raises(CheckpointError, match="l0.mix.rel"):
        load_weights(d, *manifest(spec))


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][0].update(type="delta"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(q_temp=3), "q_temp"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "no keys"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "vdim differs"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["layers"][1]["mixer"].pop("dim"), "dim"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(edit, text):
    from cretif_b200.config import ConfigError, losorax_config_from_dict
    cfg = copy.deepcopy(tiny.L_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        losorax_config_from_dict(cfg)


def test_a_reader_of_a_reader_is_refused():
    from cretif_b200.config import ConfigError, losorax_config_from_dict
    cfg = copy.deepcopy(tiny.L_A)
    cfg["layers"].append(copy.deepcopy(cfg["layers"][2]))
    cfg["layers"][3]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError, match="no keys"):
        losorax_config_from_dict(cfg)


def test_cache_requests_of_a_reader(tmp_path):
    """The layer that reads another's keys and values asks for none, but keeps its own saved
    query inputs and its own shifted row; every layer's shift has a state."""
    from cretif_b200.cache import KVRequest, StateRequest
    from cretif_b200.config import build_losorax_spec, losorax_config_from_dict
    from cretif_b200.engine.model import Model
    spec = build_losorax_spec(losorax_config_from_dict(tiny.L_A))
    reqs = Model(spec, torch.float32, "cpu").cache_requests()
    kv, st = reqs[(0, 0)]
    assert kv == KVRequest(2, 16, 0, value_dim=24)
    assert st == StateRequest(((64 + 32 + 48) * 2,), torch.float32)
    assert reqs[(2, 0)] == StateRequest((64 * 2,), torch.float32)
    assert reqs[(1, 0)] == StateRequest((2 * 16 * 16,), torch.float32)
    assert all(reqs[(i, 0, "shift")] == StateRequest((64,), torch.float32) for i in range(3))
    assert set(reqs) == {(0, 0), (1, 0), (2, 0), (0, 0, "shift"), (1, 0, "shift"), (2, 0, "shift")}
    spec_b = build_losorax_spec(losorax_config_from_dict(tiny.L_B))
    reqs = Model(spec_b, torch.float32, "cpu").cache_requests()
    assert reqs[(1, 0)] == KVRequest(1, 32, 0, value_dim=16)       # one tap: nothing to save
    assert reqs[(2, 0)] == StateRequest((64 * 3,), torch.float32)


@pytest.mark.parametrize("rows,far", [(32, 200.0), (12, 40), (7, 100), (2, 3), (64, 500), (9, 33.5),
                                      (6, 90), (16, 9)])
def test_the_edges_of_the_distance_rows_are_the_formula(rows, far):
    from cretif_b200.parts.attention import distance_edges
    edges = distance_edges(rows, far).tolist()
    assert edges[0] == 0 and edges == sorted(edges)
    for n in range(0, int(far) + 60):
        row = max(r for r in range(rows) if edges[r] <= n)
        assert row == plain.distance_bucket(n, rows, far), (n, row)
    with pytest.raises(ValueError):
        distance_edges(8, 4)


# ------------------------------------------------------------------ the plain mechanisms
def test_plain_blend_with_the_previous_row():
    h = torch.arange(12, dtype=torch.float64).reshape(4, 3) + 1
    out = plain.blend_with_previous(h, torch.tensor([0.0, 1.0, 0.5], dtype=torch.float64))
    assert torch.equal(out[:, 0], h[:, 0])                                   # 0: the row itself
    assert torch.equal(out[1:, 1], h[:-1, 1]) and out[0, 1] == 0             # 1: the row before
    assert out[2, 2] == 0.5 * (h[2, 2] + h[1, 2])


def test_plain_convolution_taps():
    z = torch.zeros(6, 1, dtype=torch.float64)
    z[2, 0] = 1.0
    y = plain.causal_conv(z, torch.tensor([[10.0, 20.0, 30.0]], dtype=torch.float64))
    assert y[:, 0].tolist() == [0, 0, 30.0, 20.0, 10.0, 0]    # the last tap is the present token


def test_plain_softmax_with_one_added():
    q = torch.zeros(1, 1, 4, dtype=torch.float64)
    k = torch.zeros(1, 1, 4, dtype=torch.float64)
    v = torch.ones(1, 1, 2, dtype=torch.float64)
    rel = torch.zeros(4, 1, dtype=torch.float64)
    o = plain.attention_scores_to_output(q, k, v, 1.0, rel, 10.0, torch.ones(1, dtype=torch.float64))
    assert torch.allclose(o, torch.full_like(o, 0.5))         # one key with score 0 and the added one
    rel[0, 0] = 50.0                                          # the bias is added after the scale
    o = plain.attention_scores_to_output(q, k, v, 0.0, rel, 10.0, torch.ones(1, dtype=torch.float64))
    assert torch.allclose(o, torch.ones_like(o))


def test_plain_query_gain_and_buckets():
    assert plain.query_gain(0, 0.3, 4) == 1.0 and plain.query_gain(2, 0.3, 4) == 1.0
    assert plain.query_gain(3, 0.3, 4) == pytest.approx(1 + 0.3 * math.log(2))
    assert [plain.distance_bucket(n, 8, 64) for n in (0, 3, 4, 7, 8, 15, 16, 63, 64, 1000)] == \
        [0, 3, 4, 4, 5, 5, 6, 7, 7, 7]


def test_plain_general_delta_rule_removes_along_the_key_and_decays():
    d = 4
    k = torch.zeros(3, 1, d, dtype=torch.float64)
    k[0, 0, 0] = 2.0
    k[1, 0, 0] = 2.0
    k[2, 0, 1] = 1.0
    v = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]], [[0.0, 0.0]]], dtype=torch.float64)
    r = torch.zeros(3, 1, d, dtype=torch.float64)
    r[:, 0, 0] = 1.0
    ones = torch.ones(3, 1, d, dtype=torch.float64)
    # full removal, no decay: the second write along the same key replaces the first
    o = plain.general_delta_rule(r, k, v, ones, ones)
    assert torch.allclose(o[0, 0], torch.tensor([2.0, 0.0], dtype=torch.float64), atol=1e-6)
    assert torch.allclose(o[1, 0], torch.tensor([0.0, 2.0], dtype=torch.float64), atol=1e-5)
    # no removal, decay one half per step on every channel: the first write fades
    o = plain.general_delta_rule(r, k, v, 0.5 * ones, 0.0 * ones)
    assert torch.allclose(o[1, 0], torch.tensor([1.0, 2.0], dtype=torch.float64))
    assert torch.allclose(o[2, 0], torch.tensor([0.5, 1.0], dtype=torch.float64))


def test_plain_routed_experts_scale_the_input():
    torch.manual_seed(0)
    H, F = 8, 6
    W = {"m.router": torch.randn(3, H, dtype=torch.float64)}
    for e in range(3):
        W[f"m.e{e}.gate"] = torch.randn(F, H, dtype=torch.float64)
        W[f"m.e{e}.up"] = torch.randn(F, H, dtype=torch.float64)
        W[f"m.e{e}.down"] = torch.randn(H, F, dtype=torch.float64)
    x = torch.randn(5, H, dtype=torch.float64)
    mlp = {"router": {"experts": 3, "top": 2}}
    y = plain.routed_experts(x, W, "m.", mlp)
    s = plain.sigmoid(x @ W["m.router"].T)
    for t in range(5):
        best = sorted(range(3), key=lambda e: -float(s[t, e]))[:2]
        want = sum(plain.swiglu((s[t, e] * x[t])[None], W, f"m.e{e}.")[0] for e in best)
        assert torch.allclose(y[t], want)
        # the scores are not renormalized and do not scale the output
        wrong = sum(s[t, e] * plain.swiglu(x[t][None], W, f"m.e{e}.")[0] for e in best)
        assert not torch.allclose(y[t], wrong)
