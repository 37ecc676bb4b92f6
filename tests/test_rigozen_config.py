"""Rigozen on the CPU: the configuration reader and the spec it builds, the random-weights
folder, and the plain implementation's mechanisms against properties they must have."""
import copy
import json

import pytest
import torch

import plain_rigozen as plain
import rigozen_tiny as tiny


def test_config_to_spec_and_manifest(tmp_path):
    from cretif_b200.config import load_config
    from cretif_b200.engine.model import manifest
    from cretif_b200.weights.random_model import write_random_model
    d = str(tmp_path / "m")
    write_random_model(d, tiny.R_A, seed=3)
    with open(d + "/config.json") as f:
        assert json.load(f)["architecture"] == "Rigozen"          # one class, named by a string
    arch, cfg, spec = load_config(d)
    assert arch.name == "Rigozen" and cfg.source_of(3) == 1
    # four runs of three layers with tensors; the borrowed run has a cache of its own
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, None), (1, None), (2, None), (1, None)]
    names, _ = manifest(spec)
    assert "l0.mix.q.conv" in names and names["l0.mix.q.conv"].shape == (32, 3)
    assert names["l0.mix.v"].shape == (96, 64) and names["l0.mix.norm"].shape == (24,)
    assert names["l1.mix.q.norm"].shape == (64,) and names["l1.mix.k.norm"].shape == (32,)
    assert "l1.mix.v" not in names and "l1.mlp.gate" not in names and "l1.norm2" not in names
    assert names["l2.mix.uk"].shape == (48, 40) and names["l2.mix.uv"].shape == (24, 40)
    assert names["l2.mix.sink"].shape == (3,) and "l3.norm1" not in names
    assert names["embed"].shape == (96, 64) and "final.norm" in names
    # every norm of a block is on the sublayer's output, with weights around zero
    for layer in spec.layers:
        for b in layer.branches:
            assert b.norm is None and b.post_norm.params["offset"] == 1.0
    cfg_b, w = plain.read_model_folder(d)
    assert float(w["l0.norm1"].abs().mean()) < 0.1 and set(w) == set(names)


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"].update(mask=7), "mask"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][3].update(weights_of=3), "weights_of"),
    (lambda c: c["layers"][3].update(weights_of=0), "another layer"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(edit, text):
    from cretif_b200.config import ConfigError, rigozen_config_from_dict
    cfg = copy.deepcopy(tiny.R_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        rigozen_config_from_dict(cfg)


def test_a_mixer_without_mask_or_scale_sees_every_key_at_the_usual_scale():
    from cretif_b200.config import build_rigozen_spec, rigozen_config_from_dict
    cfg = copy.deepcopy(tiny.R_A)
    del cfg["layers"][1]["mixer"]["mask"], cfg["layers"][1]["mixer"]["scale"]
    del cfg["layers"][3]["mixer"]["mask"], cfg["layers"][3]["mixer"]["scale"]
    spec = build_rigozen_spec(rigozen_config_from_dict(cfg))
    params = spec.layers[1].branches[0].part.params
    assert params["window"] == 0 and params["scale"] == 16 ** -0.5


def test_plain_delta_rule_recalls_what_it_stored():
    """Orthogonal unit keys, beta = 1, no decay: the state returns each key's value exactly,
    and writing a key again replaces its value."""
    d, e = 8, 5
    k = torch.eye(d, dtype=torch.float64)[:4].reshape(4, 1, d)
    v = torch.randn(4, 1, e, dtype=torch.float64)
    ones = torch.ones(4, 1, dtype=torch.float64)
    o = plain.delta_rule(k, k, v, ones, ones)
    assert torch.allclose(o, v)
    k2 = torch.cat([k, k[:1]]); v2 = torch.cat([v, -v[:1]])
    o2 = plain.delta_rule(k2, k2, v2, torch.ones(5, 1, dtype=torch.float64),
                          torch.ones(5, 1, dtype=torch.float64))
    assert torch.allclose(o2[4], -v[0])
    # with a decay g the first value has faded by g^3 when it is read after three more steps
    g = torch.full((4, 1), 0.5, dtype=torch.float64)
    q = k[:1].expand(4, 1, d)
    o3 = plain.delta_rule(q, k, v, ones, g)
    assert torch.allclose(o3[3], v[0] * 0.5 ** 3)


def test_plain_convolution_and_window_and_sink():
    z = torch.arange(12, dtype=torch.float64).reshape(6, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    y = plain.causal_conv(z, w)                     # last column weighs the present token
    assert y[0, 0] == 100 * z[0, 0] and y[2, 0] == z[0, 0] + 10 * z[1, 0] + 100 * z[2, 0]
    assert torch.equal(y[:, 1], z[:, 1])
    vis = plain.window_mask(6, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist()[:3] == [True, True, False]
    # a very large sink takes all the weight, a very small one none
    q = torch.randn(4, 2, 8, dtype=torch.float64); k = torch.randn(4, 1, 8, dtype=torch.float64)
    v = torch.randn(4, 1, 8, dtype=torch.float64)
    base = plain.windowed_softmax_attention(q, k, v, 0.3, 2)
    none = plain.windowed_softmax_attention(q, k, v, 0.3, 2, sink=torch.tensor([-80.0, -80.0], dtype=torch.float64))
    all_ = plain.windowed_softmax_attention(q, k, v, 0.3, 2, sink=torch.tensor([80.0, 80.0], dtype=torch.float64))
    assert torch.allclose(none, base) and all_.abs().max() < 1e-20


def test_plain_model_is_causal_and_reuses_a_layer():
    from cretif_b200.weights.random_model import write_random_model
    import tempfile
    d = tempfile.mkdtemp()
    write_random_model(d, tiny.R_A, seed=5)
    cfg, w = plain.read_model_folder(d)
    toks = tiny.tokens("A", 30, 1)
    streams = []
    full = plain.forward(cfg, w, toks, streams=streams)
    assert len(streams) == 4 and full.shape == (30, 96)
    assert torch.allclose(plain.forward(cfg, w, toks[:17]), full[:17], atol=1e-12)
    # the fourth layer runs the second one's tensors: a model that spells them out agrees
    cfg2 = copy.deepcopy(cfg)
    del cfg2["layers"][3]["weights_of"]
    w2 = dict(w)
    for name in list(w):
        if name.startswith("l1."):
            w2["l3." + name[3:]] = w[name]
    assert torch.allclose(plain.forward(cfg2, w2, toks), full, atol=1e-12)
