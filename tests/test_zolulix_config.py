"""Zolulix without a device: the configuration reader, the model as parts, the tensors it asks
for, random model folders, and the plain implementation on them."""
import copy
import json

import pytest
import torch

import plain_model as pm
import plain_zolulix as pz
from sonicboom_b200.config import ConfigError, ZolulixConfig, spec_from_config_dict
from sonicboom_b200.config.registry import architecture_name
from sonicboom_b200.models import tensor_requests
from zolulix_util import CONFIGS, tokens, write_model


@pytest.mark.parametrize("name", list(CONFIGS))
def test_configuration_round_trip_and_spec(name):
    cfg = CONFIGS[name]
    assert architecture_name(cfg) == "Zolulix"
    typed, spec = spec_from_config_dict(cfg)
    assert isinstance(typed, ZolulixConfig) and typed.to_dict() == cfg
    assert spec.vocab == cfg["vocab"] and spec.width == cfg["width"]
    assert spec.embedding_scale == cfg["embedding"]["scale"] and spec.head_tensor == "head"
    assert [e.cache_from for e in spec.schedule] == [l["mixer"].get("kv_from") for l in cfg["layers"]]
    for i, (l, s) in enumerate(zip(cfg["layers"], spec.layers)):
        assert s.arrangement == "sandwich_norm" and s.mixer.kind == l["type"]
        assert (s.feed_forward is None) == (l["mlp"] is None)
        assert s.depth_mix.n_inputs == i + 2 and s.depth_mix.tensor == f"l{i}.dwa"
        assert s.mixer_norm.kind == "rmsnorm_scalar" and s.mixer_norm.eps == cfg["norm"]["eps"]
        if l["mlp"] is not None:
            assert dict(s.feed_forward.params)["limit"] == l["mlp"]["limit"]
            assert s.feed_forward.intermediate == l["mlp"]["ff"]


def test_a_shared_cache_keeps_the_widest_window_of_its_users():
    _, spec = spec_from_config_dict(CONFIGS["P"])
    keep = [dict(l.mixer.params).get("keep") for l in spec.layers]
    assert keep[0] == keep[2] == 40 and keep[4] == 150          # layer 2 reads layer 0's cache with 40 keys
    assert [l.mixer.window for l in spec.layers if l.mixer.kind == "latent_attention"] == [24, 40, 150]
    assert [dict(l.mixer.params)["own_kv"] for l in spec.layers if l.mixer.kind == "latent_attention"] == \
        [True, False, True]


def test_tensor_names_and_shapes():
    cfg = CONFIGS["P"]
    _, spec = spec_from_config_dict(cfg)
    req = {r.name: tuple(r.shape) for r in tensor_requests(spec)}
    assert req["embed"] == (301, 96) and req["head"] == (301, 96) and req["final.norm"] == ()
    assert req["l0.norm1"] == req["l0.norm2b"] == ()
    assert req["l0.mix.q"] == (4 * 24, 96) and req["l0.mix.dkv"] == (48, 96) and req["l0.mix.dkv.norm"] == (40,)
    assert req["l0.mix.uk"] == (64, 40) and req["l0.mix.uv"] == (96, 40) and req["l0.mix.o"] == (96, 96)
    assert "l2.mix.dkv" not in req and "l2.mix.dkv.norm" not in req and req["l2.mix.uv"] == (48, 40)
    assert "l2.mlp.gate" not in req and "l2.norm2" not in req
    assert req["l1.mix.q"] == req["l1.mix.k"] == (48, 96) and req["l1.mix.v"] == req["l1.mix.g"] == (60, 96)
    assert req["l1.mix.i"] == (3, 96) and req["l1.mix.f.b"] == (3,) and req["l1.mix.norm"] == (60,)
    assert req["l1.mlp.gate"] == req["l1.mlp.up"] == (40, 96) and req["l1.mlp.down"] == (96, 40)
    assert [req[f"l{i}.dwa"] for i in range(5)] == [(i + 2,) for i in range(5)]


@pytest.mark.parametrize("change, message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="conv"), "layers[0].type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "layers[0].mixer.kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),       # layer 1 is no attention layer
    (lambda c: c["layers"][2]["mixer"].update(kv_from=4), "kv_from"),       # not an earlier layer
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=32), "kv_from"),      # the owner's rank differs
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0), "gate_cap"),
    (lambda c: c["layers"][1]["mlp"].update(kind="experts"), "mlp.kind"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "mlp.limit"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_a_bad_configuration_is_refused_by_key(change, message):
    cfg = copy.deepcopy(CONFIGS["P"])
    change(cfg)
    with pytest.raises(ConfigError) as e:
        spec_from_config_dict(cfg)
    assert message in str(e.value)


def test_an_unknown_architecture_is_named():
    with pytest.raises(ConfigError) as e:
        spec_from_config_dict({"architecture": "Nobody"})
    assert "Nobody" in str(e.value)


def test_random_folder_and_the_plain_implementation(tmp_path):
    cfg, tensors = write_model(tmp_path / "m", CONFIGS["Q"], seed=3)
    again_cfg, again = pm.read_model_dir(tmp_path / "m")
    assert again_cfg == cfg and set(again) == set(tensors)
    assert tensors["l0.norm1"].shape == () and tensors["l4.dwa"].shape == (6,)
    toks = tokens(cfg, 30, 1)
    streams = []
    logits = pz.forward(cfg, tensors, toks, streams)
    assert logits.shape == (30, cfg["vocab"]) and len(streams) == 5 and bool(torch.isfinite(logits).all())
    # causal: a position's logits do not depend on what follows it
    assert torch.allclose(pz.forward(cfg, tensors, toks[:17]), logits[:17], atol=1e-9)
    # a window of one key and windows of nine: the token ten places back cannot matter to layer 1
    # alone, but the recurrences carry everything, so the model as a whole does look back
    other = list(toks)
    other[0] = (other[0] + 1) % cfg["vocab"]
    assert not torch.allclose(pz.forward(cfg, tensors, other)[-1], logits[-1], atol=1e-9)
