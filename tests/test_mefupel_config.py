"""Mefupel without a device: configuration keys and their errors, the schedule a loop makes, the
tensors a model asks for, and properties of the plain implementation's mechanisms."""
import json

import pytest
import torch

import plain_mefupel as pf
from mefupel_util import CONFIGS, attention, gla, layer, model, retention
from sonicboom_b200.config import ConfigError, MefupelConfig, spec_from_config_dict
from sonicboom_b200.models import tensor_requests


def test_round_trip_and_registry():
    for cfg in CONFIGS.values():
        c, spec = spec_from_config_dict(cfg)
        assert isinstance(c, MefupelConfig) and MefupelConfig.from_dict(c.to_dict()) == c
        assert spec.architecture == "Mefupel" and spec.vocab == cfg["vocab"]


def test_a_loop_repeats_its_layers_with_an_injection_before_every_pass():
    c, spec = spec_from_config_dict(CONFIGS["A"])
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [(i.before_entry, i.embedding, i.row) for i in spec.injections] == [(1, False, 0), (3, True, 1), (5, True, 2)]
    assert [(l, t) for l, t in pf.layer_order(CONFIGS["A"])] == c.run_order()
    _, once = spec_from_config_dict(CONFIGS["B"])
    assert [e.layer for e in once.schedule] == [0, 1, 2, 3]
    assert [(i.before_entry, i.embedding, i.row, i.rows) for i in once.injections] == [(0, False, 0, 1)]
    plain = json.loads(json.dumps(CONFIGS["B"]))
    del plain["loop"]
    _, none = spec_from_config_dict(plain)
    assert none.injections == () and "loop.step" not in {r.name for r in tensor_requests(none)}
    empty = dict(plain, loop={"start": 2, "stop": 2, "times": 4})
    _, spec = spec_from_config_dict(empty)
    assert spec.injections == () and [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    assert {r.name: r.optional for r in tensor_requests(spec)}["loop.step"] is True


def test_tensor_names_and_shapes():
    _, spec = spec_from_config_dict(CONFIGS["A"])
    req = {r.name: tuple(r.shape) for r in tensor_requests(spec)}
    assert req["embed"] == (211, 64) and req["head"] == (211, 64) and req["loop.step"] == (3, 64)
    assert req["l0.mix.q"] == (64, 64) and req["l0.mix.k"] == (32, 64) and req["l0.mix.v"] == (48, 64)
    assert req["l0.mix.o"] == (64, 96) and req["l0.mlp.up"] == (40, 64) and req["l0.mlp.act"] == (4,)
    assert req["l1.mix.a1"] == (4, 64) and req["l1.mix.a2"] == (32, 4) and req["l1.mix.a2.b"] == (32,)
    assert req["l1.mix.norm"] == (12,) and req["l1.mix.g"] == (24, 64)
    assert req["l2.mix.left.q.norm"] == (128,) and req["l2.mix.left.k.norm"] == (32,) and req["l2.mix.left.sink"] == (4,)
    assert "l2.mix.left.v" not in req and req["l2.mix.left.o"] == (64, 128)
    assert req["l2.mix.right.o"] == (64, 24) and req["l2.mix.left.out"] == (64,) and req["l2.mix.right.out"] == (64,)
    assert not any(n.startswith("l2.mlp.") for n in req) and "l2.mix.right.norm" not in req
    # without a stated rank the two low-rank matrices are asked for with that size left open
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    del cfg["layers"][1]["mixer"]["decay_rank"]
    req = {r.name: tuple(r.shape) for r in tensor_requests(spec_from_config_dict(cfg)[1])}
    assert req["l1.mix.a1"] == (-1, 64) and req["l1.mix.a2"] == (32, -1)


@pytest.mark.parametrize("path,value,match", [
    (("layers", 0, "type"), "conv", r"layers\[0\].type"),
    (("layers", 0, "mixer", "kv_heads"), 3, r"layers\[0\].mixer.kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, r"layers\[0\].mixer.rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 18, r"layers\[0\].mixer.rot.dims"),
    (("layers", 0, "mixer", "vdim"), 23, r"layers\[0\].mixer.vdim"),
    (("layers", 0, "mixer", "mask"), None, r"layers\[0\].mixer.mask"),
    (("layers", 1, "mixer", "tau"), 0, r"layers\[1\].mixer.tau"),
    (("layers", 2, "mixer", "left", "vdim"), 16, r"layers\[2\].mixer.left.vdim"),
    (("layers", 2, "mixer", "right", "decay"), [0.5], r"layers\[2\].mixer.right.decay"),
    (("layers", 2, "mixer", "right"), None, r"layers\[2\].mixer.right"),
    (("layers", 0, "mlp", "kind"), "moe", r"layers\[0\].mlp.kind"),
    (("loop", "stop"), 9, "loop"),
    (("loop", "times"), 0, "loop.times"),
    (("norm", "eps"), -1.0, "norm.eps"),
    (("width",), "wide", "width"),
])
def test_errors_name_the_key(path, value, match):
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    at = cfg
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=match):
        spec_from_config_dict(cfg)


def test_random_weights_need_a_stated_rank():
    from sonicboom_b200.weights import RandomSource
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    del cfg["layers"][1]["mixer"]["decay_rank"]
    with pytest.raises(ValueError, match="l1.mix.a1"):
        RandomSource(tensor_requests(spec_from_config_dict(cfg)[1]), 1)


# ------------------------------------------------------------------ the plain implementation itself
def test_rotations_keep_lengths_and_undo_each_other():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 3, 12, generator=g, dtype=torch.float64)
    pos = torch.arange(7) + 100
    for layout in ("interleaved", "halves"):
        y = pf.rotate(x, pos, 1000.0, 8, layout)
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1)) and torch.equal(y[..., 8:], x[..., 8:])
        assert torch.allclose(pf.rotate(y, pos, 1000.0, 8, layout, sign=-1.0), x)
    a = pf.rotate(x, pos, 1000.0, 12, "interleaved")
    b = pf.rotate(x[..., [0, 2, 4, 6, 8, 10, 1, 3, 5, 7, 9, 11]], pos, 1000.0, 12, "halves")
    assert torch.allclose(a[..., 0::2], b[..., :6]) and torch.allclose(a[..., 1::2], b[..., 6:])


def test_a_sink_only_shrinks_the_weights():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(9, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    plain = pf.windowed_softmax_attention(q, k, v, 0.5, 4)
    low = pf.windowed_softmax_attention(q, k, v, 0.5, 4, sink=torch.tensor([-50.0, -50.0], dtype=torch.float64))
    assert torch.allclose(plain, low)
    s = torch.tensor([0.3, 2.0], dtype=torch.float64)
    with_sink = pf.windowed_softmax_attention(q, k, v, 0.5, 4, sink=s)
    # position 0 sees one key with score s0: its weight is e^s0 / (e^s0 + e^sink)
    for h in range(2):
        s0 = (q[0, h] @ k[0, h]) * 0.5
        assert torch.allclose(with_sink[0, h], v[0, h] * torch.exp(s0) / (torch.exp(s0) + torch.exp(s[h])))


def test_rotated_values_depend_on_distance_only():
    """Turning the values by their position and the sum back by the query's is the same as turning
    each value by the distance to the query."""
    g = torch.Generator().manual_seed(2)
    T, dv = 6, 8
    w = torch.softmax(torch.randn(T, generator=g, dtype=torch.float64), 0)
    v = torch.randn(T, 1, dv, generator=g, dtype=torch.float64)
    pos = torch.arange(T)
    i = T - 1
    summed = (w[:, None, None] * pf.rotate(v, pos, 100.0, dv, "interleaved")).sum(0, keepdim=True)
    back = pf.rotate(summed, torch.tensor([i]), 100.0, dv, "interleaved", sign=-1.0)
    direct = (w[:, None, None] * pf.rotate(v, pos - i, 100.0, dv, "interleaved")).sum(0, keepdim=True)
    assert torch.allclose(back, direct)


def test_recurrence_equals_the_sum_it_unrolls_to():
    g = torch.Generator().manual_seed(3)
    T, H, d, dv = 8, 2, 3, 5
    q, k = (torch.randn(T, H, d, generator=g, dtype=torch.float64) for _ in range(2))
    v = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
    a = torch.rand(T, H, d, generator=g, dtype=torch.float64)
    o = pf.linear_recurrence(q, k, v, a)
    for h in range(H):
        t = T - 1
        want = torch.zeros(dv, dtype=torch.float64)
        for j in range(t + 1):
            decay = a[j + 1:t + 1, h].prod(0)
            want += ((q[t, h] * decay * k[j, h]).sum()) * v[j, h]
        assert torch.allclose(o[t, h], want)


def test_polynorm_is_scale_free_in_its_input():
    g = torch.Generator().manual_seed(4)
    h = torch.randn(3, 6, generator=g, dtype=torch.float64)
    W = {"up": torch.randn(10, 6, generator=g, dtype=torch.float64),
         "down": torch.eye(10, dtype=torch.float64), "act": torch.tensor([0.5, -1.0, 2.0, 0.25], dtype=torch.float64)}
    a = pf.polynorm_ff(h, W, "", 0.0)
    b = pf.polynorm_ff(3.0 * h, W, "", 0.0)
    assert torch.allclose(a, b)


def test_random_model_folder_reads_back(tmp_path):
    """`write_random_model` on a Mefupel configuration: every requested tensor with its shape, the
    same bits for the same seed, and the plain implementation runs on the folder."""
    import plain_model as pm
    from sonicboom_b200 import write_random_model
    cfg = CONFIGS["A"]
    write_random_model(tmp_path / "a", cfg, seed=4, std=0.05, bias_std=0.1, norm_std=0.1)
    write_random_model(tmp_path / "b", cfg, seed=4, std=0.05, bias_std=0.1, norm_std=0.1)
    _, ta = pm.read_model_dir(tmp_path / "a")
    _, tb = pm.read_model_dir(tmp_path / "b")
    want = {r.name: tuple(r.shape) for r in tensor_requests(spec_from_config_dict(cfg)[1])}
    assert {n: tuple(t.shape) for n, t in ta.items()} == want
    assert all(torch.equal(ta[n], tb[n]) for n in ta)
    logits = pf.forward(cfg, ta, [1, 2, 3, 4, 5])
    assert tuple(logits.shape) == (5, cfg["vocab"]) and bool(torch.isfinite(logits).all())
