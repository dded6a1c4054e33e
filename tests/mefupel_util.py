"""Small Mefupel configurations for the tests, and model folders made from them.

The configurations differ from each other in every size and option: layer order, a loop over two
layers run three times and a "loop" that runs one layer once, no loop at all, query groups of 1,
2 and 4, key sizes that are and are not multiples of 16, value sizes smaller and larger than the
key size, rotated prefixes shorter than a head and whole heads, windows of 1, 9, 20, 70 and 150,
recurrences with one head and with several, decays near and far from one, layers without a
feed-forward, inner sizes that are no multiple of 8."""
import json
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, window, dims=None, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": scale if scale is not None else dim ** -0.5, "mask": {"size": window},
            "rot": {"base": base, "dims": dim if dims is None else dims}}


def gla(heads, dim, vdim, tau=8.0, rank=4):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}


def retention(heads, dim, vdim, decay, dims=None, base=10000.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
            "rot": {"base": base, "dims": dim if dims is None else dims}}


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model(vocab, width, layers, loop=None, eps=1e-5):
    d = {"architecture": "Mefupel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


CONFIGS = {
    # a loop over the middle two layers, run three times; values wider than keys; a rotated prefix
    "A": model(211, 64, [
        layer("attention", attention(4, 2, 16, 24, window=9, dims=8, scale=0.3), ff=40),
        layer("gla", gla(2, 16, 12, tau=8.0, rank=4), ff=72),
        layer("parallel", {"left": attention(4, 1, 32, 32, window=20, dims=16, scale=0.2),
                           "right": retention(3, 16, 8, [0.9, 0.95, 0.999], dims=8)}),
        layer("attention", attention(2, 2, 8, 8, window=150, base=500.0), ff=24),
    ], loop=(1, 3, 3)),
    # the side-by-side layer first and looped once; one recurrence head; key sizes 24 and 40; a
    # window of one key; an inner size that is no multiple of 8; head size 64 and 128 kernels
    "B": model(150, 96, [
        layer("parallel", {"left": attention(2, 2, 64, 64, window=70, base=300000.0),
                           "right": retention(1, 24, 40, [0.97], base=2e6)}, ff=50),
        layer("gla", gla(3, 40, 33, tau=1.0, rank=8)),
        layer("attention", attention(6, 3, 128, 64, window=1, dims=2, base=100.0), ff=64),
        layer("gla", gla(1, 16, 16, tau=30.0, rank=2), ff=16),
    ], loop=(0, 1, 1), eps=1e-6),
}
INIT = dict(std=0.08, bias_std=0.3, norm_std=0.2)


def write_model(path, cfg, seed, edit=None, drop_rank=False):
    """A model folder with seeded random weights; `edit(tensors)` may change them (float32 in,
    stored as bfloat16).  With `drop_rank` config.json does not state the rank of a decay's
    low-rank map.  Returns (config as written, float32 tensors as stored)."""
    import plain_model as pm
    from sonicboom_b200 import write_random_model
    from sonicboom_b200.weights.safetensors_io import write_safetensors
    path = Path(path)
    write_random_model(path, cfg, seed=seed, **INIT)
    _, tensors = pm.read_model_dir(path)
    for name in [n for n in tensors if n.endswith(".sink")]:
        tensors[name] = tensors[name] * 5.0           # sinks that weigh as much as a few keys
    if edit is not None:
        edit(tensors)
    stored = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    write_safetensors(path / "model.safetensors",
                      [(n, t.dtype, tuple(t.shape), (lambda t=t: t)) for n, t in stored.items()])
    if drop_rank:
        cfg = json.loads(json.dumps(cfg))
        for L in cfg["layers"]:
            L["mixer"].pop("decay_rank", None)
    (path / "config.json").write_text(json.dumps(cfg))
    return cfg, {n: t.float() for n, t in stored.items()}


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
