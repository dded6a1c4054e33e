"""Small Zolulix configurations for the tests, and model folders made from them.

The configurations differ from each other in every size and option: layer order (attention
first, recurrence first, two of a kind in a row), heads (1 to 5), key sizes (the recurrence's 16
lives in registers, 24 and 12 in shared memory), value sizes that are no multiple of anything,
latent widths that the tensor-core attention kernels take (48, 64) and do not take (24), windows
of 1, 9, 24, 40 and 150, a reader whose window is wider than its cache owner's, two readers of
one owner, rotated dimensions fewer than rot_dim, layers without a feed-forward, limits on both
sides of 1, inner sizes that are no multiple of 8."""
import json
from pathlib import Path

import torch


def latent(heads, dim, rot_dim, vdim, rank, window, base=10000.0, dims=None, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "mask": {"size": window},
         "rot": {"base": base, "dims": dims if dims is not None else rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(kind, mixer, ff=None, limit=1.0):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def recur(heads, dim, vdim, cap=10.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def model(vocab, width, layers, scale=4.0, eps=1e-5):
    return {"architecture": "Zolulix", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # attention first; a reader (layer 2) with a wider window than its owner; the recurrence with
    # its column in registers (16) and in shared memory (24), 71 columns = two blocks
    "P": model(301, 96, [
        layer("latent_attention", latent(4, 16, 8, 24, 40, window=24), ff=72, limit=0.7),
        layer("mlstm", recur(3, 16, 20, cap=8.0), ff=40, limit=1.5),
        layer("latent_attention", latent(4, 16, 8, 12, 40, window=40, kv_from=0)),
        layer("mlstm", recur(2, 24, 70), ff=72, limit=0.7),
        layer("latent_attention", latent(2, 8, 4, 10, 20, window=150, base=500.0, dims=2), ff=64, limit=2.0),
    ], scale=3.0),
    # recurrence first, one head everywhere, a window of one key, two readers of one owner, two
    # attention layers in a row, a latent width of 64
    "Q": model(200, 64, [
        layer("mlstm", recur(1, 12, 33, cap=15.0)),
        layer("latent_attention", latent(1, 24, 16, 40, 48, window=9, base=250000.0), ff=48, limit=1.0),
        layer("latent_attention", latent(5, 8, 16, 8, 48, window=1, base=250000.0, kv_from=1), ff=48, limit=0.5),
        layer("latent_attention", latent(3, 16, 16, 16, 48, window=9, base=250000.0, kv_from=1)),
        layer("mlstm", recur(4, 16, 16), ff=100, limit=3.0),
    ], scale=8.0, eps=1e-6),
}
INIT = dict(std=0.08, bias_std=0.5, norm_std=0.2)


def write_model(path, cfg, seed, edit=None):
    """A model folder with seeded random weights; `edit(tensors)` may change them (float32 in,
    stored as bfloat16).  Returns (config, float32 tensors as stored)."""
    import plain_model as pm
    from sonicboom_b200 import write_random_model
    from sonicboom_b200.weights.safetensors_io import write_safetensors
    path = Path(path)
    write_random_model(path, cfg, seed=seed, **INIT)
    _, tensors = pm.read_model_dir(path)
    # depth coefficients that sum to about one keep the stream's size from layer to layer
    for name in [n for n in tensors if n.endswith(".dwa")]:
        tensors[name] = tensors[name] / tensors[name].numel()
    if edit is not None:
        edit(tensors)
    stored = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    write_safetensors(path / "model.safetensors",
                      [(n, t.dtype, tuple(t.shape), (lambda t=t: t)) for n, t in stored.items()])
    (path / "config.json").write_text(json.dumps(cfg))
    return cfg, {n: t.float() for n, t in stored.items()}


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
