"""Typed configuration of the Zolulix decoder, read from its own config.json keys.

A Zolulix model is a list of layers, each with its own mixer (attention over a cached low-rank
latent, or the matrix-memory recurrence mLSTM), an optional clamped gated feed-forward, RMS
norms with one number each before and after every sublayer, and a learned weighted sum over the
embedding output and all layer results that feeds the next layer.  config.json gives every size
and every constant that may differ between models:

    architecture            "Zolulix"
    vocab, width            sizes of the embedding / head and of the residual stream
    embedding.scale         multiplies the embedding rows
    norm.eps                eps of every RMS norm
    layers[i].type          "latent_attention" | "mlstm"
    layers[i].mixer         that mixer's sizes and constants (below)
    layers[i].mlp           null, or {kind: "dense", ff, limit}

    latent_attention:  heads, dim, rot_dim, vdim, kv_rank, scale, mask.size, rot.base, rot.dims,
                       and optionally kv_from (the layer whose cache it reads)
    mlstm:             heads, dim, vdim, gate_cap

What the design fixes is written into the part records by `to_spec`: interleaved rotation pairs,
a softmax over a sliding window of mask.size keys, the sigmoid slope 1.702 of the feed-forward,
the tensor names (`l<i>.norm1`, `l<i>.mix.q`, `l<i>.mlp.gate`, `l<i>.dwa`, `final.norm`, `head`, ...).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .specs import (ConfigError, DepthMixSpec, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec,
                    NormSpec, PositionSpec, ScheduleEntry)

GLU_SLOPE = 1.702              # y = g sigmoid(1.702 g) (u + 1)
MAX_POSITIONS = 1 << 30        # the design names no longest sequence; the cache bounds it


def _sub(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"missing/invalid config key: {where}{key} (expected an object)")
    return v


def _num(d: dict, key: str, where: str, kind=int, positive=True):
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float) if kind is float else int):
        raise ConfigError(f"missing/invalid config key: {where}{key} (expected "
                          f"{'a number' if kind is float else 'an integer'}, got {v!r})")
    if positive and not v > 0:
        raise ConfigError(f"missing/invalid config key: {where}{key} (must be > 0, got {v!r})")
    return kind(v)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                   # unrotated query/key dimensions per head
    rot_dim: int               # rotated query/key dimensions per head (the key part is shared)
    vdim: int
    kv_rank: int
    scale: float
    window: int                # mask.size
    rot_base: float
    rot_dims: int              # how many of the rot_dim dimensions turn
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class MLSTMConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class ZolulixLayer:
    type: str
    mixer: object
    mlp: Optional[DenseFFConfig]


@dataclass(frozen=True)
class ZolulixConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: tuple
    architecture: str = "Zolulix"

    @classmethod
    def from_dict(cls, d: dict) -> "ZolulixConfig":
        vocab = _num(d, "vocab", "")
        width = _num(d, "width", "")
        scale = _num(_sub(d, "embedding", ""), "scale", "embedding.", float)
        eps = _num(_sub(d, "norm", ""), "eps", "norm.", float, positive=False)
        if eps < 0:
            raise ConfigError("missing/invalid config key: norm.eps (must be >= 0)")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("missing/invalid config key: layers (a non-empty list)")
        layers = []
        for i, L in enumerate(raw):
            w = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"missing/invalid config key: layers[{i}] (expected an object)")
            kind, m = L.get("type"), _sub(L, "mixer", w)
            mw = w + "mixer."
            if kind == "latent_attention":
                rot = _sub(m, "rot", mw)
                kv_from = m.get("kv_from")
                if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int)):
                    raise ConfigError(f"missing/invalid config key: {mw}kv_from (expected a layer index)")
                mixer = LatentAttentionConfig(
                    heads=_num(m, "heads", mw), dim=_num(m, "dim", mw), rot_dim=_num(m, "rot_dim", mw),
                    vdim=_num(m, "vdim", mw), kv_rank=_num(m, "kv_rank", mw),
                    scale=_num(m, "scale", mw, float), window=_num(_sub(m, "mask", mw), "size", mw + "mask."),
                    rot_base=_num(rot, "base", mw + "rot.", float), rot_dims=_num(rot, "dims", mw + "rot."),
                    kv_from=kv_from)
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"missing/invalid config key: {mw}rot.dims ({mixer.rot_dims} must be "
                                      f"even and at most rot_dim = {mixer.rot_dim})")
            elif kind == "mlstm":
                mixer = MLSTMConfig(heads=_num(m, "heads", mw), dim=_num(m, "dim", mw),
                                    vdim=_num(m, "vdim", mw), gate_cap=_num(m, "gate_cap", mw, float))
            else:
                raise ConfigError(f"unsupported config key: {w}type = {kind!r} "
                                  "(latent_attention or mlstm)")
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"unsupported config key: {w}mlp.kind = "
                                      f"{mlp.get('kind') if isinstance(mlp, dict) else mlp!r} (only 'dense')")
                mlp = DenseFFConfig(ff=_num(mlp, "ff", w + "mlp."), limit=_num(mlp, "limit", w + "mlp.", float))
            layers.append(ZolulixLayer(kind, mixer, mlp))
        for i, L in enumerate(layers):
            j = getattr(L.mixer, "kv_from", None)
            if j is None:
                continue
            w = f"layers[{i}].mixer.kv_from"
            if not 0 <= j < i:
                raise ConfigError(f"missing/invalid config key: {w} ({j} is not an earlier layer)")
            src = layers[j].mixer
            if not isinstance(src, LatentAttentionConfig) or src.kv_from is not None:
                raise ConfigError(f"missing/invalid config key: {w} (layer {j} has no latent cache of its own)")
            mine = L.mixer
            if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != \
                    (mine.kv_rank, mine.rot_dim, mine.rot_base, mine.rot_dims):
                raise ConfigError(f"missing/invalid config key: {w} (layer {j}'s kv_rank, rot_dim and "
                                  "rotation differ from this layer's)")
        return cls(vocab=vocab, width=width, embedding_scale=scale, eps=eps, layers=tuple(layers))

    def to_dict(self) -> dict:
        """config.json content that `from_dict` reads back to an equal configuration."""
        out = []
        for L in self.layers:
            m = L.mixer
            if L.type == "latent_attention":
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                         "kv_rank": m.kv_rank, "scale": m.scale, "mask": {"size": m.window},
                         "rot": {"base": m.rot_base, "dims": m.rot_dims}}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap}
            mlp = None if L.mlp is None else {"kind": "dense", "ff": L.mlp.ff, "limit": L.mlp.limit}
            out.append({"type": L.type, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": out}

    def to_spec(self) -> ModelSpec:
        """The model as parts: one sandwich-norm block per layer, each followed by the weighted
        sum over all streams so far; a `kv_from` layer reads the named layer's cache entry."""
        d, eps = self.width, self.eps
        layers, schedule = [], []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            m = L.mixer
            if L.type == "latent_attention":
                # the cache entry keeps what its owner and every reader of it may still look at
                owner = i if m.kv_from is None else m.kv_from
                keep = max([self.layers[owner].mixer.window] +
                           [o.mixer.window for o in self.layers if getattr(o.mixer, "kv_from", None) == owner])
                mixer = MixerSpec(
                    kind="latent_attention", width=d, n_heads=m.heads, n_kv_heads=1, head_dim=m.dim,
                    window=m.window, scale=m.scale,
                    position=PositionSpec(kind="rope_interleaved", head_dim=m.rot_dim, theta=m.rot_base,
                                          rotary_dim=m.rot_dims),
                    prefix=p + "mix.",
                    params=(("rot_dim", m.rot_dim), ("vdim", m.vdim), ("kv_rank", m.kv_rank), ("eps", eps),
                            ("keep", keep), ("own_kv", m.kv_from is None)))
                schedule.append(ScheduleEntry(i, m.kv_from))
            else:
                mixer = MixerSpec(kind="mlstm", width=d, n_heads=m.heads, head_dim=m.dim, prefix=p + "mix.",
                                  params=(("vdim", m.vdim), ("gate_cap", m.gate_cap), ("eps", eps)))
                schedule.append(ScheduleEntry(i))
            ff = None if L.mlp is None else FeedForwardSpec(
                kind="glu_clamped", width=d, intermediate=L.mlp.ff, activation="sigmoid", prefix=p + "mlp.",
                params=(("limit", L.mlp.limit), ("slope", GLU_SLOPE), ("names", ("gate", "up", "down"))))

            def norm(name):
                return NormSpec("rmsnorm_scalar", d, eps, p + name)
            layers.append(LayerSpec(
                arrangement="sandwich_norm", mixer=mixer, mixer_norm=norm("norm1"),
                mixer_post_norm=norm("norm1b"), feed_forward=ff,
                feed_forward_norm=norm("norm2") if ff is not None else None,
                feed_forward_post_norm=norm("norm2b") if ff is not None else None,
                depth_mix=DepthMixSpec("weighted_sum", i + 2, p + "dwa")))
        spec = ModelSpec(
            architecture=self.architecture, width=d, vocab=self.vocab, max_positions=MAX_POSITIONS,
            embedding_tensor="embed", layers=tuple(layers), schedule=tuple(schedule),
            final_norm=NormSpec("rmsnorm_scalar", d, eps, "final.norm"), head_tensor="head",
            embedding_scale=self.embedding_scale)
        spec.validate()
        return spec
