"""Typed configuration of the Mefupel decoder, read from its own config.json keys.

A Mefupel model is a list of layers in which one RMS norm (weight stored as an offset from one)
feeds a mixer and a feed-forward side by side, x + mixer(norm(x)) + ff(norm(x)).  A stretch of the
layers may run several times in a row with the same weights; every pass has its own cache and
state, starts with a learned vector added to the stream, and every pass but the first also adds
the embedding output once more.  config.json gives every size and every constant that may differ
between models:

    architecture            "Mefupel"
    vocab, width            sizes of the embedding / head and of the residual stream
    norm.eps                eps of every RMS norm
    loop                    optional {start, stop, times}: layers start .. stop-1 run `times` times
    layers[i].type          "attention" | "gla" | "parallel"
    layers[i].mixer         that mixer's sizes and constants (below)
    layers[i].mlp           null, or {kind: "dense", ff}

    attention:  heads, kv_heads, dim, vdim, scale, mask.size, rot.base, rot.dims
    gla:        heads, dim, vdim, tau   (the rank of the decay's low-rank map is the shape of its
                first matrix; `decay_rank` may state it, and must when weights are made at random)
    parallel:   left  {heads, kv_heads, dim, vdim, scale, mask.size, rot.base, rot.dims}
                right {heads, dim, vdim, decay [heads], rot.base, rot.dims}

What the design fixes is written into the part records by `to_spec`: which layout of pairs each
mixer rotates in, values rotated by their own position in "attention", keys as values, the norm
over whole projections and the sink in "parallel"'s left side, the scalings of the recurrences'
queries and keys, the tensor names (`l<i>.norm1`, `l<i>.mix.q`, `l<i>.mlp.up`, `loop.step`, ...).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .specs import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                    ScheduleEntry, StreamInjection)
from .zolulix import MAX_POSITIONS, _num, _sub


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                # mask.size
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class GLAConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: Optional[int] = None


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class SideBySideConfig:
    left: WindowAttentionConfig
    right: RetentionConfig


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class MefupelLayer:
    type: str
    mixer: object
    mlp: Optional[DenseFFConfig]


def _rot(m: dict, where: str, dim: int):
    rot = _sub(m, "rot", where)
    base, dims = _num(rot, "base", where + "rot.", float), _num(rot, "dims", where + "rot.", positive=False)
    if dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"missing/invalid config key: {where}rot.dims ({dims} must be even and at most "
                          f"dim = {dim})")
    return base, dims


def _attention(m: dict, where: str) -> WindowAttentionConfig:
    dim = _num(m, "dim", where)
    base, dims = _rot(m, where, dim)
    a = WindowAttentionConfig(
        heads=_num(m, "heads", where), kv_heads=_num(m, "kv_heads", where), dim=dim, vdim=_num(m, "vdim", where),
        scale=_num(m, "scale", where, float), window=_num(_sub(m, "mask", where), "size", where + "mask."),
        rot_base=base, rot_dims=dims)
    if a.heads % a.kv_heads:
        raise ConfigError(f"missing/invalid config key: {where}kv_heads ({a.heads} query heads are not a "
                          f"multiple of {a.kv_heads})")
    return a


@dataclass(frozen=True)
class MefupelConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    loop: Optional[LoopConfig] = None
    architecture: str = "Mefupel"

    @classmethod
    def from_dict(cls, d: dict) -> "MefupelConfig":
        vocab, width = _num(d, "vocab", ""), _num(d, "width", "")
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
            if kind == "attention":
                mixer = _attention(m, mw)
                if mixer.vdim % 2:
                    raise ConfigError(f"missing/invalid config key: {mw}vdim ({mixer.vdim}: values rotate in "
                                      "pairs and need an even size)")
            elif kind == "gla":
                rank = m.get("decay_rank")
                mixer = GLAConfig(heads=_num(m, "heads", mw), dim=_num(m, "dim", mw), vdim=_num(m, "vdim", mw),
                                  tau=_num(m, "tau", mw, float),
                                  decay_rank=None if rank is None else _num(m, "decay_rank", mw))
            elif kind == "parallel":
                left = _attention(_sub(m, "left", mw), mw + "left.")
                if left.vdim != left.dim:
                    raise ConfigError(f"missing/invalid config key: {mw}left.vdim ({left.vdim}: the values "
                                      f"are the keys, so it must equal dim = {left.dim})")
                r, rw = _sub(m, "right", mw), mw + "right."
                dim = _num(r, "dim", rw)
                base, dims = _rot(r, rw, dim)
                decay = r.get("decay")
                heads = _num(r, "heads", rw)
                if not isinstance(decay, list) or len(decay) != heads or \
                        any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in decay):
                    raise ConfigError(f"missing/invalid config key: {rw}decay (a list of {heads} numbers, one "
                                      "per head)")
                mixer = SideBySideConfig(left, RetentionConfig(
                    heads=heads, dim=dim, vdim=_num(r, "vdim", rw), decay=tuple(float(x) for x in decay),
                    rot_base=base, rot_dims=dims))
            else:
                raise ConfigError(f"unsupported config key: {w}type = {kind!r} (attention, gla or parallel)")
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"unsupported config key: {w}mlp.kind = "
                                      f"{mlp.get('kind') if isinstance(mlp, dict) else mlp!r} (only 'dense')")
                mlp = DenseFFConfig(ff=_num(mlp, "ff", w + "mlp."))
            layers.append(MefupelLayer(kind, mixer, mlp))
        loop = d.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("missing/invalid config key: loop (expected an object)")
            loop = LoopConfig(start=_num(loop, "start", "loop.", positive=False),
                              stop=_num(loop, "stop", "loop.", positive=False), times=_num(loop, "times", "loop."))
            if not 0 <= loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"missing/invalid config key: loop ({loop.start} .. {loop.stop} is no "
                                  f"stretch of the {len(layers)} layers)")
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers), loop=loop)

    def to_dict(self) -> dict:
        """config.json content that `from_dict` reads back to an equal configuration."""
        def attention(a):
            return {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
                    "mask": {"size": a.window}, "rot": {"base": a.rot_base, "dims": a.rot_dims}}
        out = []
        for L in self.layers:
            m = L.mixer
            if L.type == "attention":
                mixer = attention(m)
            elif L.type == "gla":
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "tau": m.tau}
                if m.decay_rank is not None:
                    mixer["decay_rank"] = m.decay_rank
            else:
                r = m.right
                mixer = {"left": attention(m.left),
                         "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim, "decay": list(r.decay),
                                   "rot": {"base": r.rot_base, "dims": r.rot_dims}}}
            out.append({"type": L.type, "mixer": mixer,
                        "mlp": None if L.mlp is None else {"kind": "dense", "ff": L.mlp.ff}})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.eps}, "layers": out}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return d

    def run_order(self) -> list:
        """(layer, pass number or None) in run order; a number marks the first layer of a pass."""
        n, loop = len(self.layers), self.loop
        if loop is None or loop.start == loop.stop:
            return [(i, None) for i in range(n)]
        order = [(i, None) for i in range(loop.start)]
        for t in range(loop.times):
            order += [(i, t if i == loop.start else None) for i in range(loop.start, loop.stop)]
        return order + [(i, None) for i in range(loop.stop, n)]

    def to_spec(self) -> ModelSpec:
        """The model as parts: one block per layer in which mixer and feed-forward read the same
        norm; a layer inside the loop appears once per pass in the schedule (each run with a cache
        entry and state of its own), and every pass starts with an injection into the stream."""
        d, eps = self.width, self.eps

        def attention(a, prefix, layout, **more):
            return MixerSpec(
                kind="window_attention", width=d, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim,
                window=a.window, scale=a.scale,
                position=PositionSpec(kind=layout, head_dim=a.dim, theta=a.rot_base, rotary_dim=a.rot_dims),
                prefix=prefix, params=(("vdim", a.vdim), ("eps", eps)) + tuple(more.items()))

        layers = []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            m = L.mixer
            if L.type == "attention":
                mixer = attention(m, p + "mix.", "rope_interleaved", rotate_values=True)
            elif L.type == "gla":
                mixer = MixerSpec(
                    kind="linear_recurrence", width=d, n_heads=m.heads, head_dim=m.dim, prefix=p + "mix.",
                    params=(("vdim", m.vdim), ("decay", "low_rank"), ("tau", m.tau), ("decay_rank", m.decay_rank),
                            ("q_scale", float(m.dim) ** -0.5), ("norm_weight", "norm"), ("eps", eps)))
            else:
                left = attention(m.left, p + "mix.left.", "rope_halves", values="keys",
                                 qk_norm=("q.norm", "k.norm"), sink="sink")
                r = m.right
                right = MixerSpec(
                    kind="linear_recurrence", width=d, n_heads=r.heads, head_dim=r.dim, prefix=p + "mix.right.",
                    position=PositionSpec(kind="rope_halves", head_dim=r.dim, theta=r.rot_base,
                                          rotary_dim=r.rot_dims),
                    params=(("vdim", r.vdim), ("decay", "per_head"), ("head_decay", r.decay),
                            ("k_scale", float(r.dim) ** -0.5), ("eps", eps)))
                mixer = MixerSpec(kind="side_by_side", width=d, prefix=p + "mix.",
                                  params=(("left", left), ("right", right), ("left_out", "left.out"),
                                          ("right_out", "right.out"), ("eps", eps)))
            ff = None if L.mlp is None else FeedForwardSpec(
                kind="polynorm", width=d, intermediate=L.mlp.ff, activation="polynorm", prefix=p + "mlp.",
                params=(("eps", eps), ("names", ("up", "down", "act"))))
            layers.append(LayerSpec(arrangement="parallel_residual", mixer=mixer,
                                    mixer_norm=NormSpec("rmsnorm_one_plus", d, eps, p + "norm1"),
                                    feed_forward=ff, feed_forward_norm=None))
        order = self.run_order()
        times = self.loop.times if self.loop is not None else 0
        injections = tuple(StreamInjection(before_entry=e, embedding=t > 0, tensor="loop.step", rows=times, row=t)
                           for e, (_, t) in enumerate(order) if t is not None)
        spec = ModelSpec(
            architecture=self.architecture, width=d, vocab=self.vocab, max_positions=MAX_POSITIONS,
            embedding_tensor="embed", layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i, _ in order),
            final_norm=NormSpec("rmsnorm_one_plus", d, eps, "final.norm"), head_tensor="head",
            injections=injections,
            # a loop over no layers leaves its vectors in the file unused
            unused_tensors=(("loop.step", (times, d)),) if self.loop is not None and not injections else ())
        spec.validate()
        return spec
