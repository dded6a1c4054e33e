"""Two mixers on the same input, joined by their mean: with L and R the two results,

    y = (rms(L) * w_left + rms(R) * w_right) / 2,      rms(u) = u / sqrt(mean(u^2) + eps)

over the model width, with plain weights.  `params`: `left`, `right` (the two `MixerSpec`s, of
any registered kinds), `left_out`, `right_out` (tensor names of the two weights after the
prefix), `eps`.  At most one of the two may keep paged keys and values, and at most one
fixed-size state: a schedule entry owns one cache entry and one state row.

The halves of the weights are made at bind (halving is exact), so each side joins the stream
with the kernel that norms a sublayer's result and adds it (`ops.norm_add`)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorRequest
from .base import MIXERS, Mixer, make, register_mixer


@register_mixer("side_by_side")
class SideBySide(Mixer):
    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype = spec, dtype
        p = dict(spec.params)
        try:
            self.sides = [make(MIXERS, "mixer", p[k], dtype, device) for k in ("left", "right")]
            self.names = (p["left_out"], p["right_out"])
        except KeyError as e:
            raise ConfigError(f"side_by_side needs the parameter {e.args[0]}") from None
        self.eps = float(p.get("eps", 1e-6))
        if sum(s.kv_need() is not None for s in self.sides) > 1 or \
                sum(s.state_need() is not None for s in self.sides) > 1:
            raise ConfigError("side_by_side: both sides ask for the same kind of cache")
        self.half_weights = None

    def kv_need(self):
        return next((n for n in (s.kv_need() for s in self.sides) if n is not None), None)

    def state_need(self):
        return next((n for n in (s.state_need() for s in self.sides) if n is not None), None)

    def tensor_requests(self):
        p, d = self.spec.prefix, self.spec.width
        return [r for s in self.sides for r in s.tensor_requests()] + \
            [TensorRequest(p + n, (d,), "norm") for n in self.names]

    def bind(self, get):
        for s in self.sides:
            s.bind(get)
        self.half_weights = [(get(self.spec.prefix + n) * 0.5).contiguous() for n in self.names]

    def first_weights(self, rows):
        return self.sides[0].first_weights(rows)

    def forward(self, h, ctx, residual=None):
        x = residual if residual is not None else \
            torch.zeros((h.shape[0], self.spec.width), dtype=torch.float32, device=h.device)
        for side, w in zip(self.sides, self.half_weights):
            ctx.next_norm = ctx.next_weights = None        # a side's result is normed before it joins
            y = side.forward(h, ctx)
            ops.norm_add(y, x, w, self.eps, x)
        return x
