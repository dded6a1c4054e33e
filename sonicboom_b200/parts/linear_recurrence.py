"""Linear attention as a recurrence over a matrix state, the mixer of gated linear attention and
of retention:

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t          per head, S_0 = 0,

with q, k of `head_dim` and v of `vdim` values per head.  `decay` chooses a_t:
  "low_rank"  one decay per key channel and token, a = sigmoid(z)^(1/tau) with z = A2 (A1 h) + b
              (tensors a1 [rank, width], a2 [heads*head_dim, rank], a2.b; `tau`; the rank is
              `decay_rank`, or whatever the stored a1 has when that is None);
  "per_head"  one fixed decay per head, `head_decay` (a tuple of numbers).
`q_scale` / `k_scale` multiply q and k (after the rotation, when the spec has a position
encoding: a prefix of every q and k head turns by the token's position).  Every head's o is
divided by its root mean square (`eps`) and, with `norm_weight` = a tensor name, multiplied by
that weight [vdim], which all heads share; the heads are concatenated, multiplied by silu(G h)
and projected by O.

q, k, v, g and the first half of the decay map are one product; the map's second half, the
decays, the rotation, the state and the recurrence are float32 whatever the activation dtype.  The state (float32 [heads, vdim, head_dim]) is fixed-size
per-sequence state of the cache, zeroed when a slot is taken and carried from step to step; the
recurrence runs token by token for prompts, portions and single tokens alike.

Tensors after the prefix: q, k [heads*head_dim, width]; v, g [heads*vdim, width]; o [width,
heads*vdim]; and what `decay` and `norm_weight` name."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.kv import StateNeed
from ..weights.loader import TensorRequest
from .attention import _cat
from .base import POSITION_ENCODINGS, Mixer, make, register_mixer


@register_mixer("linear_recurrence")
class LinearRecurrence(Mixer):
    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype, self.device = spec, dtype, device
        p = dict(spec.params)
        self.h, self.dim = spec.n_heads, spec.head_dim
        self.vd = int(p.get("vdim", self.dim))
        self.eps = float(p.get("eps", 1e-6))
        self.q_scale, self.k_scale = float(p.get("q_scale", 1.0)), float(p.get("k_scale", 1.0))
        self.decay = p.get("decay")
        self.norm_name = p.get("norm_weight")
        self.head_decay = None
        if self.decay == "low_rank":
            self.tau, self.rank = float(p.get("tau", 1.0)), p.get("decay_rank")
            if not self.tau > 0.0:
                raise ConfigError(f"linear_recurrence tau {self.tau} must be positive")
        elif self.decay == "per_head":
            values = tuple(p.get("head_decay", ()))
            if len(values) != self.h:
                raise ConfigError(f"linear_recurrence head_decay has {len(values)} values for {self.h} heads")
            self.head_decay = torch.tensor(values, dtype=torch.float64).to(torch.float32).to(device)
        else:
            raise ConfigError(f"linear_recurrence decay {self.decay!r} (low_rank or per_head)")
        self.rot, self.interleaved, self.inv_freq = 0, False, None
        if spec.position is not None and spec.position.rotary_dim > 0:
            pe = make(POSITION_ENCODINGS, "position encoding", spec.position, dtype, device)
            self.interleaved = getattr(pe, "layout", "halves") == "interleaved"
            self.rot, self.inv_freq = spec.position.rotary_dim, pe.inv_freq
        self.k_off, self.v_off = self.h * self.dim, 2 * self.h * self.dim
        self.g_off = self.v_off + self.h * self.vd
        self.w_in = self.w_a2 = self.b_a2 = self.norm_w = self.w_o = None
        self.a1_off = 0

    def state_need(self):
        return StateNeed((self.h, self.vd, self.dim), torch.float32)

    def tensor_requests(self):
        p, d, h = self.spec.prefix, self.spec.width, self.h
        req = [TensorRequest(p + "q", (h * self.dim, d)), TensorRequest(p + "k", (h * self.dim, d)),
               TensorRequest(p + "v", (h * self.vd, d)), TensorRequest(p + "g", (h * self.vd, d)),
               TensorRequest(p + "o", (d, h * self.vd))]
        if self.decay == "low_rank":
            r = -1 if self.rank is None else int(self.rank)      # -1: whatever the stored tensors have
            req += [TensorRequest(p + "a1", (r, d)), TensorRequest(p + "a2", (h * self.dim, r)),
                    TensorRequest(p + "a2.b", (h * self.dim,), "bias")]
        if self.norm_name:
            req.append(TensorRequest(p + self.norm_name, (self.vd,), "norm"))
        return req

    def bind(self, get):
        from ..config.specs import ConfigError
        p = self.spec.prefix
        parts = [get(p + n) for n in ("q", "k", "v", "g")]
        self.w_o = get(p + "o")
        if self.decay == "low_rank":
            w_a1, self.w_a2, self.b_a2 = get(p + "a1"), get(p + "a2"), get(p + "a2.b")
            if w_a1.shape[0] != self.w_a2.shape[1]:
                raise ConfigError(f"{p}a1 has {w_a1.shape[0]} rows, {p}a2 {self.w_a2.shape[1]} columns")
            if self.w_a2.dtype != self.b_a2.dtype:
                self.w_a2, self.b_a2 = self.w_a2.float(), self.b_a2.float()
            parts.append(w_a1)                       # the map's first half rides on the projection
            self.a1_off = self.g_off + self.h * self.vd
        self.w_in = _cat(parts)
        if self.norm_name:
            self.norm_w = get(p + self.norm_name)

    def forward(self, h, ctx, residual=None):
        rows, plan = h.shape[0], ctx.plan
        proj = torch.empty((rows, self.w_in.shape[0]), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_in, proj)
        z = None
        if self.decay == "low_rank":
            z = torch.empty((rows, self.h * self.dim), dtype=torch.float32, device=h.device)
            ops.linrec_prep(proj, 0, self.k_off, self.h, self.dim, self.q_scale, self.k_scale, self.rot,
                            self.interleaved, self.inv_freq, plan.row_pos, z, 1.0 / self.tau,
                            low_rank=(self.w_a2, self.b_a2, self.a1_off))
        elif self.rot > 0 or self.q_scale != 1.0 or self.k_scale != 1.0:
            ops.linrec_prep(proj, 0, self.k_off, self.h, self.dim, self.q_scale, self.k_scale, self.rot,
                            self.interleaved, self.inv_freq, plan.row_pos)
        o = torch.empty((rows, self.h, self.vd), dtype=torch.float32, device=h.device)
        ops.linrec_scan(proj, 0, self.k_off, self.v_off, plan, self.h, self.dim, self.vd, z, self.head_decay,
                        ctx.state(), o)
        mixed = torch.empty((rows, self.h * self.vd), dtype=self.dtype, device=h.device)
        ops.linrec_out(o, proj, self.g_off, self.h, self.vd, self.norm_w, self.eps, mixed)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(mixed, self.w_o, out, ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)
