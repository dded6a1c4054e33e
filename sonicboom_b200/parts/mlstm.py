"""The matrix-memory recurrence of xLSTM (mLSTM) as a mixer.

Per head, with q = Wq h / sqrt(dim), k = Wk h (dim each), v = Wv h (vdim), the log input gate
i = cap tanh((Wi h + bi) / cap) and the log forget gate f = logsigmoid(cap tanh((Wf h + bf) / cap)):
    m_t = max(f + m_{t-1}, i),   S_t = exp(f + m_{t-1} - m_t) S_{t-1} + exp(i - m_t) k v^T,
    n_t likewise with k alone,   o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6),
S, n and m starting at zero.  Each head's o is divided by its root mean square (eps), the heads
are concatenated, multiplied by a weight over all heads' values and by sigmoid(Wg h), and
projected by Wo.

The six input projections are one product over [q | k | v | g | i | f] rows whose float32 result
feeds the recurrence kernel directly; the state (S with n as one more column, stored column by
column with a copy of m after each: float32 [heads, vdim + 1, dim + 1 rounded up to 4]) is fixed-size per-sequence state of the cache
(`StateNeed`), zeroed when a slot is taken and carried from step to step.

Tensors after the prefix: q, k [heads*dim, width]; v, g [heads*vdim, width]; i, f [heads, width];
i.b, f.b [heads]; norm [heads*vdim]; o [width, heads*vdim].
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.kv import StateNeed
from ..weights.loader import TensorRequest
from .base import Mixer, register_mixer


@register_mixer("mlstm")
class MLSTM(Mixer):
    def __init__(self, spec, dtype, device):
        from ..config.specs import ConfigError
        self.spec, self.dtype, self.device = spec, dtype, device
        p = dict(spec.params)
        self.h, self.dim = spec.n_heads, spec.head_dim
        try:
            self.vd, self.cap = int(p["vdim"]), float(p["gate_cap"])
        except KeyError as e:
            raise ConfigError(f"mlstm needs the parameter {e.args[0]}") from None
        if not self.cap > 0.0:
            raise ConfigError(f"mlstm gate_cap {self.cap} must be positive")
        self.eps = float(p.get("eps", 1e-6))
        self.q_scale = float(self.dim) ** -0.5
        self.w_in = self.b_i = self.b_f = self.norm_w = self.w_o = None

    def state_need(self):
        return StateNeed((self.h, self.vd + 1, (self.dim + 4) // 4 * 4), torch.float32)      # columns in 16-byte steps

    def tensor_requests(self):
        p, d, h = self.spec.prefix, self.spec.width, self.h
        return [TensorRequest(p + "q", (h * self.dim, d)), TensorRequest(p + "k", (h * self.dim, d)),
                TensorRequest(p + "v", (h * self.vd, d)), TensorRequest(p + "g", (h * self.vd, d)),
                TensorRequest(p + "i", (h, d)), TensorRequest(p + "f", (h, d)),
                TensorRequest(p + "i.b", (h,), "bias"), TensorRequest(p + "f.b", (h,), "bias"),
                TensorRequest(p + "norm", (h * self.vd,), "norm"),
                TensorRequest(p + "o", (d, h * self.vd))]

    def bind(self, get):
        p = self.spec.prefix
        ws = [get(p + n) for n in ("q", "k", "v", "g", "i", "f")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        self.b_i, self.b_f = get(p + "i.b"), get(p + "f.b")
        if self.b_i.dtype != self.b_f.dtype:
            self.b_i, self.b_f = self.b_i.float(), self.b_f.float()
        self.norm_w = get(p + "norm")
        self.w_o = get(p + "o")

    def forward(self, h, ctx, residual=None):
        rows = h.shape[0]
        proj = torch.empty((rows, self.w_in.shape[0]), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_in, proj)
        num = torch.empty((rows, self.h, self.vd + 1), dtype=torch.float32, device=h.device)
        m_row = torch.empty((rows, self.h), dtype=torch.float32, device=h.device)
        ops.mlstm_scan(proj, ctx.plan, self.h, self.dim, self.vd, self.b_i, self.b_f, self.cap,
                       self.q_scale, ctx.state(), num, m_row)
        mixed = torch.empty((rows, self.h * self.vd), dtype=self.dtype, device=h.device)
        ops.mlstm_out(num, m_row, proj, self.h, self.dim, self.vd, self.norm_w, self.eps, mixed)
        out = residual if residual is not None else \
            torch.empty((rows, self.spec.width), dtype=torch.float32, device=h.device)
        return ctx.linear(mixed, self.w_o, out, ops.EPI_RESIDUAL if residual is not None else ops.EPI_NONE,
                          residual=residual, act_dtype=self.dtype)
