"""Depth mixing: what a layer hands on is a combination of the embedding output and every block
result so far, not its own result alone.

"weighted_sum": with X_0 the embedding output and X_(j+1) the result of schedule entry j, entry
i hands on  sum over j = 0 .. i+1 of w[j] X_j  with its own learned coefficients w [i + 2].  The
model keeps the X_j of a step side by side (`[entries + 1, rows, width]` float32) and calls
`forward` after each block; the sum runs in ascending j in float32, and the first norm of the
entry that runs next can be written with it."""
from __future__ import annotations

from .. import ops
from ..weights.loader import TensorRequest
from .base import DEPTH_MIXES, Part, register_depth_mix


@register_depth_mix("weighted_sum")
class WeightedDepthSum(Part):
    def __init__(self, spec, dtype, device):
        self.spec, self.coef = spec, None

    def tensor_requests(self):
        return [TensorRequest(self.spec.tensor, (self.spec.n_inputs,), "norm")]

    def bind(self, get):
        self.coef = get(self.spec.tensor)

    def joins(self, weight) -> bool:
        """Whether `forward` can also make the last stream from a block's last sublayer result
        (`join`): the kernel reads the norm's weight as it reads the coefficients."""
        return weight.dtype == self.coef.dtype

    def forward(self, streams, out, next_norm=None, join=None):
        """out = sum_j coef[j] * streams[j] over the first n_inputs streams.  `join` = (y, x,
        weight, eps): the last stream is x + norm(y) * weight and is written first."""
        return ops.depth_mix(streams, self.spec.n_inputs, self.coef, out, next_norm, join)
