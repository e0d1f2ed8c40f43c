"""RMSNorm fused with the residual add (the reference's norm: src/rmsnorm.py:20-28; its adds:
src/decoder_layer.py:49,54)."""
from __future__ import annotations

import torch

from ..ops import kernels
from .base import Norm, PendingNorm
from .registry import register_part


@register_part("norm", "rms")
class RMSNorm(Norm):
    """``out = v * rsqrt(mean(v^2) + eps) * weight`` with ``v = resid + delta``, in float32.
    ``weight_offset`` c: the stored weight lies around zero and the factor is ``c + weight``
    (added once, in float32, when the part is built).  ``scalar_weight``: the stored weight is one
    number for all coordinates (a tensor without dimensions), spread over the row when the part
    is built, so every kernel that takes a norm's weight vector takes this norm too."""

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        if params.get("scalar_weight", False):
            self.weight = self.expect("weight", ()).to(torch.float32).reshape(1).expand(self.size).contiguous()
        else:
            self.weight = self.expect("weight", (self.size,))
        offset = float(params.get("weight_offset", 0.0))
        if offset != 0.0:
            self.weight = (self.weight.to(torch.float32) + offset).contiguous()

    def forward(self, resid, delta, out, num_rows, rows=None, write_resid=True):
        kernels.add_rmsnorm(resid, delta, self.weight, self.eps, out, num_rows, rows, write_resid)
        return out

    def pending(self, resid, out, num_rows):
        return PendingNorm(self, resid, out, num_rows)


@register_part("norm", "layer_norm")
class LayerNorm(Norm):
    """Layer norm with a weight and no bias: ``out = (v - mean(v)) / sqrt(var(v) + eps) * weight``
    where ``var`` is the mean of the squared deviations, ``v = resid + delta``, in float32."""

    center = True

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = self.expect("weight", (self.size,))

    def forward(self, resid, delta, out, num_rows, rows=None, write_resid=True):
        kernels.norm_rows(resid, delta, self.weight, self.eps, True, out, num_rows, rows, write_resid)
        return out
