"""RMSNorm over rows of the fp32 residual stream.

y = (x * 1/sqrt(mean(x^2) + eps)) * w, weight used as it is
(src/kernels/transformer/norm.zig:4-37).  ``scalar``: the checkpoint holds one gain for the whole
row (a tensor without dimensions) instead of a weight per coordinate.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_norm
from .base import Norm, ParamSpec


@register_norm("rms_norm")
class RMSNorm(Norm):
    reads_stream_by_kernel = True

    def __init__(self, size: int, eps: float, scalar: bool = False):
        self.size = int(size)
        self.eps = float(eps)
        self.scalar = bool(scalar)
        self.weight: Optional[torch.Tensor] = None
        self.gain: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec(() if self.scalar else (self.size,), kind="vector", init="one_plus_normal")}

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        self.weight = params["weight"]
        if self.scalar:
            # the kernels (and the products that fold a norm in) read a weight per coordinate: the one
            # gain, widened to 32 bits (exact), repeated along the row
            self.gain = self.weight
            self.weight = self.gain.float().reshape(1).expand(self.size).contiguous()

    def tensors(self) -> Dict[str, torch.Tensor]:
        return {"weight": self.gain if self.scalar else self.weight}

    def forward(self, out: torch.Tensor, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        self.rt.k.rmsnorm(out, x, self.weight, self.eps, rows)


@register_norm("none")
class NoNorm(Norm):
    """Stands where a layer has nothing to norm (a layer without a feed-forward): no tensors, never run."""

    def __init__(self, size: int):
        self.size = int(size)

    def forward(self, out: torch.Tensor, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        raise RuntimeError("a 'none' norm stands for a part that does not exist and is never run")
