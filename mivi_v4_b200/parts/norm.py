"""Norms."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("norm", "rmsnorm")
class RMSNorm(Part):
    """y = x * (mean(x^2) + eps)^-1/2 * weight over the last dimension, in
    float32 (crates/mivi-core/src/simd/norm.rs:38-72; math.rs:14-29).  ``one_plus``: the checkpoint stores the
    weight around zero and the factor is 1 + weight (added once, in float32, when the weights are loaded)."""

    def __init__(self, dim: int, eps: float, one_plus: bool = False):
        self.dim, self.eps, self.one_plus = int(dim), float(eps), bool(one_plus)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.dim,), "vector", "bias" if self.one_plus else "norm")}

    def load(self, t) -> None:
        self.weight = (t["weight"].float() + 1.0).contiguous() if self.one_plus else t["weight"]

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return K.rmsnorm(x, self.weight, self.eps, out, rows)

    def link(self, step, name: str) -> K.NormLink:
        """This norm as something the products around it carry (steps of few tokens): buffers for
        the rows bf16(x * weight) and the tile sums of squares, from the step's workspace."""
        n = step.n_tokens
        return K.NormLink(self, self.weight, self.eps, self.dim,
                          step.ws.get("link_rows_" + name, (n, self.dim), torch.bfloat16),
                          step.ws.get("link_sums_" + name, (n, -(-self.dim // 64) * 4), torch.float32))


@register("norm", "layernorm")
class LayerNorm(Part):
    """y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * weight (+ bias, with ``bias``) over the last
    dimension, in float32.  It is not carried by the products around it (it has no ``link``): it always runs as
    a kernel."""

    def __init__(self, dim: int, eps: float, bias: bool = False):
        self.dim, self.eps, self.has_bias = int(dim), float(eps), bool(bias)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"weight": ParamSpec((self.dim,), "vector", "norm")}
        if self.has_bias:
            specs["bias"] = ParamSpec((self.dim,), "vector", "bias")
        return specs

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return K.layernorm(x, self.weight, self.eps, out, rows, bias=self.bias)
