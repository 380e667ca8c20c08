"""Layer norm with weight and bias.

out = (x - mean) / sqrt(var + eps) * w + b, with var the mean of the squared
deviations; fp32 throughout. Parameters: eps, dim, the weight's tensor name
and the bias's (`bias`; None: no bias).

A sublayer whose output goes straight into `add_normed` does well to hand it
over in fp32 (its last product's accumulators, unrounded): the norm subtracts the
row's mean, and where the mean is large against the spread, a bfloat16 rounding
of the output would be magnified by that ratio.

It serves both placements: `apply` norms rows of the residual stream (a
model's last norm, or a pre-norm block), and `add_normed` norms a sublayer's
OUTPUT and adds it to the stream, x <- x + LN(y), for blocks that norm
behind the sublayer.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..ops import kernels
from .base import Norm, Residual, TensorSpec, register_norm


class LayerNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.eps = float(spec["eps"])
        self.dim = int(spec["dim"])
        self.name = str(spec["name"])
        self.bias_name: Optional[str] = spec.get("bias")
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.act_dtype = torch.float32

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [TensorSpec(self.name, (self.dim,), role="gain", init="gain", std=0.1)]
        if self.bias_name is not None:
            specs.append(TensorSpec(self.bias_name, (self.dim,), role="gain", init="normal", std=0.1))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.weight = tensors[self.name]
        self.bias = tensors[self.bias_name].to(self.weight.dtype) if self.bias_name is not None else None
        self.act_dtype = runtime.act_dtype

    def apply(self, stream: Residual, rows: Optional[torch.Tensor] = None, lazy: bool = False):
        x = stream.flush()
        return kernels.layernorm_rows(x, self.weight, self.bias, self.eps, self.act_dtype, rows=rows)

    def add_normed(self, stream: Residual, y: torch.Tensor, copy: bool = False) -> Optional[torch.Tensor]:
        """x <- x + LN(y); with `copy` also returns the new x in the activation type."""
        x = stream.flush()
        return kernels.layernorm_add(x, y, self.weight, self.bias, self.eps, copy=copy, copy_dtype=self.act_dtype)


register_norm("layernorm", LayerNorm)
