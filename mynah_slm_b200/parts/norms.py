"""RMSNorm with a plain gain, or with a gain stored around zero.

out = x * (1 / sqrt(mean(x^2) + eps)) * w, the reference's form (mynah-slm
src/kernels.c:118-128); the gain multiplies as it is, it is not 1 + w
(src/kernels.h:29-33: a (1+w) norm is a different function, not a flag of
this one). That other function is here as a part of its own kind,
`rmsnorm_offset`: out = x / sqrt(mean(x^2) + eps) * (1 + w); the sum 1 + w is
formed once, in fp32, when the weights are bound. Parameters of both: eps,
dim, and the gain's tensor name.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..ops import kernels
from .base import Norm, Residual, TensorSpec, register_norm


class RMSNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.eps = float(spec["eps"])
        self.dim = int(spec["dim"])
        self.name = str(spec["name"])
        self.gain: Optional[torch.Tensor] = None
        self.act_dtype = torch.float32

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.dim,), role="gain", init="gain", std=0.1)]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.gain = tensors[self.name]
        self.act_dtype = runtime.act_dtype

    def apply(self, stream: Residual, rows: Optional[torch.Tensor] = None, lazy: bool = False):
        delta, scale = stream.take_pending()
        if lazy and rows is None:
            return kernels.NormedInput(stream, delta, self.gain, self.eps, self.act_dtype, delta_scale=scale)
        return kernels.rmsnorm(stream.x, self.gain, self.eps, self.act_dtype, delta=delta, rows=rows, delta_scale=scale)


class OffsetRMSNorm(RMSNorm):
    """The gain is stored around zero and applied as 1 + w."""

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.dim,), role="gain", init="normal", std=0.1)]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.gain = (tensors[self.name].to(torch.float32) + 1.0).contiguous()
        self.act_dtype = runtime.act_dtype


register_norm("rmsnorm", RMSNorm)
register_norm("rmsnorm_offset", OffsetRMSNorm)
