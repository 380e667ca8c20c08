"""Dense feed-forward without a gate: x -> W_down . act(W_up . x), no bias.

Parameters: hidden_size, intermediate_size, activation ("gelu" or "gelu_erf":
0.5 z (1 + erf(z / sqrt 2)); "gelu_tanh"; "silu"; "relu"; "relu2", the square
of relu), and the two tensors' names (`up`, `down`). The activation is
computed in fp32 from the product's rows. `output` says in what type the last
product leaves its rows: "fp32" (the default: unrounded, for a norm that
follows the sublayer) or "act" (the run's activation type, for a residual add).
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.keys import ConfigError
from ..ops import kernels
from .base import FeedForward, TensorSpec, register_ffn


class DenseMLP(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.D = int(spec["hidden_size"])
        self.F = int(spec["intermediate_size"])
        self.act = str(spec.get("activation", "gelu_erf"))
        if self.act not in kernels.ACTIVATIONS:
            raise ConfigError(f"dense_mlp: activation {self.act!r} is not built in "
                              f"(known: {', '.join(sorted(kernels.ACTIVATIONS))})")
        self.out_fp32 = str(spec.get("output", "fp32")) == "fp32"
        self.up_name, self.down_name = str(spec["up"]), str(spec["down"])
        self.w_up = self.w_down = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.up_name, (self.F, self.D)), TensorSpec(self.down_name, (self.D, self.F))]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.w_up, self.w_down = tensors[self.up_name], tensors[self.down_name]

    def streamed_tensors(self) -> list:
        return [self.w_up, self.w_down]

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        u = kernels.linear(h, self.w_up)
        kernels.activation(u, self.act, out=u)
        return kernels.linear(u, self.w_down, out_dtype=torch.float32 if self.out_fp32 else None)


register_ffn("dense_mlp", DenseMLP)
