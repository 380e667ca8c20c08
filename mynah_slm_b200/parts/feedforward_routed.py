"""Feed-forward of several small experts, of which every token uses `top`, picked
without a router: a table [vocab, top] gives each token id its experts (the
entries of a row differ), and each counts 1/top.

An expert, with h its input (no biases):

  g = min(W_gate h, limit),   u = clamp(W_up h, -limit, limit)
  y = g * sigmoid(alpha g) * (u + 1),   out = W_down y

The step's (token, choice) pairs are sorted by expert on the device and the two
products run tile by tile over rows that share an expert (`csrc/moe.cu`); the
experts' matrices are stacked at bind time.

Parameters: hidden_size, intermediate_size (of one expert), experts, top, limit,
alpha (1.702 unless given), vocab_size, table (tensor name) and expert_prefix:
expert e's tensors are `<expert_prefix><e>.gate`, `.up` and `.down`.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.keys import ConfigError
from ..ops import kernels
from .base import FeedForward, TensorSpec, register_ffn


class TableRoutedExperts(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.F, self.E, self.top, self.V = (g("hidden_size"), g("intermediate_size"), g("experts"), g("top"),
                                                    g("vocab_size"))
        self.limit = float(spec["limit"])
        self.alpha = float(spec.get("alpha", 1.702))
        self.table_name = str(spec["table"])
        self.prefix = str(spec["expert_prefix"])
        if not 1 <= self.top <= self.E:
            raise ConfigError(f"table_routed_experts: top {self.top} does not fit {self.E} experts")
        if self.E > 1024:
            raise ConfigError(f"table_routed_experts: {self.E} experts exceed the 1024 that the routing kernel counts")

    def _name(self, e: int, which: str) -> str:
        return f"{self.prefix}{e}.{which}"

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [TensorSpec(self.table_name, (self.V, self.top), role="table", init=f"distinct:{self.E}")]
        for e in range(self.E):
            specs += [TensorSpec(self._name(e, "gate"), (self.F, self.D)), TensorSpec(self._name(e, "up"), (self.F, self.D)),
                      TensorSpec(self._name(e, "down"), (self.D, self.F))]
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.table = tensors[self.table_name].contiguous()
        self.w_gu = torch.stack([torch.stack([tensors[self._name(e, "gate")], tensors[self._name(e, "up")]])
                                 for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[self._name(e, "down")] for e in range(self.E)]).contiguous()

    def streamed_tensors(self) -> list:
        return []          # a step reads only the experts its tokens pick

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return kernels.moe_table_ffn(h, self.table, self.w_gu, self.w_down, ctx, self.top, self.limit, self.alpha)


register_ffn("table_routed_experts", TableRoutedExperts)
