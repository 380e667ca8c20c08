"""Mamba-1 mixer: a gated selective state-space scan.

With h the mixer's input (`csrc/selective_scan.cu` and `csrc/seq_conv.cu` state the formulas):

  [x | z] = W_in h                                  (inner each)
  x <- silu(conv(x))                                 causal, per channel, `conv` taps, with bias
  [dt | B | C] = W_x x                               (dt_rank, state, state)
  dt <- softplus(W_dt dt + dt_bias)                  one step size per channel
  S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,   A = -exp(A_log)
  y_c = sum_n S[c, n] C_n + D_c x_c;   out = W_o (y * silu(z))

S (fp32, [inner, state]) and the convolution's last taps-1 inputs are the
sequence's state. Step sizes, decays and the recurrence are fp32; the step
projection's output stays fp32 on its way to the softplus.

Parameters: hidden_size, inner, state, dt_rank, conv (taps), and the tensors'
names: in, conv_name, conv_bias, x, dt, dt_bias, A_log, D, o.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import PartSpec
from ..ops import kernels
from .base import CacheView, Mixer, StateRequest, TensorSpec, register_mixer

_NAMES = ("in", "conv_name", "conv_bias", "x", "dt", "dt_bias", "A_log", "D", "o")


class Mamba1(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.inner, self.N, self.R, self.taps = g("hidden_size"), g("inner"), g("state"), g("dt_rank"), g("conv")
        self.names = {k: str(spec[k]) for k in _NAMES}
        if self.N > 256:
            from ..config.keys import ConfigError
            raise ConfigError(f"mamba1: a state of {self.N} values a channel exceeds the 256 that the scan kernel holds")

    def tensor_specs(self) -> list[TensorSpec]:
        n, D, I, N, R = self.names, self.D, self.inner, self.N, self.R
        return [TensorSpec(n["in"], (2 * I, D)),
                TensorSpec(n["conv_name"], (I, self.taps), init="normal", std=0.2),
                TensorSpec(n["conv_bias"], (I,), role="gain", init="normal", std=0.1),
                TensorSpec(n["x"], (R + 2 * N, I)),
                TensorSpec(n["dt"], (I, R), init="normal", std=0.1),
                TensorSpec(n["dt_bias"], (I,), role="gain", init="normal", std=0.5),
                TensorSpec(n["A_log"], (I, N), role="gain", init="normal", std=0.5),
                TensorSpec(n["D"], (I,), role="gain", init="gain", std=0.1),
                TensorSpec(n["o"], (D, I))]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        n = self.names
        self.w_in, self.w_x, self.w_dt, self.w_o = tensors[n["in"]], tensors[n["x"]], tensors[n["dt"]], tensors[n["o"]]
        self.conv_w = tensors[n["conv_name"]]
        self.conv_b = tensors[n["conv_bias"]].to(self.conv_w.dtype)
        self.A_log = tensors[n["A_log"]]
        self.dt_b = tensors[n["dt_bias"]].to(self.A_log.dtype)
        self.Dv = tensors[n["D"]].to(self.A_log.dtype)
        self.act_dtype = runtime.act_dtype

    def streamed_tensors(self) -> list:
        return [self.w_in, self.w_x, self.w_dt, self.w_o]

    def state_request(self):
        req = {"scan": StateRequest((self.inner, self.N), torch.float32)}
        if self.taps > 1:
            req["conv"] = StateRequest((self.taps - 1, self.inner), torch.float32)
        return req

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        I, N, R = self.inner, self.N, self.R
        xz = kernels.linear(h, self.w_in)
        x = kernels.causal_conv(xz[:, :I], self.conv_w, self.conv_b, cache.state.get("conv"), ctx, self.act_dtype,
                                act="silu")
        dbc = kernels.linear(x, self.w_x)
        dt_raw = kernels.linear(dbc[:, :R], self.w_dt, out_dtype=torch.float32)
        y = kernels.selective_scan(x, xz[:, I:], dt_raw, dbc[:, R:R + N], dbc[:, R + N:], self.dt_b, self.A_log, self.Dv,
                                   cache.state["scan"], ctx)
        return kernels.linear(y, self.w_o, out_dtype=torch.float32)        # unrounded into the norm that follows


register_mixer("mamba1", Mamba1)
