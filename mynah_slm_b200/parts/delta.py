"""Gated delta rule mixer: linear attention whose state is corrected towards
each new value along its key, with a learned per-head decay.

With h the mixer's input (`csrc/delta_rule.cu` states the formulas):

  q = W_q h, k = W_k h   (kv_heads x dim),   v = W_v h   (heads x vdim);   no biases
  each passes a short causal convolution per channel (no bias) and silu
  q, k <- unit vectors per head, x / sqrt(sum(x^2) + 1e-6);   q <- q * dim^(-1/2)
  beta = sigmoid(W_b h);   g = exp(-exp(A_log) * softplus(W_a h + dt_bias))      one each per head
  per head:   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
  out = W_o (o / rms(o over vdim) * norm_w * silu(W_g h))

Head h reads q/k head h // (heads / kv_heads). S (fp32, [heads, dim, vdim]) and
the convolutions' last taps-1 inputs are the sequence's state.

The six projections of h run as one product (their matrices stacked at bind
time, padded to a multiple of 8 rows), the three convolutions as one launch over
the stacked channels.

Parameters: hidden_size, heads, kv_heads, dim, vdim, conv (taps), eps, and the
tensors' names: q, k, v, q_conv, k_conv, v_conv, b, a, A_log, dt_bias, g, norm, o.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import kernels
from .base import CacheView, Mixer, StateRequest, TensorSpec, register_mixer

_NAMES = ("q", "k", "v", "q_conv", "k_conv", "v_conv", "b", "a", "A_log", "dt_bias", "g", "norm", "o")


class GatedDelta(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.H, self.G, self.dim, self.vd, self.taps = (g("hidden_size"), g("heads"), g("kv_heads"), g("dim"),
                                                               g("vdim"), g("conv"))
        self.eps = float(spec["eps"])
        self.names = {k: str(spec[k]) for k in _NAMES}
        if self.H % self.G:
            raise ConfigError(f"gated_delta: {self.H} heads are not a multiple of {self.G} q/k heads")
        if self.dim > 512:
            raise ConfigError(f"gated_delta: keys of {self.dim} values exceed the 512 that the recurrence kernel stages")
        self.n_qk = 2 * self.G * self.dim
        self.n_conv = self.n_qk + self.H * self.vd

    def tensor_specs(self) -> list[TensorSpec]:
        n, D, H, G, dim, vd, t = self.names, self.D, self.H, self.G, self.dim, self.vd, self.taps
        return [TensorSpec(n["q"], (G * dim, D)), TensorSpec(n["k"], (G * dim, D)), TensorSpec(n["v"], (H * vd, D)),
                TensorSpec(n["q_conv"], (G * dim, t), init="normal", std=0.3),
                TensorSpec(n["k_conv"], (G * dim, t), init="normal", std=0.3),
                TensorSpec(n["v_conv"], (H * vd, t), init="normal", std=0.3),
                TensorSpec(n["b"], (H, D)), TensorSpec(n["a"], (H, D)),
                TensorSpec(n["A_log"], (H,), role="gain", init="normal", std=0.5),
                TensorSpec(n["dt_bias"], (H,), role="gain", init="normal", std=0.5),
                TensorSpec(n["g"], (H * vd, D)),
                TensorSpec(n["norm"], (vd,), role="gain", init="gain", std=0.1),
                TensorSpec(n["o"], (D, H * vd))]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        n = self.names
        parts = [tensors[n[k]] for k in ("q", "k", "v", "g", "b", "a")]
        rows = sum(p.shape[0] for p in parts)
        if rows % 8:
            parts.append(torch.zeros((8 - rows % 8, self.D), dtype=parts[0].dtype, device=parts[0].device))
        self.w_all = torch.cat(parts, dim=0).contiguous()
        self.conv_w = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]], dim=0).contiguous()
        self.A_log = tensors[n["A_log"]]
        self.dt_bias = tensors[n["dt_bias"]].to(self.A_log.dtype)
        self.norm_w = tensors[n["norm"]]
        self.w_o = tensors[n["o"]]
        self.act_dtype = runtime.act_dtype

    def streamed_tensors(self) -> list:
        return [self.w_all, self.w_o]

    def state_request(self):
        req = {"S": StateRequest((self.H, self.dim, self.vd), torch.float32)}
        if self.taps > 1:
            req["conv"] = StateRequest((self.taps - 1, self.n_conv), torch.float32)
        return req

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        H, G, dim, vd = self.H, self.G, self.dim, self.vd
        p = kernels.linear(h, self.w_all)
        c0 = self.n_conv
        c1 = c0 + H * vd
        qkv = kernels.causal_conv(p[:, :c0], self.conv_w, None, cache.state.get("conv"), ctx, self.act_dtype, act="silu")
        qn, kn, g, beta = kernels.delta_prep(qkv[:, : self.n_qk], p[:, c1 + H: c1 + 2 * H], p[:, c1: c1 + H],
                                             self.A_log, self.dt_bias, H, G, dim)
        o = kernels.delta_rule(qn, kn, qkv[:, self.n_qk:], g, beta, cache.state["S"], ctx, H, G, dim, vd)
        out = kernels.gated_rmsnorm(o, p[:, c0:c1], self.norm_w, H, vd, self.eps)
        return kernels.linear(out, self.w_o, out_dtype=torch.float32)      # unrounded into the norm that follows


register_mixer("gated_delta", GatedDelta)
