"""Retention: linear attention with a fixed decay per head, no softmax and no
denominator.

With h the mixer's input (`csrc/retention.cu` states the recurrence):

  q = W_q h, k = W_k h   (heads x dim),   v = W_v h   (heads x vdim);   no biases
  q and k are rotated (the position part's pairing and tables); k <- k * dim^(-1/2) after the rotation
  per head:   S <- decay_h S + k v^T;   o = S^T q
  out = W_o (o / rms(o over the head's vdim) * silu(W_g h))          (the unit RMS has no weight)

S (fp32, [heads, dim, vdim]) is the sequence's state; it starts at zero. The
four projections of h run as one product (their matrices stacked at bind time).

Parameters: hidden_size, heads, dim, vdim, decay (one per head), eps, rot (None
or the parameters of a `rotary` position part), and the tensors' names: q, k, v,
g, o.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import kernels
from .base import CacheView, Mixer, StateRequest, TensorSpec, build_part, register_mixer


class Retention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.H, self.dim, self.vd = g("hidden_size"), g("heads"), g("dim"), g("vdim")
        self.eps = float(spec["eps"])
        self.decay = [float(x) for x in spec["decay"]]
        self.names = {k: str(spec[k]) for k in ("q", "k", "v", "g", "o")}
        if len(self.decay) != self.H:
            raise ConfigError(f"retention: {len(self.decay)} decays for {self.H} heads")
        if self.dim > 512:
            raise ConfigError(f"retention: keys of {self.dim} values exceed the 512 that the recurrence kernel stages")
        rot = spec.get("rot")
        self.position = build_part("position", PartSpec("rotary", dict(rot))) if rot else None
        if self.position is not None and self.position.dims > self.dim:
            raise ConfigError(f"retention: {self.position.dims} rotated dims exceed the head's {self.dim}")

    def tensor_specs(self) -> list[TensorSpec]:
        n, H, D = self.names, self.H, self.D
        return [TensorSpec(n["q"], (H * self.dim, D)), TensorSpec(n["k"], (H * self.dim, D)),
                TensorSpec(n["v"], (H * self.vd, D)), TensorSpec(n["g"], (H * self.vd, D)),
                TensorSpec(n["o"], (D, H * self.vd))]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        n = self.names
        parts = [tensors[n[k]] for k in ("q", "k", "v", "g")]
        rows = sum(p.shape[0] for p in parts)
        if rows % 8:
            parts.append(torch.zeros((8 - rows % 8, self.D), dtype=parts[0].dtype, device=parts[0].device))
        self.w_all = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        dev = self.w_o.device
        self.decay_t = torch.tensor(self.decay, dtype=torch.float32, device=dev)
        self.ones = torch.ones((self.vd,), dtype=torch.float32, device=dev)
        self.cos = self.sin = None
        self.rot, self.interleaved = 0, False
        if self.position is not None:
            self.position.prepare(runtime)
            self.cos, self.sin, self.rot = self.position.fused_tables()
            self.interleaved = self.position.interleaved

    def streamed_tensors(self) -> list:
        return [self.w_all, self.w_o]

    def state_request(self):
        return {"S": StateRequest((self.H, self.dim, self.vd), torch.float32)}

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        H, dim, vd = self.H, self.dim, self.vd
        p = kernels.linear(h, self.w_all)
        nq = H * dim
        qn, kn = kernels.retention_prep(p, 0, nq, H, dim, self.cos, self.sin, self.rot, self.interleaved,
                                        float(dim) ** -0.5, ctx)
        o = kernels.retention_scan(qn, kn, p, 2 * nq, self.decay_t, cache.state["S"], ctx, H, dim, vd)
        out = kernels.gated_rmsnorm(o, p[:, 2 * nq + H * vd: 2 * nq + 2 * H * vd], self.ones, H, vd, self.eps)
        return kernels.linear(out, self.w_o)


register_mixer("retention", Retention)
