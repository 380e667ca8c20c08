"""Grouped-query softmax attention whose q and k are normed over the WHOLE
projection, with rotary positions on part of each head, normed values, an
optional mix of the values with an earlier layer's, a chunked mask and a score
scale given by the configuration.

Per token, with h the mixer's input (all of this in fp32 behind the bf16
projections; `csrc/attn_prep.cu` states the formulas):

  q = W_q h, k = W_k h, v = W_v h                          (no biases)
  q <- rms_norm(q over all H*dim outputs) * q_gain         (k likewise, G*dim)
  rotate the first `rot_dims` dimensions of each head of q and k (i with i + rot_dims/2)
  v <- v / rms(v over the head's vdim)
  v <- (1 - lambda) v + lambda v_first                     (`value_mix` = "mix"; the layer with
                                                            `value_mix` = "first" leaves v_first)
  k, v -> cache;  score = q.k * scale;  softmax over the visible keys;  W_o on the heads

Visible keys: j <= i, within `window` when given, and, with `chunk` = C, only
floor(j / C) == floor(i / C), chunks counted from the sequence's position 0.
Query head h reads kv head h // (H / G).

Parameters: hidden_size, heads, kv_heads, dim, vdim, eps, scale, rot_dims,
rot_base, chunk, window, value_mix (None | "first" | "mix"), value_mix_key (the
name under which the layers of one model share v_first), and the tensors'
names: q, k, v, o, q_norm, k_norm, lambda.

Heads are stored padded to multiples of 8 (zeros), which the attention kernels'
16-byte loads need; W_o gets matching zero columns.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import kernels
from .base import CacheView, KVRequest, Mixer, TensorSpec, build_part, register_mixer


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class ProjNormAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.H, self.G, self.dim, self.vd = g("hidden_size"), g("heads"), g("kv_heads"), g("dim"), g("vdim")
        self.eps = float(spec["eps"])
        self.scale = float(spec["scale"])
        self.rot = int(spec.get("rot_dims") or 0)
        self.chunk: Optional[int] = spec.get("chunk")
        self.window: Optional[int] = spec.get("window")
        self.value_mix: Optional[str] = spec.get("value_mix")
        self.mix_key = "v_first:" + str(spec.get("value_mix_key", ""))
        self.names = {k: str(spec[k]) for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
        self.lambda_name: Optional[str] = spec.get("lambda")
        if self.H % self.G:
            raise ConfigError(f"attention: {self.H} heads are not a multiple of {self.G} kv heads")
        self.dimp, self.vdp = _pad8(self.dim), _pad8(self.vd)
        if max(self.dimp, self.vdp) > kernels.MAX_HEAD_DIM:
            raise ConfigError(f"attention: heads of {self.dim} / {self.vd} exceed {kernels.MAX_HEAD_DIM}")
        if self.rot % 2 or self.rot > self.dim or self.rot < 0:
            raise ConfigError(f"attention: {self.rot} rotated dimensions must be even and at most the head's {self.dim}")
        if self.chunk is not None and self.chunk < 1:
            raise ConfigError(f"attention: chunk {self.chunk} must be positive")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"attention: window {self.window} must be positive")
        if self.value_mix not in (None, "first", "mix"):
            raise ConfigError(f"attention: value_mix {self.value_mix!r} is not one of None, 'first', 'mix'")
        if self.value_mix == "mix" and not self.lambda_name:
            raise ConfigError("attention: value mixing needs the name of its weight")
        self.position = (build_part("position", PartSpec("rope_neox", {"theta": float(spec["rot_base"]),
                                                                       "rotary_dim": self.rot}))
                         if self.rot else None)

    def tensor_specs(self) -> list[TensorSpec]:
        n, H, G, dim, vd, D = self.names, self.H, self.G, self.dim, self.vd, self.D
        specs = [TensorSpec(n["q"], (H * dim, D)), TensorSpec(n["k"], (G * dim, D)), TensorSpec(n["v"], (G * vd, D)),
                 TensorSpec(n["o"], (D, H * vd)),
                 TensorSpec(n["q_norm"], (H * dim,), role="gain", init="gain", std=0.1),
                 TensorSpec(n["k_norm"], (G * dim,), role="gain", init="gain", std=0.1)]
        if self.lambda_name:
            # the first mixing layer's weight exists in the checkpoint but is never read
            specs.append(TensorSpec(self.lambda_name, (), role="gain", init="normal", std=0.3,
                                    ignorable=self.value_mix != "mix"))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        n = self.names
        self.w_qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        w_o = tensors[n["o"]]
        if self.vdp != self.vd:
            padded = torch.zeros((self.D, self.H, self.vdp), dtype=w_o.dtype, device=w_o.device)
            padded[:, :, : self.vd] = w_o.view(self.D, self.H, self.vd)
            w_o = padded.view(self.D, self.H * self.vdp).contiguous()
        self.w_o = w_o
        self.q_gain = tensors[n["q_norm"]]
        self.k_gain = tensors[n["k_norm"]].to(self.q_gain.dtype)
        self.lam = (tensors[self.lambda_name].to(torch.float32).reshape(1).contiguous()
                    if self.value_mix == "mix" else None)
        self.cos = self.sin = None
        if self.position is not None:
            self.position.prepare(runtime)
            self.cos, self.sin, _ = self.position.fused_tables()
        self.runtime = runtime

    def streamed_tensors(self) -> list:
        return [self.w_qkv, self.w_o]

    def kv_request(self) -> KVRequest:
        return KVRequest(self.G, self.dimp, self.window, v_head_dim=self.vdp)

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        H, G, dim, vd, dimp, vdp = self.H, self.G, self.dim, self.vd, self.dimp, self.vdp
        T = h.shape[0]
        writes = cache.writes
        pages = ctx.pages[cache.group]
        qkv = kernels.linear(h, self.w_qkv if writes else self.w_qkv[: H * dim])
        q = torch.empty((T, H * dimp), dtype=qkv.dtype, device=qkv.device)
        v_first, vmix = None, 0
        if writes and self.value_mix == "first":
            v_first = ctx.shared[self.mix_key] = torch.empty((T, G * vd), dtype=torch.float32, device=qkv.device)
            vmix = 1
        elif writes and self.value_mix == "mix":
            v_first = ctx.shared.get(self.mix_key)
            if v_first is None or v_first.shape != (T, G * vd):
                raise ConfigError("attention: no earlier layer of this step left values of this shape to mix with")
            vmix = 2
        kernels.attn_prep(qkv, q, H, G, dim, vd, dimp, vdp, self.q_gain, self.k_gain, self.eps, self.cos, self.sin,
                          self.rot, ctx, pages, cache.k if writes else None, cache.v if writes else None,
                          v_first, self.lam, vmix)
        out = torch.empty((T, H * vdp), dtype=qkv.dtype, device=qkv.device)
        from ..ops import attention_dispatch
        if ctx.is_decode:
            attention_dispatch.decode_masked(q, out, ctx, H, G, dimp, vdp, cache.k, cache.v, pages, self.window or 0,
                                             self.chunk or 0, self.scale,
                                             self.runtime.attn_scratch(ctx.B, H, vdp, ctx.decode_splits))
        else:
            attention_dispatch.prefill_masked(q, out, ctx, H, G, dimp, vdp, cache.k, cache.v, pages, self.window or 0,
                                              self.chunk or 0, self.scale)
        return kernels.linear(out, self.w_o, out_dtype=torch.float32)      # unrounded into the norm that follows


register_mixer("projnorm_attention", ProjNormAttention)
