"""A block that norms each sublayer's OUTPUT: x <- x + norm_mixer(mixer(in(x))), then
x <- x + norm_ffn(ffn(x)). The sublayers read the residual stream itself, which
stays fp32; no norm stands in front of them.

`in(x)`, optional, is a short causal convolution over time on every channel of
the stream, added to it: in(x) = x + conv(x) with a filter [hidden, taps] and no
bias (parameters `input_conv_taps`, `input_conv_name`; taps 0 or None: the mixer
reads x). The convolution's last taps-1 inputs are part of a sequence's state:
the block asks the cache for them. The feed-forward may be missing (`ffn` None).

The norms, named "mixer" and "ffn", must offer `add_normed(stream, y, copy)`.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.keys import ConfigError
from ..ops import kernels
from .base import Block, CacheView, Residual, StateRequest, TensorSpec, register_block


class PostNormResidual(Block):
    def __init__(self, spec, mixer, ffn, norms):
        super().__init__(spec, mixer, ffn, norms)
        need = ("mixer",) + (("ffn",) if ffn is not None else ())
        for n in need:
            if n not in self.norms:
                raise ConfigError(f"postnorm_residual: the layer gives no {n!r} norm")
            if not hasattr(self.norms[n], "add_normed"):
                raise ConfigError(f"postnorm_residual: norm {n!r} cannot norm a sublayer's output (no add_normed)")
        self.D = int(spec["hidden_size"])
        self.taps = int(spec.get("input_conv_taps") or 0)
        self.conv_name: Optional[str] = spec.get("input_conv_name")
        if self.taps and not self.conv_name:
            raise ConfigError("postnorm_residual: an input convolution needs its tensor's name")
        self.conv_w: Optional[torch.Tensor] = None
        self.act_dtype = torch.float32

    def tensor_specs(self) -> list[TensorSpec]:
        if not self.taps:
            return []
        return [TensorSpec(self.conv_name, (self.D, self.taps), init="normal", std=0.1)]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        if self.taps:
            self.conv_w = tensors[self.conv_name]
        self.act_dtype = runtime.act_dtype

    def state_request(self):
        if self.taps > 1:
            return {"input_conv": StateRequest((self.taps - 1, self.D), torch.float32)}
        return None

    def forward(self, stream: Residual, ctx, cache: CacheView) -> None:
        x = stream.flush()
        if self.taps:
            state = cache.block_state["input_conv"] if self.taps > 1 else None
            h = kernels.causal_conv(x, self.conv_w, None, state, ctx, self.act_dtype, add_input=True)
        else:
            h = x if self.act_dtype == torch.float32 else kernels.cast_rows(x, self.act_dtype)
        y = self.mixer.forward(h, ctx, cache)
        want_copy = self.ffn is not None and self.act_dtype != torch.float32
        xc = self.norms["mixer"].add_normed(stream, y, copy=want_copy)
        if self.ffn is not None:
            y = self.ffn.forward(xc if xc is not None else stream.x, ctx)
            self.norms["ffn"].add_normed(stream, y)


register_block("postnorm_residual", PostNormResidual)
