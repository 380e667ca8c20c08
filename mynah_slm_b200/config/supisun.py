"""Typed configuration of the Supisun design, read from its config.json.

A small decoder-only model whose layers are listed one by one: `layers[i]`
names the layer's mixer (`type`: "attention", "mamba1" or "delta"), the mixer's
sizes (`mixer`) and its feed-forward (`mlp`, or null for none). Every size and
every constant that can differ between two models of the design is read from
the file; what the design fixes (the epsilon of the unit norms, the pairing of
rotated dimensions, the activation of the feed-forward) lives in the parts.

  architecture   "Supisun"
  vocab, width, max_positions
  norm.eps       epsilon of every layer norm and RMS norm
  canon.taps     taps of the causal convolution in front of every mixer
  layers[i]      {type, mixer: {...}, mlp: {kind: "dense", ff} | null}
    attention    heads, kv_heads, dim, vdim, scale, rot: {dims, base} | absent,
                 mask: {size} | absent, v_mix: bool | absent
    mamba1       inner, state, dt_rank, conv
    delta        heads, kv_heads, dim, vdim, conv

Layer i's tensors start with "l<i>."; the block norms each sublayer's output
(`postnorm_residual`), tokens and learned positions are summed at the start,
a layer norm and an untied head end the model.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .keys import ConfigError, opt_bool, req_float, req_int, req_str
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Supisun"
MIXERS = ("attention", "mamba1", "delta")


def _obj(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: missing config key: {key} (an object)")
    return v


@dataclass(frozen=True)
class SupisunConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    canon_taps: int
    layers: tuple          # of plain dictionaries as in config.json, checked

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "SupisunConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("missing config key: layers (a non-empty list)")
        cfg = cls(vocab=req_int(d, "vocab"), width=req_int(d, "width"), max_positions=req_int(d, "max_positions"),
                  norm_eps=req_float(_obj(d, "norm", "config"), "eps"),
                  canon_taps=req_int(_obj(d, "canon", "config"), "taps"),
                  layers=tuple(copy.deepcopy(layers)))
        cfg.check()
        return cfg

    def check(self) -> None:
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be > 0, got {self.norm_eps}")
        for i, L in enumerate(self.layers):
            w = f"layers[{i}]"
            if not isinstance(L, dict):
                raise ConfigError(f"{w} is not an object")
            kind = req_str(L, "type")
            if kind not in MIXERS:
                raise ConfigError(f"{w}.type is {kind!r}; known: {', '.join(MIXERS)}")
            m = _obj(L, "mixer", w)
            if kind == "attention":
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    req_int(m, k)
                req_float(m, "scale")
                if m.get("rot") is not None:
                    rot = _obj(m, "rot", w + ".mixer")
                    dims = req_int(rot, "dims")
                    if dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"{w}.mixer.rot.dims must be even and at most dim, got {dims}")
                    if not req_float(rot, "base") > 0.0:
                        raise ConfigError(f"{w}.mixer.rot.base must be > 0")
                if m.get("mask") is not None:
                    req_int(_obj(m, "mask", w + ".mixer"), "size")
                opt_bool(m, "v_mix", False)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{w}.mixer: heads is not a multiple of kv_heads")
            elif kind == "mamba1":
                for k in ("inner", "state", "dt_rank", "conv"):
                    req_int(m, k)
            else:
                for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    req_int(m, k)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{w}.mixer: heads is not a multiple of kv_heads")
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"{w}.mlp is neither null nor an object")
                if req_str(mlp, "kind") != "dense":
                    raise ConfigError(f"{w}.mlp.kind is {mlp['kind']!r}; known: dense")
                req_int(mlp, "ff")
        first = [i for i, L in enumerate(self.layers) if L["type"] == "attention" and L["mixer"].get("v_mix")]
        for i in first[1:]:
            a, b = self.layers[first[0]]["mixer"], self.layers[i]["mixer"]
            if (a["kv_heads"], a["vdim"]) != (b["kv_heads"], b["vdim"]):
                raise ConfigError(f"layers[{i}] mixes its values with those of layers[{first[0]}], "
                                  f"but their kv_heads x vdim differ")

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                "canon": {"taps": self.canon_taps}, "layers": copy.deepcopy(list(self.layers))}

    # ---------------------------------------------------------------- spec
    def _mixer(self, i: int, L: Mapping[str, Any], first_mix: int | None) -> PartSpec:
        p = f"l{i}.mix."
        m = L["mixer"]
        if L["type"] == "attention":
            rot = m.get("rot") or {}
            mix = None
            if m.get("v_mix"):
                mix = "first" if i == first_mix else "mix"
            return PartSpec("projnorm_attention", {
                "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                "vdim": m["vdim"], "eps": self.norm_eps, "scale": float(m["scale"]),
                "rot_dims": rot.get("dims", 0), "rot_base": float(rot.get("base", 10000.0)),
                "chunk": (m.get("mask") or {}).get("size"), "window": None,
                "value_mix": mix, "value_mix_key": "supisun", "lambda": p + "vmix" if mix else None,
                "q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_norm": p + "q.norm", "k_norm": p + "k.norm"})
        if L["type"] == "mamba1":
            return PartSpec("mamba1", {
                "hidden_size": self.width, "inner": m["inner"], "state": m["state"], "dt_rank": m["dt_rank"],
                "conv": m["conv"], "in": p + "in", "conv_name": p + "conv", "conv_bias": p + "conv.b", "x": p + "x",
                "dt": p + "dt", "dt_bias": p + "dt.b", "A_log": p + "A_log", "D": p + "D", "o": p + "o"})
        return PartSpec("gated_delta", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
            "vdim": m["vdim"], "conv": m["conv"], "eps": self.norm_eps,
            "q": p + "q", "k": p + "k", "v": p + "v", "q_conv": p + "q.conv", "k_conv": p + "k.conv",
            "v_conv": p + "v.conv", "b": p + "b", "a": p + "a", "A_log": p + "A_log", "dt_bias": p + "dt_bias",
            "g": p + "g", "norm": p + "norm", "o": p + "o"})

    def model_spec(self) -> ModelSpec:
        mixing = [i for i, L in enumerate(self.layers) if L["type"] == "attention" and L["mixer"].get("v_mix")]
        first_mix = mixing[0] if mixing else None
        layers = []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            ln = lambda name: PartSpec("layernorm", {"eps": self.norm_eps, "dim": self.width, "name": p + name,
                                                     "bias": p + name + ".b"})
            mlp = L.get("mlp")
            ffn = None
            norms = {"mixer": ln("norm1")}
            if mlp is not None:
                ffn = PartSpec("dense_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                             "activation": "gelu_erf", "up": p + "mlp.up", "down": p + "mlp.down"})
                norms["ffn"] = ln("norm2")
            layers.append(LayerSpec(
                block=PartSpec("postnorm_residual", {"hidden_size": self.width, "input_conv_taps": self.canon_taps,
                                                     "input_conv_name": p + "canon1"}),
                mixer=self._mixer(i, L, first_mix), ffn=ffn, norms=norms, prefix=p))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=self.max_positions,
            layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            embedding=PartSpec("token_position_embedding", {"name": "embed", "position_name": "pos",
                                                            "vocab_size": self.vocab, "dim": self.width,
                                                            "max_positions": self.max_positions}),
            final_norm=PartSpec("layernorm", {"eps": self.norm_eps, "dim": self.width, "name": "final.norm",
                                              "bias": "final.norm.b"}),
            head=PartSpec("linear_head", {"tied": False, "name": "head", "vocab_size": self.vocab, "dim": self.width}))
        spec.validate()
        return spec
