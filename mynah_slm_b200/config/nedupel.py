"""Typed configuration of the Nedupel design, read from its config.json.

A small decoder-only model whose layers are listed one by one: `layers[i]`
names the layer's mixer (`type`: "latent_attention" or "retention"), the
mixer's sizes (`mixer`) and its feed-forward (`mlp`, or null for none). Every
size and every constant that can differ between two models of the design is
read from the file; what the design fixes (the pairing of rotated dimensions of
each mixer, the activations, the constant in the experts' gate) lives here and
in the parts.

  architecture      "Nedupel"
  vocab, width
  embedding.scale   the token embedding is multiplied by it
  residual_mult     every sublayer's output is multiplied by it on its way into the stream
  logit_scale       the logits are multiplied by it
  norm.eps          epsilon of every RMS norm (the gains are stored around zero: 1 + w)
  layers[i]         {type, mixer: {...}, mlp: {...} | null}
    latent_attention  heads, dim, rot_dim, vdim, kv_rank, scale, rot: {dims, base, scaling?}, kv_from?: j
                      (kv_from: the layer has no down-projection and reads layer j's cache)
    retention         heads, dim, vdim, decay: [per head], rot: {dims, base, scaling?} | absent
    mlp               {kind: "dense", ff}  |  {kind: "moe", expert: {ff, limit}, router: {experts, top}}
  max_positions     optional; the design itself has no limit, so 2^20 unless given

Layer i's tensors start with "l<i>."; the block is pre-norm with two norms
(`norm1`, `norm2`), a norm (`final.norm`) and an untied head (`head`) end the
model.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .keys import ConfigError, opt_int, req_float, req_int, req_str
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Nedupel"
MIXERS = ("latent_attention", "retention")
GATE_ALPHA = 1.702          # the experts' gate is g * sigmoid(GATE_ALPHA g)


def _obj(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: missing config key: {key} (an object)")
    return v


def _check_rot(rot: Any, limit: int, where: str) -> None:
    if not isinstance(rot, dict):
        raise ConfigError(f"{where}.rot is not an object")
    dims = req_int(rot, "dims")
    if dims % 2 or dims > limit:
        raise ConfigError(f"{where}.rot.dims must be even and at most {limit}, got {dims}")
    if not req_float(rot, "base") > 0.0:
        raise ConfigError(f"{where}.rot.base must be > 0")
    if rot.get("scaling") is not None:
        sc = _obj(rot, "scaling", where + ".rot")
        for k in ("factor", "original", "fast", "slow"):
            if not req_float(sc, k) > 0.0:
                raise ConfigError(f"{where}.rot.scaling.{k} must be > 0")


@dataclass(frozen=True)
class NedupelConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    logit_scale: float
    layers: tuple          # of plain dictionaries as in config.json, checked
    has_max_positions: bool = False

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "NedupelConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("missing config key: layers (a non-empty list)")
        mp = opt_int(d, "max_positions", None)
        cfg = cls(vocab=req_int(d, "vocab"), width=req_int(d, "width"), max_positions=mp if mp is not None else 1 << 20,
                  norm_eps=req_float(_obj(d, "norm", "config"), "eps"),
                  embedding_scale=req_float(_obj(d, "embedding", "config"), "scale"),
                  residual_mult=req_float(d, "residual_mult"), logit_scale=req_float(d, "logit_scale"),
                  layers=tuple(copy.deepcopy(layers)), has_max_positions=mp is not None)
        cfg.check()
        return cfg

    def check(self) -> None:
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be > 0, got {self.norm_eps}")
        if self.max_positions < 1:
            raise ConfigError(f"max_positions must be >= 1, got {self.max_positions}")
        for i, L in enumerate(self.layers):
            w = f"layers[{i}]"
            if not isinstance(L, dict):
                raise ConfigError(f"{w} is not an object")
            kind = req_str(L, "type")
            if kind not in MIXERS:
                raise ConfigError(f"{w}.type is {kind!r}; known: {', '.join(MIXERS)}")
            m = _obj(L, "mixer", w)
            if kind == "latent_attention":
                for k in ("heads", "vdim", "kv_rank"):
                    req_int(m, k)
                req_int(m, "dim", minimum=0)
                req_int(m, "rot_dim", minimum=0)
                req_float(m, "scale")
                if m.get("rot") is not None:
                    _check_rot(m["rot"], m["rot_dim"], w + ".mixer")
                src = opt_int(m, "kv_from", None)
                if src is not None:
                    if not 0 <= src < i:
                        raise ConfigError(f"{w}.mixer.kv_from names layer {src}, which does not run before layer {i}")
                    S = self.layers[src]
                    if S.get("type") != "latent_attention" or S["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{w}.mixer.kv_from names layer {src}, which keeps no latent cache of its own")
                    for k in ("kv_rank", "rot_dim", "rot"):
                        if S["mixer"].get(k) != m.get(k):
                            raise ConfigError(f"{w}.mixer.{k} differs from that of layer {src}, whose cache it reads")
            else:
                for k in ("heads", "dim", "vdim"):
                    req_int(m, k)
                decay = m.get("decay")
                if (not isinstance(decay, list) or len(decay) != m["heads"]
                        or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay)):
                    raise ConfigError(f"{w}.mixer.decay must list one number per head")
                if m.get("rot") is not None:
                    _check_rot(m["rot"], m["dim"], w + ".mixer")
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"{w}.mlp is neither null nor an object")
                mk = req_str(mlp, "kind")
                if mk == "dense":
                    req_int(mlp, "ff")
                elif mk == "moe":
                    ex, ro = _obj(mlp, "expert", w + ".mlp"), _obj(mlp, "router", w + ".mlp")
                    req_int(ex, "ff")
                    req_float(ex, "limit")
                    if req_int(ro, "top") > req_int(ro, "experts"):
                        raise ConfigError(f"{w}.mlp.router.top exceeds the number of experts")
                else:
                    raise ConfigError(f"{w}.mlp.kind is {mk!r}; known: dense, moe")

    def to_dict(self) -> dict[str, Any]:
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult,
             "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.has_max_positions:
            d["max_positions"] = self.max_positions
        return d

    # ---------------------------------------------------------------- spec
    def _mixer(self, i: int, L: Mapping[str, Any]) -> PartSpec:
        p = f"l{i}.mix."
        m = L["mixer"]
        rot = m.get("rot")
        if L["type"] == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                "vdim": m["vdim"], "kv_rank": m["kv_rank"], "eps": self.norm_eps, "scale": float(m["scale"]),
                "window": None, "own_kv": m.get("kv_from") is None,
                "rot": {**rot, "pairing": "interleaved"} if rot else None,
                "q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv", "o": p + "o"})
        return PartSpec("retention", {
            "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
            "decay": [float(x) for x in m["decay"]], "eps": self.norm_eps,
            "rot": {**rot, "pairing": "half"} if rot else None,
            "q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "o": p + "o"})

    def _ffn(self, i: int, mlp: Mapping[str, Any]) -> PartSpec:
        p = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return PartSpec("dense_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "relu2",
                                          "output": "act", "up": p + "up", "down": p + "down"})
        return PartSpec("table_routed_experts", {
            "hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"], "experts": mlp["router"]["experts"],
            "top": mlp["router"]["top"], "limit": float(mlp["expert"]["limit"]), "alpha": GATE_ALPHA,
            "vocab_size": self.vocab, "table": p + "table", "expert_prefix": p + "e"})

    def model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            norm = lambda name: PartSpec("rmsnorm_offset", {"eps": self.norm_eps, "dim": self.width, "name": name})
            mlp = L.get("mlp")
            norms = {"mixer": norm(p + "norm1")}
            if mlp is not None:
                norms["ffn"] = norm(p + "norm2")
            layers.append(LayerSpec(
                block=PartSpec("prenorm_residual", {"residual_mult": self.residual_mult}),
                mixer=self._mixer(i, L), ffn=self._ffn(i, mlp) if mlp is not None else None, norms=norms, prefix=p))
            # one run a layer, in order: schedule index == layer index
            schedule.append(ScheduleEntry(i, cache_from=L["mixer"].get("kv_from") if L["type"] == "latent_attention" else None))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=self.max_positions,
            layers=tuple(layers), schedule=tuple(schedule),
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": self.vocab, "dim": self.width,
                                                   "scale": self.embedding_scale}),
            final_norm=PartSpec("rmsnorm_offset", {"eps": self.norm_eps, "dim": self.width, "name": "final.norm"}),
            head=PartSpec("linear_head", {"tied": False, "name": "head", "vocab_size": self.vocab, "dim": self.width,
                                          "logit_scale": self.logit_scale}))
        spec.validate()
        return spec
