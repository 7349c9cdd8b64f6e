"""Typed configuration of the Pufuzen decoder: a small decoder-only model whose layers mix
tokens with a minGRU recurrence or with attention over a cached latent (with a sliding window,
or with rotary positions and a softmax sink), each sublayer's output scaled by a gate of the
sublayer's input, and a dense feed-forward with the PolyNorm activation.

config.json keys: `architecture` ("Pufuzen"), `vocab`, `width`, `logit_scale`, `norm.eps`, and
`layers`: a list of {`type`, `mixer` (the mixer's sizes), `mlp` (null or {`kind`: "dense", `ff`})}.
  type "mingru":              mixer {width}
  type "latent_attention":    mixer {heads, dim, vdim, q_rank, kv_rank, scale, mask {size}}
                              (no positions; a query sees itself and the mask.size - 1 keys before;
                              a mixer without `mask` sees every earlier key)
  type "latent_attention_2":  mixer {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale,
                              rot {base, dims}} (causal; rotary lanes; a sink per head)
Tensors: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.rg1`, `l<i>.rg2`
(+ `.b`), `final.norm`, `head`.  Every size is read here; none stands in the parts.
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List

from .registry import register_architecture
from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec, as_float, as_int, require_keys

ARCHITECTURE = "Pufuzen"
# The design has no longest position (no tables); what the engine uses as its bound on a
# request's length.
POSITIONS = 1 << 20

_MIXER_KEYS = {
    "mingru": ["width"],
    "latent_attention": ["heads", "dim", "vdim", "q_rank", "kv_rank", "scale"],
    "latent_attention_2": ["heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot"],
}


class PufuzenConfig:
    def __init__(self, raw: Dict[str, Any]):
        self.raw = raw
        self.vocab = as_int(raw, "vocab", 1)
        self.width = as_int(raw, "width", 1)
        self.logit_scale = as_float(raw, "logit_scale") if raw.get("logit_scale") is not None else 1.0
        if not isinstance(raw["norm"], dict) or "eps" not in raw["norm"]:
            raise ConfigError("config.json norm must be an object with eps")
        self.eps = as_float(raw["norm"], "eps")
        if self.eps < 0:
            raise ConfigError("norm.eps must not be negative")
        self.layers: List[Dict[str, Any]] = raw["layers"]
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json layers must be a list with at least one layer")
        for index, layer in enumerate(self.layers):
            self._check_layer(index, layer)

    @staticmethod
    def _check_layer(index: int, layer: Dict[str, Any]) -> None:
        what = f"{ARCHITECTURE} layer {index}"
        if not isinstance(layer, dict):
            raise ConfigError(f"{what} must be an object")
        require_keys(layer, ["type", "mixer"], what)
        kind = layer["type"]
        if kind not in _MIXER_KEYS:
            raise ConfigError(f"{what}: unknown type {kind!r} (known: {', '.join(sorted(_MIXER_KEYS))})")
        m = layer["mixer"]
        if not isinstance(m, dict):
            raise ConfigError(f"{what}: mixer must be an object")
        require_keys(m, _MIXER_KEYS[kind], what + " mixer")
        for key in _MIXER_KEYS[kind]:
            if key not in ("scale", "mask", "rot"):
                as_int(m, key, 1)
        if kind != "mingru":
            as_float(m, "scale")
        if kind != "mingru" and m.get("mask") is not None:      # no mask: every earlier key is seen
            if not isinstance(m["mask"], dict) or "size" not in m["mask"]:
                raise ConfigError(f"{what}: mask must be an object with size")
            as_int(m["mask"], "size", 1)
        if kind == "latent_attention_2":
            if not isinstance(m["rot"], dict):
                raise ConfigError(f"{what}: rot must be an object with base and dims")
            require_keys(m["rot"], ["base", "dims"], what + " rot")
            dims = as_int(m["rot"], "dims", 2)
            if dims % 2 or dims > m["rot_dim"] or as_float(m["rot"], "base") <= 0:
                raise ConfigError(f"{what}: rot.dims must be even and at most rot_dim, rot.base positive")
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"{what}: mlp is null or an object of kind dense")
            as_int(mlp, "ff", 1)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PufuzenConfig":
        require_keys(raw, ["vocab", "width", "layers", "norm"], ARCHITECTURE)      # no logit_scale: 1
        return cls(copy.deepcopy(raw))

    def to_dict(self) -> Dict[str, Any]:
        out = copy.deepcopy(self.raw)
        out.pop("architectures", None)
        out["architecture"] = ARCHITECTURE
        return out

    def _mixer(self, index: int, layer: Dict[str, Any]) -> PartSpec:
        m, prefix = layer["mixer"], f"l{index}.mix"
        if layer["type"] == "mingru":
            return PartSpec("min_gru", {"hidden_size": self.width, "width": m["width"]}, prefix)
        params = {"hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                  "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": self.eps}
        # a query sees itself and the mask.size - 1 keys before it
        window = int(m["mask"]["size"]) - 1 if m.get("mask") is not None else None
        if layer["type"] == "latent_attention":
            params.update(rot_dim=0, window=window, sink=False, position=None)
        else:
            params.update(rot_dim=m["rot_dim"], window=window, sink=True,
                          position=PartSpec("rope_interleaved", {"base": float(m["rot"]["base"]),
                                                                 "dims": int(m["rot"]["dims"])}))
        return PartSpec("latent_attention", params, prefix)

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm", {"size": self.width, "eps": self.eps})
        gate = PartSpec("residual_gate", {"hidden_size": self.width})
        layers = []
        for index, layer in enumerate(self.layers):
            p = f"l{index}"
            parts = dict(mixer=self._mixer(index, layer),
                         mixer_norm=PartSpec("rms_norm", dict(norm.params, tensor=p + ".norm1"), p),
                         mixer_gate=gate.with_prefix(p + ".rg1"))
            if layer.get("mlp") is None:
                layers.append(LayerSpec("gated_pre_norm_mixer_only", **parts))
                continue
            parts.update(
                feed_forward=PartSpec("poly_norm_mlp", {"hidden_size": self.width, "inner_size": layer["mlp"]["ff"],
                                                        "eps": self.eps}, p + ".mlp"),
                feed_forward_norm=PartSpec("rms_norm", dict(norm.params, tensor=p + ".norm2"), p),
                feed_forward_gate=gate.with_prefix(p + ".rg2"))
            layers.append(LayerSpec("gated_pre_norm_residual", **parts))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "tensor": "embed"}, "embed"),
            layers=tuple(layers), order=tuple(LayerCall(i) for i in range(len(layers))),
            # logits = head(norm(x)) * logit_scale: the constant rides in the final norm's gain
            final_norm=PartSpec("rms_norm", dict(norm.params, tensor="final.norm", gain_scale=self.logit_scale),
                                "final"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": None,
                                      "tensor": "head"}, "head"))
        spec.validate()
        return spec


register_architecture(ARCHITECTURE, PufuzenConfig)
