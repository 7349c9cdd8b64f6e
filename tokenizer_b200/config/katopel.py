"""Typed configuration of the Katopel decoder: a small decoder-only model whose layers mix tokens
with the gated delta rule (a linear recurrence over a matrix state per head) or with two mixers
side by side (grouped-query attention inside chunks of positions, and the gated delta rule), with
a layer norm in front of and behind every sublayer, a gated feed-forward that is dense or made of
routed experts with a shared one, a stack of layers that may run several times in a row with the
same weights, a scaled embedding and logits from the embedding table itself.

config.json keys: `architecture` ("Katopel"), `vocab`, `width`, `embedding.scale`, `norm.eps`,
`loop` {start, stop, times} (optional: layers start .. stop - 1 run `times` times; each pass has
caches and states of its own; before every pass but the first the embedding's output is added to
the stream, and before every pass row t of `loop.step`), and `layers`: a list of {`type`, `mixer`,
`mlp`}.
  type "delta":     mixer {heads, kv_heads, dim, vdim, conv}
  type "parallel":  mixer {left {heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims}},
                           right {heads, kv_heads, dim, vdim, conv}, left_scale, right_scale}
                    (no `mask`: every earlier key is seen; no `rot`: no rotation)
  mlp: null, {kind "dense", ff} or {kind "moe", expert {ff}, router {experts, top}, shared {ff} (optional)}
Tensors: `embed`, `loop.step`, `l<i>.norm1`, `.norm1b`, `.norm2`, `.norm2b` (+ `.b`), `l<i>.mix.*`,
`l<i>.mlp.*`, `final.norm` (+ `.b`).  Every size is read here; none stands in the parts.
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional

from .registry import register_architecture
from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec, as_float, as_int, require_keys

ARCHITECTURE = "Katopel"
# The design has no longest position (angles are computed, not tabulated); what the engine uses
# as its bound on a request's length.
POSITIONS = 1 << 20


def _object(raw: Dict[str, Any], key: str, what: str) -> Dict[str, Any]:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"{what}: {key} must be an object")
    return value


class KatopelConfig:
    def __init__(self, raw: Dict[str, Any]):
        self.raw = raw
        self.vocab = as_int(raw, "vocab", 1)
        self.width = as_int(raw, "width", 1)
        self.eps = as_float(_object(raw, "norm", ARCHITECTURE), "eps")
        if self.eps < 0:
            raise ConfigError("norm.eps must not be negative")
        embedding = raw.get("embedding")
        self.embedding_scale = as_float(embedding, "scale") if isinstance(embedding, dict) and "scale" in embedding else 1.0
        self.layers: List[Dict[str, Any]] = raw["layers"]
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json layers must be a list with at least one layer")
        for index, layer in enumerate(self.layers):
            self._check_layer(index, layer)
        self.loop: Optional[Dict[str, int]] = None
        if raw.get("loop") is not None:
            loop = _object(raw, "loop", ARCHITECTURE)
            require_keys(loop, ["start", "stop", "times"], ARCHITECTURE + " loop")
            start, stop, times = as_int(loop, "start", 0), as_int(loop, "stop", 0), as_int(loop, "times", 1)
            if stop > len(self.layers) or start > stop:
                raise ConfigError(f"loop {start} .. {stop} does not lie inside the {len(self.layers)} layers")
            if stop > start:
                self.loop = {"start": start, "stop": stop, "times": times}

    # ---- checks ------------------------------------------------------------------------------
    @staticmethod
    def _check_delta(m: Dict[str, Any], what: str) -> None:
        require_keys(m, ["heads", "kv_heads", "dim", "vdim", "conv"], what)
        for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
            as_int(m, key, 1)
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{what}: {m['heads']} heads do not divide into {m['kv_heads']} kv_heads")

    @staticmethod
    def _check_attention(m: Dict[str, Any], what: str) -> None:
        require_keys(m, ["heads", "kv_heads", "dim", "vdim", "scale"], what)
        for key in ("heads", "kv_heads", "dim", "vdim"):
            as_int(m, key, 1)
        as_float(m, "scale")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{what}: {m['heads']} heads do not divide into {m['kv_heads']} kv_heads")
        if m.get("mask") is not None:
            as_int(_object(m, "mask", what), "size", 1)
        if m.get("rot") is not None:
            rot = _object(m, "rot", what)
            require_keys(rot, ["base", "dims"], what + " rot")
            dims = as_int(rot, "dims", 2)
            if dims % 2 or dims > m["dim"] or as_float(rot, "base") <= 0:
                raise ConfigError(f"{what}: rot.dims must be even and at most dim, rot.base positive")

    @classmethod
    def _check_layer(cls, index: int, layer: Dict[str, Any]) -> None:
        what = f"{ARCHITECTURE} layer {index}"
        if not isinstance(layer, dict):
            raise ConfigError(f"{what} must be an object")
        require_keys(layer, ["type", "mixer"], what)
        m = _object(layer, "mixer", what)
        if layer["type"] == "delta":
            cls._check_delta(m, what + " mixer")
        elif layer["type"] == "parallel":
            require_keys(m, ["left", "right", "left_scale", "right_scale"], what + " mixer")
            cls._check_attention(_object(m, "left", what), what + " mixer.left")
            cls._check_delta(_object(m, "right", what), what + " mixer.right")
            as_float(m, "left_scale")
            as_float(m, "right_scale")
        else:
            raise ConfigError(f"{what}: unknown type {layer['type']!r} (known: delta, parallel)")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
            raise ConfigError(f"{what}: mlp is null or an object of kind dense or moe")
        if mlp["kind"] == "dense":
            as_int(mlp, "ff", 1)
            return
        as_int(_object(mlp, "expert", what + " mlp"), "ff", 1)
        router = _object(mlp, "router", what + " mlp")
        require_keys(router, ["experts", "top"], what + " mlp.router")
        if as_int(router, "top", 1) > as_int(router, "experts", 1):
            raise ConfigError(f"{what}: a token cannot use {router['top']} of {router['experts']} experts")
        if mlp.get("shared") is not None:
            as_int(_object(mlp, "shared", what + " mlp"), "ff", 1)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "KatopelConfig":
        require_keys(raw, ["vocab", "width", "layers", "norm"], ARCHITECTURE)
        return cls(copy.deepcopy(raw))

    def to_dict(self) -> Dict[str, Any]:
        out = copy.deepcopy(self.raw)
        out.pop("architectures", None)
        out["architecture"] = ARCHITECTURE
        return out

    # ---- the model as data -------------------------------------------------------------------
    def _delta(self, m: Dict[str, Any], prefix: str) -> PartSpec:
        return PartSpec("gated_delta_net", {"hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"],
                                            "dim": m["dim"], "vdim": m["vdim"], "conv": m["conv"], "eps": self.eps},
                        prefix)

    def _attention(self, m: Dict[str, Any], prefix: str) -> PartSpec:
        position = None
        if m.get("rot") is not None:
            position = PartSpec("rope_interleaved", {"base": float(m["rot"]["base"]), "dims": int(m["rot"]["dims"])})
        return PartSpec("gqa_rotary", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
            "vdim": m["vdim"], "scale": float(m["scale"]), "bias": True, "window": None,
            "chunk": int(m["mask"]["size"]) if m.get("mask") is not None else None, "position": position}, prefix)

    def _mixer(self, index: int, layer: Dict[str, Any]) -> PartSpec:
        m, prefix = layer["mixer"], f"l{index}.mix"
        if layer["type"] == "delta":
            return self._delta(m, prefix)
        return PartSpec("parallel_mixers", {"left": self._attention(m["left"], prefix + ".left"),
                                            "right": self._delta(m["right"], prefix + ".right"),
                                            "left_scale": float(m["left_scale"]),
                                            "right_scale": float(m["right_scale"])}, prefix)

    def _feed_forward(self, index: int, mlp: Dict[str, Any]) -> PartSpec:
        prefix = f"l{index}.mlp"
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "silu",
                                          "names": (".gate", ".up", ".down")}, prefix)
        shared = mlp.get("shared")
        return PartSpec("routed_mlp", {"hidden_size": self.width, "experts": mlp["router"]["experts"],
                                       "top": mlp["router"]["top"], "expert_inner": mlp["expert"]["ff"],
                                       "shared_inner": shared["ff"] if shared is not None else 0,
                                       "activation": "silu"}, prefix)

    def _norm(self, name: str) -> PartSpec:
        return PartSpec("layer_norm", {"size": self.width, "eps": self.eps, "tensor": name}, name)

    def run_order(self) -> List[LayerCall]:
        """The calls of the layers: those before the loop, the looped ones `times` times (each call
        with a cache and state of its own), the rest.  A pass's first call carries what the pass
        adds to the stream."""
        n = len(self.layers)
        if self.loop is None:
            return [LayerCall(i) for i in range(n)]
        start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order = [LayerCall(i) for i in range(start)]
        for t in range(times):
            entry = PartSpec("pass_entry", {"tensor": "loop.step", "passes": times, "hidden_size": self.width,
                                            "index": t, "add_embedding": t > 0}, "loop")
            order += [LayerCall(i, before=entry if i == start else None) for i in range(start, stop)]
        return order + [LayerCall(i) for i in range(stop, n)]

    def model_spec(self) -> ModelSpec:
        layers = []
        for index, layer in enumerate(self.layers):
            p = f"l{index}"
            parts = dict(mixer=self._mixer(index, layer), mixer_norm=self._norm(p + ".norm1"),
                         mixer_post_norm=self._norm(p + ".norm1b"))
            if layer.get("mlp") is None:
                layers.append(LayerSpec("sandwich_norm_mixer_only", **parts))
                continue
            parts.update(feed_forward=self._feed_forward(index, layer["mlp"]),
                         feed_forward_norm=self._norm(p + ".norm2"), feed_forward_post_norm=self._norm(p + ".norm2b"))
            layers.append(LayerSpec("sandwich_norm_residual", **parts))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "tensor": "embed", "scale": self.embedding_scale}, "embed"),
            layers=tuple(layers), order=tuple(self.run_order()), final_norm=self._norm("final.norm"),
            # logits = embed x: the table itself, without the embedding's scale
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": "embed"}, "head"))
        spec.validate()
        return spec


register_architecture(ARCHITECTURE, KatopelConfig)
