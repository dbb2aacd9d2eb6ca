"""Typed configuration of the Letanex decoder, read from its config.json.

config.json: ``architecture`` ("Letanex"), ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list whose entries give
``type`` and the sizes of that mixer (``mixer``) and the feed-forward (``mlp``, or null for none):

* ``attention``: differential attention with grouped key/value heads: ``heads``, ``kv_heads``, ``dim``, ``vdim``,
  ``scale``, ``diff``, ``rot`` = {``base``, ``dims``[, ``scaling``: {``factor``}]} (half-split pairs over the first
  ``dims`` elements of each map, frequencies divided by the factor), optionally ``kv_from``: the layer whose cached
  keys and values this layer reads with queries of its own;
* ``lightning``: linear attention with a decay per head and a state per request: ``heads``, ``dim``, ``vdim``, ``decay``.

``mlp``: {``kind``: "dense", ``ff``} (squared ReLU), or {``kind``: "moe", ``router``: {``experts``, ``identity``, ``top``,
``scale``}, ``expert``: {``ff``, ``limit``}[, ``shared``: {``ff``, ``limit``}]}.  Every size and constant comes from the
file; only ``max_positions`` (the rotary tables' length) has a default.

The model: token embedding; per layer x += norm1b(mixer(norm1(x))), x += norm2b(ffn(norm2(x))) with layer norms that
have a weight and no bias; a final norm and the head.  Tensor names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Any, Mapping

from .specs import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec

DEFAULT_MAX_POSITIONS = 65536
MIXER_TYPES = ("attention", "lightning")
GLU_ALPHA = 1.702              # the experts' activation g * sigmoid(1.702 g): fixed by the design


def _is_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def _number(value) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)


def _positive_int(raw: Mapping, key: str, where: str) -> int:
    value = raw.get(key)
    if not _is_int(value) or value <= 0:
        raise ConfigError(f"Invalid Letanex config: {where}.{key} must be a positive integer.")
    return value


def _positive(raw: Mapping, key: str, where: str) -> float:
    value = raw.get(key)
    if not _number(value) or value <= 0:
        raise ConfigError(f"Invalid Letanex config: {where}.{key} must be a positive number.")
    return float(value)


def _parse_mixer(index: int, kind: str, m: Mapping) -> dict:
    where = f"layers[{index}].mixer"
    out = {"heads": _positive_int(m, "heads", where), "dim": _positive_int(m, "dim", where),
           "vdim": _positive_int(m, "vdim", where)}
    if kind == "lightning":
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != out["heads"] or not all(_number(d) and d >= 0 for d in decay):
            raise ConfigError(f"Invalid Letanex config: {where}.decay must list one non-negative number per head.")
        out["decay"] = [float(d) for d in decay]
        return out
    out["kv_heads"] = _positive_int(m, "kv_heads", where)
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"Invalid Letanex config: {where}.heads must be a multiple of kv_heads.")
    out["scale"] = _positive(m, "scale", where)
    diff = m.get("diff")
    if not _number(diff):
        raise ConfigError(f"Invalid Letanex config: {where}.diff must be a number.")
    out["diff"] = float(diff)
    rot = m.get("rot")
    if not isinstance(rot, Mapping):
        raise ConfigError(f"Invalid Letanex config: {where}.rot is missing.")
    dims = rot.get("dims")
    if not _is_int(dims) or dims < 0 or dims % 2 or dims > out["dim"]:
        raise ConfigError(f"Invalid Letanex config: {where}.rot.dims must be even and at most dim.")
    parsed = {"base": _positive(rot, "base", where + ".rot"), "dims": dims}
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, Mapping):
            raise ConfigError(f"Invalid Letanex config: {where}.rot.scaling must be an object.")
        parsed["scaling"] = {"factor": _positive(scaling, "factor", where + ".rot.scaling")}
    out["rot"] = parsed
    kv_from = m.get("kv_from")
    if kv_from is not None:
        if not _is_int(kv_from) or not 0 <= kv_from < index:
            raise ConfigError(f"Invalid Letanex config: {where}.kv_from must name an earlier layer.")
        out["kv_from"] = kv_from
    return out


def _parse_mlp(index: int, mlp) -> dict | None:
    where = f"layers[{index}].mlp"
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"Invalid Letanex config: {where} must be null or of kind 'dense' or 'moe'.")
    if mlp["kind"] == "dense":
        return {"kind": "dense", "ff": _positive_int(mlp, "ff", where)}
    router, expert, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
    if not isinstance(router, Mapping):
        raise ConfigError(f"Invalid Letanex config: {where}.router is missing.")
    experts, identity = router.get("experts"), router.get("identity", 0)
    if not _is_int(experts) or not _is_int(identity) or experts < 0 or identity < 0 or experts + identity == 0:
        raise ConfigError(f"Invalid Letanex config: {where}.router needs non-negative experts and identity, not both zero.")
    top = _positive_int(router, "top", where + ".router")
    if top > experts + identity:
        raise ConfigError(f"Invalid Letanex config: {where}.router.top exceeds the number of experts.")
    out = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top,
                                     "scale": _positive(router, "scale", where + ".router")}}
    if experts:
        if not isinstance(expert, Mapping):
            raise ConfigError(f"Invalid Letanex config: {where}.expert is missing.")
        out["expert"] = {"ff": _positive_int(expert, "ff", where + ".expert"), "limit": _positive(expert, "limit", where + ".expert")}
    elif isinstance(expert, Mapping):
        out["expert"] = dict(expert)
    if shared is not None:
        if not isinstance(shared, Mapping):
            raise ConfigError(f"Invalid Letanex config: {where}.shared must be an object.")
        out["shared"] = {"ff": _positive_int(shared, "ff", where + ".shared"), "limit": _positive(shared, "limit", where + ".shared")}
    return out


@dataclass(frozen=True)
class LetanexLayer:
    type: str
    mixer: dict
    mlp: dict | None

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer, "mlp": self.mlp}


@dataclass(frozen=True)
class LetanexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    architecture = "Letanex"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LetanexConfig":
        if not isinstance(raw, Mapping) or raw.get("architecture") != cls.architecture:
            raise ConfigError("Invalid Letanex config.")
        vocab, width = _positive_int(raw, "vocab", "config"), _positive_int(raw, "width", "config")
        if not isinstance(raw.get("norm"), Mapping):
            raise ConfigError("Invalid Letanex config: norm is missing.")
        eps = _positive(raw["norm"], "eps", "config.norm")
        if not isinstance(raw.get("layers"), list) or not raw["layers"]:
            raise ConfigError("Invalid Letanex config: layers must be a non-empty list.")
        layers = []
        for index, layer in enumerate(raw["layers"]):
            if not isinstance(layer, Mapping) or layer.get("type") not in MIXER_TYPES or not isinstance(layer.get("mixer"), Mapping):
                raise ConfigError(f"Invalid Letanex config: layers[{index}] needs a type of {', '.join(MIXER_TYPES)} and a mixer.")
            layers.append(LetanexLayer(layer["type"], _parse_mixer(index, layer["type"], layer["mixer"]),
                                       _parse_mlp(index, layer.get("mlp"))))
        for index, layer in enumerate(layers):
            source = layer.mixer.get("kv_from")
            if source is None:
                continue
            other = layers[source]
            keys = ("kv_heads", "dim", "vdim", "rot")
            if other.type != "attention" or "kv_from" in other.mixer or any(other.mixer[k] != layer.mixer[k] for k in keys):
                raise ConfigError(f"Invalid Letanex config: layers[{index}].mixer.kv_from must name an attention layer with "
                                  "projections of its own and this layer's key/value heads, sizes and rotation.")
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_positions) or max_positions <= 0:
            raise ConfigError("Invalid Letanex config: max_positions must be a positive integer.")
        eos_ids = ()
        if raw.get("eos_token_id") is not None:
            from .qwen2 import parse_eos_ids
            eos_ids = parse_eos_ids(raw["eos_token_id"], vocab)
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers), max_positions=max_positions, eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def with_eos(self, eos_token_id) -> "LetanexConfig":
        from .qwen2 import parse_eos_ids
        return replace(self, eos_token_ids=parse_eos_ids(eos_token_id, self.vocab))

    def _mixer_spec(self, layer: LetanexLayer) -> PartSpec:
        m = layer.mixer
        if layer.type == "lightning":
            return PartSpec("decay_linear_attention", {
                "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "value_dim": m["vdim"], "decay": tuple(m["decay"]),
                "eps": self.norm_eps, "activation": "silu",
                "names": {key: "mix." + key for key in ("q", "k", "v", "g", "o", "norm")}})
        rot = m["rot"]
        position = PartSpec("none", {})
        if rot["dims"]:
            position = PartSpec("rope_linear", {"dims": rot["dims"], "theta": rot["base"], "max_positions": self.max_positions,
                                                "factor": (rot.get("scaling") or {}).get("factor", 1.0)})
        return PartSpec("multimap_attention", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "value_dim": m["vdim"],
            "scale": m["scale"], "position": position, "maps": 2, "diff": m["diff"], "norm_eps": self.norm_eps,
            "out_scale": 1.0 - m["diff"], "own_kv": "kv_from" not in m,
            "names": {key: "mix." + key for key in ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2")}})

    def _mlp_spec(self, mlp: dict | None) -> PartSpec:
        if mlp is None:
            return PartSpec("none", {})
        if mlp["kind"] == "dense":
            return PartSpec("relu2_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                          "names": {"up": "mlp.up", "down": "mlp.down"}})
        router, expert, shared = mlp["router"], mlp.get("expert") or {}, mlp.get("shared")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "experts": router["experts"], "identity": router["identity"], "top": router["top"],
            "scale": router["scale"], "expert_ff": expert.get("ff", 0), "expert_limit": expert.get("limit", 0.0), "alpha": GLU_ALPHA,
            "shared_ff": shared["ff"] if shared else None, "shared_limit": shared["limit"] if shared else None,
            "names": {"router": "mlp.router", "correction": "mlp.correction", "expert": "mlp.e{}.", "shared": "mlp.shared."}})

    def model_spec(self) -> ModelSpec:
        norm = {"size": self.width, "eps": self.norm_eps, "suffix": ""}
        layers, order = [], []
        slot_of: dict[int, int] = {}
        slots = 0
        for index, layer in enumerate(self.layers):
            names = ("norm1", "norm1b") + (("norm2", "norm2b") if layer.mlp is not None else ())
            norms = tuple(PartSpec("layernorm", {**norm, "name": name}) for name in names)
            layers.append(LayerSpec("sandwich_norm", f"l{index}.", self._mixer_spec(layer), self._mlp_spec(layer.mlp), norms))
            source = layer.mixer.get("kv_from")
            if source is not None:
                order.append(LayerCall(layer=index, cache=slot_of[source], writes_cache=False))
            else:
                # every layer call names a cache slot; a mixer that keeps nothing per token gets a slot without buffers
                slot_of[index] = slots
                order.append(LayerCall(layer=index, cache=slots, writes_cache=True))
                slots += 1
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "embed", "suffix": ""}),
            layers=tuple(layers), order=tuple(order),
            final_norm=PartSpec("layernorm", {**norm, "name": "final.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "head", "suffix": "",
                                      "any_inner_size": True}),
            eos_token_ids=self.eos_token_ids)
