"""Typed configuration of the Tulipel decoder, read from its config.json.

config.json: ``architecture`` ("Tulipel"), ``vocab``, ``width``, ``postln_alpha``, ``logit_softcap``,
``norm.eps`` and ``layers``, a list whose entries give ``type`` (``latent_attention``: queries through a
latent of rank ``q_rank``, interleaved rotary pairs; ``latent_attention_2``: queries straight from the
stream, half-split pairs, frequencies stretched as ``rot.scaling`` says), the mixer's sizes (``mixer``:
``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``rot`` = {``base``, ``dims``[, ``scaling``]},
optionally ``kv_from``: the layer whose cached rows this layer reads) and its feed-forward (``mlp``:
{``kind``: "dense", ``ff``} or null).  Every size and constant comes from there; nothing has a default
except ``max_positions`` (the length of the rotary tables), which the file need not give.

The model: token embedding; per layer x <- norm1(alpha x + mixer(x)), x <- norm2(alpha x + ffn(x)) with
RMS norms whose weights are stored around zero (gain 1 + w); after layer i the stream becomes
sum_j dwa_i[j] X_j over the embedding's output X_0 and the layers' results X_1..X_(i+1); a final norm, the
head, and logits <- softcap * tanh(logits / softcap).  Tensor names: ``embed``, ``l<i>.norm1|norm2``,
``l<i>.mix.*``, ``l<i>.mlp.up|down|act``, ``l<i>.dwa``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Any, Mapping

from .specs import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec

DEFAULT_MAX_POSITIONS = 65536
MIXER_TYPES = ("latent_attention", "latent_attention_2")


def _is_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def _number(value) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)


def _positive_int(raw: Mapping, key: str, where: str) -> int:
    value = raw.get(key)
    if not _is_int(value) or value <= 0:
        raise ConfigError(f"Invalid Tulipel config: {where}.{key} must be a positive integer.")
    return value


def _positive(raw: Mapping, key: str, where: str) -> float:
    value = raw.get(key)
    if not _number(value) or value <= 0:
        raise ConfigError(f"Invalid Tulipel config: {where}.{key} must be a positive number.")
    return float(value)


@dataclass(frozen=True)
class TulipelLayer:
    type: str
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: tuple | None          # (factor, original, fast, slow)
    q_rank: int | None
    kv_from: int | None
    ff: int | None                     # None: no feed-forward

    def to_dict(self) -> dict:
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.rot_scaling))
        mixer = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                 "scale": self.scale, "rot": rot}
        if self.q_rank is not None:
            mixer["q_rank"] = self.q_rank
        if self.kv_from is not None:
            mixer["kv_from"] = self.kv_from
        return {"type": self.type, "mixer": mixer, "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


def _parse_layer(index: int, raw) -> TulipelLayer:
    where = f"layers[{index}]"
    if not isinstance(raw, Mapping) or raw.get("type") not in MIXER_TYPES or not isinstance(raw.get("mixer"), Mapping):
        raise ConfigError(f"Invalid Tulipel config: {where} needs a type of {', '.join(MIXER_TYPES)} and a mixer.")
    m = raw["mixer"]
    kind = raw["type"]
    heads, vdim, kv_rank = (_positive_int(m, key, where + ".mixer") for key in ("heads", "vdim", "kv_rank"))
    dim, rot_dim = m.get("dim"), m.get("rot_dim")
    if not _is_int(dim) or not _is_int(rot_dim) or dim < 0 or rot_dim < 0 or dim + rot_dim == 0:
        raise ConfigError(f"Invalid Tulipel config: {where}.mixer needs non-negative dim and rot_dim, not both zero.")
    scale = _positive(m, "scale", where + ".mixer")
    rot = m.get("rot")
    rot_base, rot_dims, rot_scaling = 10000.0, 0, None
    if rot_dim:
        if not isinstance(rot, Mapping):
            raise ConfigError(f"Invalid Tulipel config: {where}.mixer.rot is missing.")
        rot_base = _positive(rot, "base", where + ".mixer.rot")
        rot_dims = _positive_int(rot, "dims", where + ".mixer.rot")
        if rot_dims % 2 or rot_dims > rot_dim or rot_base <= 1:
            raise ConfigError(f"Invalid Tulipel config: {where}.mixer.rot.dims must be even and at most rot_dim, base above 1.")
        scaling = rot.get("scaling")
        if kind == "latent_attention_2" and scaling is not None:
            if not isinstance(scaling, Mapping):
                raise ConfigError(f"Invalid Tulipel config: {where}.mixer.rot.scaling must be an object.")
            rot_scaling = tuple(_positive(scaling, key, where + ".mixer.rot.scaling") for key in ("factor", "original", "fast", "slow"))
    q_rank = None
    if kind == "latent_attention":
        q_rank = _positive_int(m, "q_rank", where + ".mixer")
    kv_from = m.get("kv_from")
    if kv_from is not None and (not _is_int(kv_from) or not 0 <= kv_from < index):
        raise ConfigError(f"Invalid Tulipel config: {where}.mixer.kv_from must name an earlier layer.")
    mlp = raw.get("mlp")
    ff = None
    if mlp is not None:
        if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
            raise ConfigError(f"Invalid Tulipel config: {where}.mlp must be null or of kind 'dense'.")
        ff = _positive_int(mlp, "ff", where + ".mlp")
    return TulipelLayer(type=kind, heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
                        rot_base=rot_base, rot_dims=rot_dims, rot_scaling=rot_scaling, q_rank=q_rank, kv_from=kv_from, ff=ff)


@dataclass(frozen=True)
class TulipelConfig:
    vocab: int
    width: int
    postln_alpha: float
    logit_softcap: float
    norm_eps: float
    layers: tuple
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    architecture = "Tulipel"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TulipelConfig":
        if not isinstance(raw, Mapping) or raw.get("architecture") != cls.architecture:
            raise ConfigError("Invalid Tulipel config.")
        vocab, width = _positive_int(raw, "vocab", "config"), _positive_int(raw, "width", "config")
        alpha = raw.get("postln_alpha")
        if not _number(alpha):
            raise ConfigError("Invalid Tulipel config: postln_alpha must be a number.")
        softcap = _positive(raw, "logit_softcap", "config")
        if not isinstance(raw.get("norm"), Mapping):
            raise ConfigError("Invalid Tulipel config: norm is missing.")
        eps = _positive(raw["norm"], "eps", "config.norm")
        if not isinstance(raw.get("layers"), list) or not raw["layers"]:
            raise ConfigError("Invalid Tulipel config: layers must be a non-empty list.")
        layers = tuple(_parse_layer(i, layer) for i, layer in enumerate(raw["layers"]))
        for i, layer in enumerate(layers):
            if layer.kv_from is None:
                continue
            source = layers[layer.kv_from]
            same = (source.kv_rank, source.rot_dim, source.rot_dims, source.rot_base, source.rot_scaling, source.type) == \
                   (layer.kv_rank, layer.rot_dim, layer.rot_dims, layer.rot_base, layer.rot_scaling, layer.type)
            if source.kv_from is not None or not same:
                raise ConfigError(f"Invalid Tulipel config: layers[{i}].mixer.kv_from must name a layer that caches rows of "
                                  "its own, with this layer's kv_rank, rot_dim and rotation.")
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_positions) or max_positions <= 0:
            raise ConfigError("Invalid Tulipel config: max_positions must be a positive integer.")
        eos = raw.get("eos_token_id")
        eos_ids = ()
        if eos is not None:
            from .qwen2 import parse_eos_ids
            eos_ids = parse_eos_ids(eos, vocab)
        return cls(vocab=vocab, width=width, postln_alpha=float(alpha), logit_softcap=softcap, norm_eps=eps, layers=layers,
                   max_positions=max_positions, eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "postln_alpha": self.postln_alpha,
               "logit_softcap": self.logit_softcap, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def with_eos(self, eos_token_id) -> "TulipelConfig":
        from .qwen2 import parse_eos_ids
        return replace(self, eos_token_ids=parse_eos_ids(eos_token_id, self.vocab))

    def model_spec(self) -> ModelSpec:
        norm = {"size": self.width, "eps": self.norm_eps, "offset": 1.0, "suffix": ""}
        layers, order, ignorable = [], [], []
        slot_of: dict[int, int] = {}
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}."
            if layer.type == "latent_attention":
                position = PartSpec("rope_interleaved", {"dims": layer.rot_dims, "theta": layer.rot_base,
                                                         "max_positions": self.max_positions})
            else:
                scaling = None if layer.rot_scaling is None else dict(zip(("factor", "original", "fast", "slow"), layer.rot_scaling))
                position = PartSpec("rope_yarn", {"dims": layer.rot_dims, "theta": layer.rot_base,
                                                  "max_positions": self.max_positions, "scaling": scaling})
            if not layer.rot_dim:
                position = PartSpec("none", {})
            mixer = PartSpec("latent_attention", {
                "hidden_size": self.width, "heads": layer.heads, "dim": layer.dim, "rot_dim": layer.rot_dim,
                "value_dim": layer.vdim, "kv_rank": layer.kv_rank, "q_rank": layer.q_rank, "scale": layer.scale,
                "eps": self.norm_eps, "position": position, "own_kv": layer.kv_from is None, "sink": True,
                "names": {key: "mix." + key.replace("_norm", ".norm") for key in
                          ("q", "dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "sink", "o")}})
            norms = [PartSpec("rmsnorm", {**norm, "name": "norm1"})]
            if layer.ff is None:
                ffn = PartSpec("none", {})
                ignorable.append(prefix + "norm2")
            else:
                ffn = PartSpec("polynorm_mlp", {"hidden_size": self.width, "intermediate_size": layer.ff, "eps": self.norm_eps,
                                                "names": {"up": "mlp.up", "down": "mlp.down", "act": "mlp.act"}})
                norms.append(PartSpec("rmsnorm", {**norm, "name": "norm2"}))
            layers.append(LayerSpec("post_norm", prefix, mixer, ffn, tuple(norms), {"alpha": self.postln_alpha}))
            if layer.kv_from is None:
                slot_of[index] = len(slot_of)
                order.append(LayerCall(layer=index, cache=slot_of[index], writes_cache=True))
            else:
                order.append(LayerCall(layer=index, cache=slot_of[layer.kv_from], writes_cache=False))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "embed", "suffix": ""}),
            layers=tuple(layers), order=tuple(order),
            final_norm=PartSpec("rmsnorm", {**norm, "name": "final.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "head", "suffix": "",
                                      "softcap": self.logit_softcap, "any_inner_size": True}),
            eos_token_ids=self.eos_token_ids, ignorable_tensors=tuple(ignorable),
            stream=PartSpec("depth_weighted_average", {"names": tuple(f"l{i}.dwa" for i in range(len(self.layers)))}))
