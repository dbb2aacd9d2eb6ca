"""Tiny Letanex configurations and model folders for the tests.

The first two configurations differ in every size and constant and avoid choices that would hide a mix-up: query/key
and value sizes of a head differ in one and are equal in the other, one has as many key/value heads as heads, the
rotated width is smaller than a map's vectors, one rotation has no scaling, one decay is exactly 1, one router takes
a single expert and another nearly all, one mixture has no identity experts and one no shared expert, one layer has
no feed-forward, each has a layer that reads another layer's keys and values, and each starts with another mixer.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

import plain_letanex as plain


def attention(heads, kv_heads, dim, vdim, scale, diff, base, dims, factor=None, kv_from=None):
    rot = {"base": base, "dims": dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff, "rot": rot}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return "attention", mixer


def lightning(heads, dim, vdim, decay):
    return "lightning", {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, scale, ff, limit, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top, "scale": scale},
           "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


P = {"architecture": "Letanex", "vocab": 301, "width": 72, "norm": {"eps": 1e-5},
     "layers": [
         layer(lightning(3, 8, 20, (0.9, 0.5, 0.99)), moe(5, 2, 2, 2.0, 24, 1.0, shared=(40, 3.0))),
         layer(attention(6, 2, 16, 24, 0.3, 0.3, 500.0, 8, factor=4.0), dense(100)),
         layer(attention(4, 2, 16, 24, 0.2, 0.6, 500.0, 8, factor=4.0, kv_from=1), None),
         layer(lightning(1, 24, 8, (1.0,)), moe(3, 0, 1, 1.0, 16, 0.5)),
         layer(attention(2, 1, 12, 40, 0.25, 0.8, 90000.0, 12), moe(4, 3, 5, 0.7, 8, 2.5, shared=(16, 1.0))),
     ]}
Q = {"architecture": "Letanex", "vocab": 255, "width": 64, "norm": {"eps": 1e-6},
     "layers": [
         layer(attention(3, 3, 8, 8, 0.4, 0.1, 10000.0, 4, factor=1.5), moe(4, 1, 4, 1.5, 32, 1.5, shared=(24, 2.0))),
         layer(lightning(2, 16, 16, (0.7, 0.95)), dense(48)),
         layer(attention(6, 3, 8, 8, 0.5, 0.45, 10000.0, 4, factor=1.5, kv_from=0), moe(6, 2, 3, 1.0, 16, 1.0)),
     ]}
# sizes that the tensor-core kernels of the bfloat16 path are built for (key vectors of 16 and 64 with values of 32 and 64,
# a recurrent state with keys of 64, experts in multiples of 8)
R = {"architecture": "Letanex", "vocab": 277, "width": 96, "norm": {"eps": 1e-5},
     "layers": [
         layer(lightning(2, 64, 32, (0.9, 0.99)), moe(6, 1, 2, 1.2, 32, 1.5, shared=(48, 2.0))),
         layer(attention(4, 1, 16, 32, 0.35, 0.4, 2000.0, 8, factor=2.0), dense(160)),
         layer(attention(2, 1, 16, 32, 0.3, 0.7, 2000.0, 8, factor=2.0, kv_from=1), moe(4, 0, 2, 1.0, 64, 1.0)),
         layer(attention(2, 2, 64, 64, 0.2, 0.5, 50000.0, 64), None),
     ]}
CONFIGS = {"P": (P, 3, 16), "Q": (Q, 4, 8), "R": (R, 5, 16)}            # name -> (config.json, seed, page size)
MIXER_SCALE = {"P": 3.0, "Q": 3.0, "R": 1.5}       # R's long key vectors make sharp scores already


def make_model_dir(base, name: str) -> Path:
    """A folder written by the package's random-weights mode, then made harder: the mixers' matrices are scaled up so
    that they are a large share of the stream (a wrong key or a lost state must move the logits), the routers'
    matrices so that a token's scores are nearly one-hot, and the corrections are steps of 0.4 in shuffled order: the
    taken experts are the token's winner and those the corrections favour, and few choices are close calls (the
    mechanism's own test routes with moderate scores)."""
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.weights import write_random_model, write_safetensors
    from sprout_lm_b200.weights.safetensors_io import SafetensorsFile
    raw, seed, _ = CONFIGS[name]
    directory = write_random_model(Path(base) / f"letanex_{name}", parse_config(raw), seed=seed)
    rng = np.random.default_rng(seed)
    tensors = {}
    handle = SafetensorsFile(directory / "model.safetensors")
    try:
        for key in handle.names():
            value = handle.tensor(key).float()
            if ".mix." in key and value.dim() == 2:
                value = value * MIXER_SCALE[name]
            elif key.endswith(".router"):
                value = value * 100.0               # decisive scores: few nearly tied choices for bfloat16 to fall either way
            elif key.endswith(".correction"):
                value = torch.from_numpy((rng.permutation(value.numel()) * 0.4).astype(np.float32))
            elif ".mlp." in key and value.dim() == 2:
                value = value * 4.0
            elif key == "head":
                value = value * 5.0                 # logits of order one
            tensors[key] = value.to(torch.bfloat16)
    finally:
        handle.close()
    write_safetensors(directory / "model.safetensors", tensors, metadata={"format": "pt"})
    return directory


_models: dict = {}
_logits: dict = {}


def plain_model(directory):
    key = str(directory)
    if key not in _models:
        _models[key] = plain.read_model_folder(directory)
    return _models[key]


def plain_logits(directory, tokens) -> np.ndarray:
    key = (str(directory), tuple(tokens))
    if key not in _logits:
        _logits[key] = plain.logits(*plain_model(directory), list(tokens))
    return _logits[key]


def compare(directory, requests: dict, got: dict, tol: float, label: str, page: int, outliers: float = 0.0):
    """Every place that came back against the oracle, by the root mean square of the difference over the vocabulary
    (the logits' own root mean square is near one); a failure names the first wrong token and its place.
    ``outliers``: the share of places that may lie over the bar.  In 32-bit no place may differ.  In bfloat16 a
    router's nearly tied choice sometimes falls the other way (some ten times among these requests' tokens), and what
    that changes stays in the recurrent state and the cached values of the request's later tokens; so there the bar
    holds for the median (at half its height) and for three quarters of the places, which a fault of a kernel's
    indexing or dispatch would move, while keys at borders, far keys and carried state are held to tight bars in
    bfloat16 by the mechanisms' own tests, where nothing is routed."""
    assert got, "no logits came back"
    errors, first = [], None
    for rid, tokens in requests.items():
        want = plain_logits(directory, tokens)
        for pos in range(len(tokens)):
            if (rid, pos) not in got:
                continue
            err = float(np.sqrt(np.mean((got[(rid, pos)] - want[pos]) ** 2)))
            errors.append(err)
            if (not np.isfinite(err) or err > tol) and first is None:
                first = (f"{label}: request {rid} position {pos} of {len(tokens)} (position % {page} = {pos % page}, "
                         f"% 128 = {pos % 128}) differs by {err:.3e} > {tol}")
    errors = np.asarray(errors)
    over = int(np.sum(~(errors <= tol)))
    if over > outliers * len(errors):
        raise AssertionError(f"{first}; {over} of {len(errors)} places are over the bar")
    if outliers:
        assert np.median(errors) <= tol / 2, f"{label}: the median difference {np.median(errors):.3e} is over half the bar"
    return float(errors.max())
