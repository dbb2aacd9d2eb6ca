"""Tiny Tulipel configurations and model folders for the tests.

The two configurations differ in every size and constant, and neither repeats a choice that would hide a
mix-up: unrotated, rotated and value sizes of a head all differ, the latent is not heads x anything, the
rotated width differs from the number of rotated elements in one layer, alpha is 1 in one and not in the
other, one starts with each kind of mixer, one has a layer without a feed-forward, both have a layer that
reads another layer's cached rows, and Q's sizes are no multiples of 8 or 16.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

import plain_tulipel as plain


def _mixer(heads, dim, rot_dim, vdim, kv_rank, scale, base, dims=None, q_rank=None, kv_from=None, scaling=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if q_rank is not None:
        out["q_rank"] = q_rank
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


P = {"architecture": "Tulipel", "vocab": 301, "width": 72, "postln_alpha": 1.7, "logit_softcap": 12.0, "norm": {"eps": 1e-6},
     "layers": [
         _layer("latent_attention", _mixer(3, 24, 8, 20, 48, 0.2, 5000.0, q_rank=40), 136),
         _layer("latent_attention_2", _mixer(5, 16, 16, 24, 32, 0.15, 30000.0, scaling=(4.0, 64, 16.0, 2.0)), None),
         _layer("latent_attention", _mixer(2, 12, 8, 16, 48, 0.3, 5000.0, q_rank=24, kv_from=0), 72),
         _layer("latent_attention_2", _mixer(1, 8, 24, 8, 16, 0.25, 700.0, dims=16), 40),
         _layer("latent_attention_2", _mixer(4, 8, 16, 12, 32, 0.1, 30000.0, kv_from=1, scaling=(4.0, 64, 16.0, 2.0)), 88),
     ]}
Q = {"architecture": "Tulipel", "vocab": 255, "width": 62, "postln_alpha": 1.0, "logit_softcap": 3.0, "norm": {"eps": 1e-5},
     "layers": [
         _layer("latent_attention_2", _mixer(3, 10, 6, 14, 20, 0.4, 90000.0, scaling=(16.0, 32, 8.0, 1.0)), 50),
         _layer("latent_attention", _mixer(2, 6, 10, 4, 28, 0.22, 250.0, q_rank=18), 30),
         _layer("latent_attention_2", _mixer(6, 4, 6, 10, 20, 0.35, 90000.0, kv_from=0, scaling=(16.0, 32, 8.0, 1.0)), 54),
     ]}
CONFIGS = {"P": (P, 3, 16), "Q": (Q, 4, 8)}            # name -> (config.json, seed, page size)


def make_model_dir(base, name: str) -> Path:
    """A folder written by the package's random-weights mode, then made harder: the mixers' matrices are
    scaled up so that attention is a large share of the stream (a wrong key must move the logits), the sinks
    are of order one, and the depth-average weights mix the whole history."""
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.weights import write_random_model, write_safetensors
    from sprout_lm_b200.weights.safetensors_io import SafetensorsFile
    raw, seed, _ = CONFIGS[name]
    directory = write_random_model(Path(base) / f"tulipel_{name}", parse_config(raw), seed=seed)
    rng = np.random.default_rng(seed)
    tensors = {}
    handle = SafetensorsFile(directory / "model.safetensors")
    try:
        for key in handle.names():
            value = handle.tensor(key).float()
            if ".mix." in key and value.dim() == 2:
                value = value * 4.0
            elif key.endswith(".sink"):
                value = torch.from_numpy(rng.normal(0.0, 1.5, size=value.shape).astype(np.float32))
            elif key.endswith(".dwa"):
                value = value + torch.from_numpy(rng.normal(0.0, 0.3, size=value.shape).astype(np.float32))
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


def compare(directory, requests: dict, got: dict, tol: float, label: str, page: int):
    """Every place that came back against the oracle; a failure names the first wrong token and its place."""
    assert got, "no logits came back"
    worst = 0.0
    for rid, tokens in requests.items():
        want = plain_logits(directory, tokens)
        for pos in range(len(tokens)):
            if (rid, pos) not in got:
                continue
            err = float(np.abs(got[(rid, pos)] - want[pos]).max())
            if not np.isfinite(err) or err > tol:
                raise AssertionError(f"{label}: request {rid} position {pos} of {len(tokens)} (position % {page} = {pos % page}, "
                                     f"% 128 = {pos % 128}) differs by {err:.3e} > {tol}")
            worst = max(worst, err)
    return worst
