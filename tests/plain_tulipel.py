"""Plain, slow Tulipel decoder for tests: whole sequences, no cache, no paging, float64.

The oracle that the engine's Tulipel path is compared with.  It shares no code with the package:
one function per mechanism, written from the model's equations, and the safetensors reader of the
other oracle.  A model is (config dict as in config.json, {tensor name: array}).

Notation: T tokens, W stream width, H heads, d unrotated and r rotated query/key elements per head,
v value elements per head, R latent size.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np

from plain_qwen2 import read_safetensors

F64 = np.float64


def read_model_folder(directory):
    directory = Path(directory)
    config = json.loads((directory / "config.json").read_text())
    tensors = {name: value.astype(F64) for name, value in read_safetensors(directory / "model.safetensors").items()}
    return config, tensors


# ---------------------------------------------------------------- norms and activations
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(np.square(x), axis=-1, keepdims=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight w lies around zero: the gain is 1 + w."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


def polynorm(z, coefficients, eps):
    a, b, c, e = coefficients
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def feed_forward(h, up, down, coefficients, eps):
    return polynorm(h @ up.T, coefficients, eps) @ down.T


def softcap(logits, cap):
    return cap * np.tanh(logits / cap)


# ---------------------------------------------------------------- rotation
def rotation_frequencies(rot):
    """One frequency per rotated pair; stretched when rot has 'scaling'.  Also the factor on cos and sin."""
    n, base = rot["dims"], rot["base"]
    freq = np.array([base ** (-2.0 * i / n) for i in range(n // 2)], dtype=F64)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def pair_index(turns):
        return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_index(scaling["fast"])), 0)
    hi = min(math.ceil(pair_index(scaling["slow"])), n - 1)
    out = np.empty_like(freq)
    for i in range(n // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = freq[i] / factor * ramp + freq[i] * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate(vectors, positions, rot, interleaved):
    """vectors [T, ..., r]: the first rot['dims'] elements turn by position * frequency, pair by pair;
    pairs are (2i, 2i+1) when interleaved, else (i, i + dims/2); the rest pass."""
    n = rot["dims"]
    freq, magnitude = rotation_frequencies(rot)
    out = np.array(vectors, dtype=F64, copy=True)
    for t, p in enumerate(positions):
        for i in range(n // 2):
            a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + n // 2)
            c, s = math.cos(p * freq[i]) * magnitude, math.sin(p * freq[i]) * magnitude
            u, w = vectors[t][..., a], vectors[t][..., b]
            out[t][..., a] = u * c - w * s
            out[t][..., b] = w * c + u * s
    return out


# ---------------------------------------------------------------- attention
def softmax_with_sink(scores, sink):
    """scores [T, T] already masked with -inf; the denominator holds exp(sink) once more."""
    top = np.maximum(scores.max(axis=-1, keepdims=True), sink)
    e = np.exp(scores - top)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - top))


def latent_rows(layer, tensors, prefix, h, eps, interleaved):
    """What a layer caches per token: the normed latent [T, R] and the rotated shared key part [T, r]."""
    m = layer["mixer"]
    both = h @ tensors[prefix + "mix.dkv"].T
    latent = norm_plain(both[:, :m["kv_rank"]], tensors[prefix + "mix.dkv.norm"], eps)
    shared = both[:, m["kv_rank"]:]
    if m["rot_dim"]:
        shared = rotate(shared, range(h.shape[0]), m["rot"], interleaved)
    return latent, shared


def attention(layer, tensors, prefix, h, eps, rows):
    """Head by head, in the unfolded form: keys and values are made from the latent per head."""
    m = layer["mixer"]
    H, d, r, v = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = h.shape[0]
    interleaved = layer["type"] == "latent_attention"
    if interleaved:
        q = norm_plain(h @ tensors[prefix + "mix.dq"].T, tensors[prefix + "mix.dq.norm"], eps) @ tensors[prefix + "mix.uq"].T
    else:
        q = h @ tensors[prefix + "mix.q"].T
    q = q.reshape(T, H, d + r)
    latent, shared = rows
    keys = (latent @ tensors[prefix + "mix.uk"].T).reshape(T, H, d)
    values = (latent @ tensors[prefix + "mix.uv"].T).reshape(T, H, v)
    q_rot = rotate(q[:, :, d:], range(T), m["rot"], interleaved) if r else q[:, :, d:]
    mask = np.triu(np.full((T, T), -np.inf), k=1)
    heads = []
    for n in range(H):
        scores = (q[:, n, :d] @ keys[:, n, :].T + q_rot[:, n, :] @ shared.T) * m["scale"] + mask
        heads.append(softmax_with_sink(scores, tensors[prefix + "mix.sink"][n]) @ values[:, n, :])
    return np.concatenate(heads, axis=-1) @ tensors[prefix + "mix.o"].T


# ---------------------------------------------------------------- the model
def hidden_states(config, tensors, tokens):
    """(stream after every layer, after the depth average; the final stream)."""
    eps, alpha = config["norm"]["eps"], config["postln_alpha"]
    x = tensors["embed"][np.asarray(tokens, dtype=np.int64)]
    results, cached, after = [x], {}, []
    for i, layer in enumerate(config["layers"]):
        prefix = f"l{i}."
        source = layer["mixer"].get("kv_from")
        if source is None:
            cached[i] = latent_rows(layer, tensors, prefix, x, eps, layer["type"] == "latent_attention")
        rows = cached[i if source is None else source]
        x = norm_around_zero(alpha * x + attention(layer, tensors, prefix, x, eps, rows), tensors[prefix + "norm1"], eps)
        if layer["mlp"] is not None:
            ff = feed_forward(x, tensors[prefix + "mlp.up"], tensors[prefix + "mlp.down"], tensors[prefix + "mlp.act"], eps)
            x = norm_around_zero(alpha * x + ff, tensors[prefix + "norm2"], eps)
        results.append(x)
        weights = tensors[prefix + "dwa"]
        x = sum(weights[j] * results[j] for j in range(i + 2))
        after.append(x)
    return after, x


def logits(config, tensors, tokens):
    _, x = hidden_states(config, tensors, tokens)
    x = norm_around_zero(x, tensors["final.norm"], config["norm"]["eps"])
    return softcap(x @ tensors["head"].T, config["logit_softcap"])


def greedy(config, tensors, prompt, new_tokens):
    history, out = list(prompt), []
    for _ in range(new_tokens):
        token = int(np.argmax(logits(config, tensors, history)[-1]))
        out.append(token)
        history.append(token)
    return out
