"""A plain, slow implementation of the Letanex decoder in float64 numpy: one function per mechanism,
written from the model's equations, sharing nothing with the package.  ``forward`` runs a whole
sequence at once (no cache, no state carried): it is what the engine's steps are held against.

Notation: T tokens, W the model's width; a config is the dict of the model's config.json; weights
a dict name -> float64 array.
"""
from __future__ import annotations

import numpy as np


# ------------------------------------------------------------------------------ small pieces
def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis; var = mean of squared deviations."""
    mean = x.mean(axis=-1, keepdims=True)
    dev = x - mean
    var = (dev * dev).mean(axis=-1, keepdims=True)
    return dev / np.sqrt(var + eps) * w


def rms(x, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softmax(z):
    z = z - z.max(axis=-1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(axis=-1, keepdims=True)


def rotate(x, positions, rot):
    """x [T, n, dim]: the first rot['dims'] elements of every vector turn, element i paired with
    element i + dims/2, by the angle position * base**(-2i/dims) / factor."""
    dims, base = rot["dims"], rot["base"]
    factor = (rot.get("scaling") or {}).get("factor", 1.0)
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims) / factor
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


# ------------------------------------------------------------------------------ mixers
def attention_keys_values(h, weights, prefix, m, positions):
    """Rotated keys [T, G, 2, dim] and values [T, G, vdim] of a layer that projects its own."""
    T = h.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ weights[prefix + "k"].T).reshape(T, G * 2, dim)
    k = rotate(k, positions, m["rot"]).reshape(T, G, 2, dim)
    v = (h @ weights[prefix + "v"].T).reshape(T, G, vdim)
    return k, v


def differential_heads(q, k, v, positions, scale, lam, eps, out_scale):
    """q [T, H, 2, dim] (rotated), k [S, G, 2, dim] (rotated; key j sits at position j), v [S, G, vdim]:
    per head a_0 - lam a_1 over the keys j <= position, divided by its root mean square, times out_scale.
    Returns [T, H, vdim]."""
    T, H = q.shape[:2]
    G = k.shape[1]
    visible = np.asarray(positions)[:, None] >= np.arange(k.shape[0])[None, :]
    out = np.zeros((T, H, v.shape[-1]))
    for head in range(H):
        g = head // (H // G)
        maps = []
        for which in range(2):
            score = (q[:, head, which, :] @ k[:, g, which, :].T) * scale
            score = np.where(visible, score, -np.inf)
            maps.append(softmax(score) @ v[:, g, :])
        out[:, head] = rms(maps[0] - lam * maps[1], eps) * out_scale
    return out


def differential_lambda(weights, prefix, diff):
    return np.exp(np.sum(weights[prefix + "lq1"] * weights[prefix + "lk1"])) \
        - np.exp(np.sum(weights[prefix + "lq2"] * weights[prefix + "lk2"])) + diff


def differential_attention(h, weights, prefix, m, eps, k, v, positions=None):
    """Two softmax maps per head over the same values; o = a1 - lambda a2, divided by its root mean
    square over the head, times (1 - diff); then the output projection.  ``k``/``v``: all keys and
    values of the sequence (own or another layer's)."""
    T = h.shape[0]
    H, dim = m["heads"], m["dim"]
    positions = np.arange(T) if positions is None else positions
    q = (h @ weights[prefix + "q"].T).reshape(T, H * 2, dim)
    q = rotate(q, positions, m["rot"]).reshape(T, H, 2, dim)
    lam = differential_lambda(weights, prefix, m["diff"])
    o = differential_heads(q, k, v, positions, m["scale"], lam, eps, 1.0 - m["diff"])
    return o.reshape(T, -1) @ weights[prefix + "o"].T


def decay_recurrence(q, k, v, decay, state=None):
    """q, k [T, H, dim], v [T, H, vdim]: S = decay_h S + k v^T, o = S^T q token by token.  (o [T, H, vdim], S)."""
    T, H, dim = q.shape
    S = np.zeros((H, dim, v.shape[-1])) if state is None else state.copy()
    out = np.zeros((T, H, v.shape[-1]))
    decay = np.asarray(decay, dtype=np.float64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hdv,hd->hv", S, q[t])
    return out, S


def lightning(h, weights, prefix, m, eps, state=None):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, token by token; the heads together are
    divided by their root mean square, times '.norm', times sigmoid(W_g h); then W_o.
    Returns (output, final state [heads, dim, vdim])."""
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ weights[prefix + "q"].T).reshape(T, H, dim)
    k = silu(h @ weights[prefix + "k"].T).reshape(T, H, dim)
    v = silu(h @ weights[prefix + "v"].T).reshape(T, H, vdim)
    out, S = decay_recurrence(q, k, v, m["decay"], state)
    o = rms(out.reshape(T, H * vdim), eps) * weights[prefix + "norm"]
    o = o * sigmoid(h @ weights[prefix + "g"].T)
    return o @ weights[prefix + "o"].T, S


# ------------------------------------------------------------------------------ feed-forwards
def dense_ff(h, weights, prefix):
    z = np.maximum(h @ weights[prefix + "up"].T, 0.0)
    return (z * z) @ weights[prefix + "down"].T


def clamped_expert(h, weights, prefix, limit):
    g = np.minimum(h @ weights[prefix + "gate"].T, limit)
    u = np.clip(h @ weights[prefix + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ weights[prefix + "down"].T


def route(h, weights, prefix, router):
    """(chosen experts [T, top], their weights [T, top]); expert ids >= router['experts'] are identity experts."""
    z = h @ weights[prefix + "router"].T
    s = softmax(z)
    choice = s + weights[prefix + "correction"]
    top = router["top"]
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(s, chosen, axis=-1)
    return chosen, picked / (picked.sum(axis=-1, keepdims=True) + 1e-20) * router["scale"]


def mixture_ff(h, weights, prefix, mlp):
    router = mlp["router"]
    chosen, weight = route(h, weights, prefix, router)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weight[t]):
            if e >= router["experts"]:
                out[t] += w * h[t]
            else:
                out[t] += w * clamped_expert(h[t:t + 1], weights, f"{prefix}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += clamped_expert(h, weights, prefix + "shared.", mlp["shared"]["limit"])
    return out


def feed_forward(h, weights, prefix, mlp):
    return dense_ff(h, weights, prefix) if mlp["kind"] == "dense" else mixture_ff(h, weights, prefix, mlp)


# ------------------------------------------------------------------------------ the model
def forward(config, weights, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (positions 0..T-1); with ``return_layers`` also the
    residual stream after every layer [layers, T, W]."""
    eps = config["norm"]["eps"]
    tokens = np.asarray(tokens)
    positions = np.arange(len(tokens))
    x = weights["embed"][tokens]
    kept = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = layer_norm(x, weights[p + "norm1"], eps)
        if layer["type"] == "attention":
            source = m.get("kv_from")
            if source is None:
                kept[i] = attention_keys_values(h, weights, p + "mix.", m, positions)
                source = i
            y = differential_attention(h, weights, p + "mix.", m, eps, *kept[source])
        elif layer["type"] == "lightning":
            y, _ = lightning(h, weights, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, weights[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = layer_norm(x, weights[p + "norm2"], eps)
            x = x + layer_norm(feed_forward(h, weights, p + "mlp.", layer["mlp"]), weights[p + "norm2b"], eps)
        after.append(x)
    logits = layer_norm(x, weights["final.norm"], eps) @ weights["head"].T
    return (logits, np.stack(after)) if return_layers else logits


# ------------------------------------------------------------------------------ model folders
def read_model_folder(directory):
    """(config, weights as float64) of a folder with config.json and model.safetensors (its own little reader: an
    8-byte length, a JSON header, the data)."""
    import json
    import struct
    from pathlib import Path
    directory = Path(directory)
    config = json.loads((directory / "config.json").read_text())
    raw = (directory / "model.safetensors").read_bytes()
    size = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + size])
    data = raw[8 + size:]
    weights = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        chunk = data[begin:end]
        if info["dtype"] == "BF16":
            values = (np.frombuffer(chunk, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif info["dtype"] == "F32":
            values = np.frombuffer(chunk, dtype="<f4").astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        weights[name] = values.reshape(info["shape"])
    return config, weights


def logits(config, weights, tokens):
    return forward(config, weights, tokens)


def greedy(config, weights, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(np.argmax(forward(config, weights, tokens)[-1])))
    return tokens[len(prompt):]
