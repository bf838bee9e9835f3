"""A plain, slow implementation of the Labolix decoder: NumPy float64, one whole sequence at a
time, one function per mechanism, no cache and no batching.  It reads the raw ``config.json``
dictionary and a dictionary of arrays by checkpoint name, and shares nothing with the engine.

Notation: T tokens, width W; a mixer's input is h [T, W]; positions are 0 .. T-1.
"""

from __future__ import annotations

import math

import numpy as np


# ---- small pieces --------------------------------------------------------------------------------

def dynamic_tanh(x, weight, bias, alpha):
    """tanh(alpha x) * w + b: a norm that looks at no statistics of the vector."""
    return np.tanh(float(alpha) * x) * weight + bias


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def clamped_glu(h, w_gate, w_up, w_down, limit, alpha=1.702):
    g = np.minimum(h @ w_gate.T, limit)
    u = np.clip(h @ w_up.T, -limit, limit)
    return (g * sigmoid(alpha * g) * (u + 1.0)) @ w_down.T


# ---- rotary frequencies and the three ways they are scaled -----------------------------------------

def base_frequencies(dims, base):
    return np.array([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)


def wavelength_scaled_frequencies(dims, base, factor, low, high, original):
    """Long wavelengths are slowed by ``factor``, short ones kept, the band between blended."""
    out = []
    for f in base_frequencies(dims, base):
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return np.array(out), 1.0


def ramp_scaled_frequencies(dims, base, factor, original, fast, slow):
    """A linear ramp over the pair index between the pairs that turn ``fast`` and ``slow`` times
    within the original length; also returns the factor on cos and sin."""
    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(base_frequencies(dims, base)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return np.array(out), 0.1 * math.log(factor) + 1.0


def rotary_table(rot, kind):
    """(frequencies [dims/2], magnitude) of a mixer's ``rot`` entry; ``kind`` says how a ``scaling``
    entry is to be read: 'wavelength' or 'ramp'."""
    dims, base = int(rot["dims"]), float(rot["base"])
    sc = rot.get("scaling")
    if not sc:
        return base_frequencies(dims, base), 1.0
    if kind == "wavelength":
        return wavelength_scaled_frequencies(dims, base, sc["factor"], sc["low"], sc["high"], sc["original"])
    return ramp_scaled_frequencies(dims, base, sc["factor"], sc["original"], sc["fast"], sc["slow"])


def rotate(x, positions, freqs, magnitude, layout):
    """x [T, heads, D]: the first 2 * len(freqs) channels of every head are turned, the rest pass.
    'interleaved' pairs channel 2i with 2i+1, 'half' pairs i with i + dims/2."""
    half = len(freqs)
    dims = 2 * half
    ang = positions[:, None].astype(np.float64) * freqs[None, :]
    cos, sin = (np.cos(ang) * magnitude)[:, None, :], (np.sin(ang) * magnitude)[:, None, :]
    out = x.copy()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


# ---- the three mixers ------------------------------------------------------------------------------

def softmax_with_sink(scores, visible, sink):
    """Rows of ``scores`` [T, T] over the visible keys, with exp(sink) added to the denominator."""
    s = np.where(visible, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def attention(h, m, w, prefix, eps):
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = np.arange(T)
    freqs, mag = rotary_table(m["rot"], "wavelength")
    q = rotate((h @ w[prefix + "q"].T).reshape(T, H, D), pos, freqs, mag, "interleaved")
    k = rotate((h @ w[prefix + "k"].T).reshape(T, G, D), pos, freqs, mag, "interleaved")
    v = (h @ w[prefix + "v"].T).reshape(T, G, Dv)
    visible = pos[:, None] >= pos[None, :]
    out = np.zeros((T, H, Dv))
    for head in range(H):
        g = head // (H // G)
        p = softmax_with_sink((q[:, head] @ k[:, g].T) * float(m["scale"]), visible, 0.0)
        out[:, head] = p @ v[:, g]
    return out.reshape(T, H * Dv) @ w[prefix + "o"].T


def latent_attention(h, m, w, prefix, eps):
    T = h.shape[0]
    H, D, R, Dv, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = np.arange(T)
    freqs, mag = rotary_table(m["rot"], "ramp")
    q = (h @ w[prefix + "q"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], pos, freqs, mag, "interleaved")
    down = h @ w[prefix + "dkv"].T
    c = rms_unit(down[:, :C], eps) * w[prefix + "dkv.norm"]
    k_rot = rotate(down[:, None, C:], pos, freqs, mag, "interleaved")[:, 0]
    k_plain = (c @ w[prefix + "uk"].T).reshape(T, H, D)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, Dv)
    dist = pos[:, None] - pos[None, :]
    visible = (dist >= 0) & (dist < int(m["mask"]["size"]))
    out = np.zeros((T, H, Dv))
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * float(m["scale"])
        out[:, head] = softmax_with_sink(s, visible, float(w[prefix + "sink"][head])) @ v[:, head]
    return out.reshape(T, H * Dv) @ w[prefix + "o"].T


def retention(h, m, w, prefix, eps):
    T = h.shape[0]
    H, D, Dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = np.arange(T)
    freqs, mag = rotary_table(m["rot"], "none")
    q = rotate((h @ w[prefix + "q"].T).reshape(T, H, D), pos, freqs, mag, "half")
    k = rotate((h @ w[prefix + "k"].T).reshape(T, H, D), pos, freqs, mag, "half") * D ** -0.5
    v = (h @ w[prefix + "v"].T).reshape(T, H, Dv)
    out = np.zeros((T, H, Dv))
    for head in range(H):
        S = np.zeros((D, Dv))
        decay = float(m["decay"][head])
        for t in range(T):
            S = decay * S + np.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    out = rms_unit(out, eps).reshape(T, H * Dv)
    return (out * silu(h @ w[prefix + "g"].T)) @ w[prefix + "o"].T


MIXERS = {"attention": attention, "latent_attention": latent_attention, "retention": retention}


# ---- the model -------------------------------------------------------------------------------------

def forward(config, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64); with ``return_layers`` also the residual stream
    after every layer [layers, T, W]."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)]
    streams = []
    for i, layer in enumerate(config["layers"]):
        own = f"l{layer['weights_of']}." if layer.get("weights_of") is not None else f"l{i}."
        norm = lambda name, x: dynamic_tanh(x, w[own + name], w[own + name + ".b"], w[own + name + ".alpha"])
        x = x + MIXERS[layer["type"]](norm("norm1", x), layer["mixer"], w, own + "mix.", eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            x = x + clamped_glu(norm("norm2", x), w[own + "mlp.gate"], w[own + "mlp.up"], w[own + "mlp.down"], float(mlp["limit"]))
        streams.append(x.copy())
    y = dynamic_tanh(x, w["final.norm"], w["final.norm.b"], w["final.norm.alpha"])
    logits = y @ w["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * np.tanh(logits / float(cap))
    return (logits, np.stack(streams)) if return_layers else logits


# ---- model folders, generation ---------------------------------------------------------------------

def load_model_dir(folder, dtype=np.float64):
    """(raw config.json dictionary, tensors by name) of a model folder."""
    import json
    import os

    from .decoder import read_safetensors

    with open(os.path.join(folder, "config.json"), encoding="utf-8") as fh:
        config = json.load(fh)
    return config, {k: np.asarray(v, dtype=dtype) for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}


def forward_logits(config, w, tokens):
    return forward(config, w, tokens)


def greedy_generate(config, w, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(np.argmax(forward(config, w, ids)[-1])))
    return ids[len(prompt):]


def generation_margins(config, w, prompt, generated):
    """For every generated token: how far its plain logit lies below the largest one at its place."""
    logits = forward(config, w, list(prompt) + list(generated))
    at = len(prompt) - 1
    return [float(logits[at + i].max() - logits[at + i, t]) for i, t in enumerate(generated)]
