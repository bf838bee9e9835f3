"""Plain, slow implementation of the Rirulix decoder (NumPy, whole sequences, no cache, no state
carried between calls): the oracle of the tests of that design.

One function per mechanism, written from the design's equations; it shares no code with the
engine (its own reading of config.json and of the safetensors container, ``plain.decoder``'s).
All arithmetic runs in the dtype of the weights the caller passes (float64 in the tests).

Notation: n tokens, H width, positions i, j count from 0 in a sequence.
"""

from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

import numpy as np

from .decoder import read_safetensors


def load_model_dir(model_dir: str, dtype=np.float64):
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    w = {k: v.astype(dtype) for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


def group_rms_norm(x: np.ndarray, weight: np.ndarray, groups: int, eps: float) -> np.ndarray:
    """x [n, H] cut into ``groups`` equal consecutive parts; part / sqrt(mean(part^2) + eps); times weight."""
    n, h = x.shape
    parts = x.reshape(n, groups, h // groups)
    parts = parts / np.sqrt(np.mean(parts * parts, axis=-1, keepdims=True) + eps)
    return parts.reshape(n, h) * weight


def gelu_tanh(z: np.ndarray) -> np.ndarray:
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z: np.ndarray) -> np.ndarray:
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def embed(cfg: dict, w: Dict[str, np.ndarray], ids: Sequence[int]) -> np.ndarray:
    """norm(E[token] + P[i]): the learned position vector is added as it is."""
    n = len(ids)
    x = w["embed"][np.asarray(ids)] + w["pos"][:n]
    return group_rms_norm(x, w["embed.norm"], cfg["norm"]["groups"], cfg["norm"]["eps"])


def causal_conv(x: np.ndarray, taps: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """Per channel c: out_t = sum_j taps[c, j] * x_(t - (T-1) + j) + bias[c], zeros before t = 0."""
    n, width = x.shape
    t = taps.shape[1]
    padded = np.concatenate([np.zeros((t - 1, width), dtype=x.dtype), x])
    out = np.zeros_like(x)
    for j in range(t):
        out += padded[j:j + n] * taps[:, j]
    return out + bias


def block_gate(u: np.ndarray, matrices: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """sigmoid(M[b] u_b + bias[b]) for every block b of the channels; matrices [blocks, out, in]."""
    n = u.shape[0]
    blocks = matrices.shape[0]
    ub = u.reshape(n, blocks, -1)
    out = np.stack([ub[:, b] @ matrices[b].T + bias[b] for b in range(blocks)], axis=1)
    return sigmoid(out).reshape(n, -1)


def gated_recurrence(u: np.ndarray, r: np.ndarray, i: np.ndarray, lam: np.ndarray, gain: float = 8.0) -> np.ndarray:
    """a_t = exp(-gain r_t softplus(lam)); S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0."""
    a = np.exp(-gain * r * softplus(lam))
    s = np.zeros(u.shape[1], dtype=u.dtype)
    out = np.zeros_like(u)
    for t in range(u.shape[0]):
        s = a[t] * s + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = s
    return out


def recurrent_mixer(h: np.ndarray, w: Dict[str, np.ndarray], p: str) -> np.ndarray:
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    s = gated_recurrence(u, block_gate(u, w[p + "ra"], w[p + "ra.b"]), block_gate(u, w[p + "ri"], w[p + "ri.b"]), w[p + "lam"])
    return (s * y) @ w[p + "o"].T


def visible(n: int, window: Optional[int], keep_first: int) -> np.ndarray:
    """[n, n] bool: query i sees key j when j <= i and (i - j < window or j < keep_first)."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    near = np.ones((n, n), dtype=bool) if not window else (i - j < window) | (j < keep_first)
    return (j <= i) & near


def biased_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, r1: np.ndarray, r2: np.ndarray,
                     window: Optional[int], keep_first: int) -> np.ndarray:
    """q [n, heads, D], k [n, kv, D], v [n, kv, Dv] -> [n, heads, Dv];
    score = q.k * scale - r1[h] ln(1 + r2[h] (i - j)), softmax over the visible keys."""
    n, heads, _ = q.shape
    share = heads // k.shape[1]
    see = visible(n, window, keep_first)
    dist = np.maximum(np.arange(n)[:, None] - np.arange(n)[None, :], 0).astype(q.dtype)
    out = np.zeros((n, heads, v.shape[2]), dtype=q.dtype)
    for h in range(heads):
        s = (q[:, h] @ k[:, h // share].T) * scale - r1[h] * np.log1p(r2[h] * dist)
        s = np.where(see, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (e / e.sum(axis=1, keepdims=True)) @ v[:, h // share]
    return out


def attention_mixer(h: np.ndarray, w: Dict[str, np.ndarray], p: str, m: dict, passed: dict) -> np.ndarray:
    """``passed`` carries the first value-mixing layer's values through one forward pass."""
    n = h.shape[0]
    heads, kv, d = m["heads"], m["kv_heads"], m["dim"]
    dv = m.get("vdim") or d
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(n, heads, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(n, kv, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(n, kv, dv)
    if m.get("v_mix"):
        if "values" in passed:
            mix = float(np.asarray(w[p + "vmix"]).reshape(-1)[0])
            v = (1.0 - mix) * v + mix * passed["values"]
        else:
            passed["values"] = v
    mask = m.get("mask") or {}
    o = biased_attention(q, k, v, m["scale"], w[p + "r1"], w[p + "r2"], mask.get("size"), mask.get("keep_first") or 0)
    return o.reshape(n, heads * dv) @ w[p + "o"].T + w[p + "o.b"]


def glu_expert(a: np.ndarray, w: Dict[str, np.ndarray], p: str, limit: float, alpha: float = 1.702) -> np.ndarray:
    g = np.minimum(a @ w[p + "gate"].T, limit)
    u = np.clip(a @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(alpha * g) * (u + 1.0)) @ w[p + "down"].T


def routed_feed_forward(h: np.ndarray, w: Dict[str, np.ndarray], p: str, m: dict) -> np.ndarray:
    """Scores sigmoid(Wr h); the ``top`` largest, weights as they are, on the expert's input."""
    scores = sigmoid(h @ w[p + "router"].T)
    top = m["router"]["top"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in np.argsort(-scores[t], kind="stable")[:top]:
            out[t] += glu_expert(scores[t, e] * h[t:t + 1], w, f"{p}e{e}.", m["expert"]["limit"])[0]
    if m.get("shared"):
        gate = sigmoid(h @ w[p + "shared.sg"].T)                   # [n, 1]
        out += gate * glu_expert(h, w, p + "shared.", m["shared"]["limit"])
    return out


def forward_logits(cfg: dict, w: Dict[str, np.ndarray], ids: Sequence[int], residuals: Optional[List[np.ndarray]] = None):
    groups, eps = cfg["norm"]["groups"], cfg["norm"]["eps"]
    norm = lambda x, name: group_rms_norm(x, w[name], groups, eps)
    x = embed(cfg, w, ids)
    passed: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm(x, p + "norm1")
        if layer["type"] == "rglru":
            mixed = recurrent_mixer(h, w, p + "mix.")
        else:
            mixed = attention_mixer(h, w, p + "mix.", layer["mixer"], passed)
        x = x + norm(mixed, p + "norm1b")
        if layer.get("mlp"):
            x = x + norm(routed_feed_forward(norm(x, p + "norm2"), w, p + "mlp.", layer["mlp"]), p + "norm2b")
        if residuals is not None:
            residuals.append(x.copy())
    return norm(x, "final.norm") @ w["head"].T


def greedy_generate(cfg: dict, w: Dict[str, np.ndarray], prompt: Sequence[int], n_new: int) -> List[int]:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(np.argmax(forward_logits(cfg, w, ids)[-1])))
    return ids[len(prompt):]


def generation_margins(cfg: dict, w: Dict[str, np.ndarray], prompt: Sequence[int], generated: Sequence[int]) -> List[float]:
    """For each generated token, how far its logit lies below the largest one (0: it is the choice)."""
    ids = list(prompt) + list(generated)
    logits = forward_logits(cfg, w, ids)
    return [float(logits[len(prompt) + k - 1].max() - logits[len(prompt) + k - 1][t]) for k, t in enumerate(generated)]
