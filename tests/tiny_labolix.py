"""Tiny configurations of the Labolix design for the tests, and the helper that writes them as model
folders with random weights.

The five differ in every size and option: widths, vocabularies, layer orders, which layers run with
another layer's tensors (none, one, several, of every mixer), head counts and groupings (grouped, one
kv head, as many kv heads as query heads), key and value sizes (equal and not), how many channels of
a head are turned (all, some, none), scaled frequencies or plain ones, windows (shorter than a page,
across pages, beyond a hundred tokens), latent ranks below and above the head size, decays from 0.5
to 1, layers without a feed-forward, a cap on the logits or none.

The engine's random weights (N(0, 0.02) matrices) are made larger here, so that the norm's tanh bends, attention is peaked
and the clamps of the feed-forward are reached, and the learned sinks are spread out (as drawn they
would all lie at 0, where a learned sink and a sink of score 0 cannot be told apart): a key too many
or too few, a lost state or a forgotten sink then moves the logits far beyond rounding.
"""

from __future__ import annotations

import os

import numpy as np

ARCH = "Labolix"


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = scaling
    return r


def _attn(heads, kv, dim, vdim, scale, rot):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}


def _latent(heads, dim, rot_dim, vdim, rank, scale, window, rot):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "mask": {"size": window}, "rot": rot}


def _ret(heads, dim, vdim, decay, rot):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rot}


def _mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _config(vocab, width, eps, cap, layers):
    c = {"architecture": ARCH, "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if cap:
        c["logit_softcap"] = cap
    return c


WAVE = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}       # tiny original lengths: every band of the rule is met
RAMP = {"factor": 4.0, "original": 48, "fast": 8.0, "slow": 1.0}

# 5 layers, width 96: retention first (3 heads of 16 x 24, a decay of 1 among them, half of the channels turned), grouped
# attention (6 query heads on 2 kv heads, keys of 32 with 16 turned, values of 16), latent attention with a window of 24 (a
# page and a half of 16; rank 40 above the head size of 16, 8 turned channels), then the retention and the latent layer
# once more with the first ones' tensors; one layer without a feed-forward.
_L1_RET = {"type": "retention", "mixer": _ret(3, 16, 24, [0.5, 0.96875, 1.0], _rot(8, 100.0)), "mlp": _mlp(40, 1.5)}
_L1_LAT = {"type": "latent_attention", "mixer": _latent(3, 16, 8, 24, 40, 0.25, 24, _rot(8, 1000.0, RAMP)), "mlp": None}
L1 = _config(211, 96, 1e-5, 12.0, [
    _L1_RET,
    {"type": "attention", "mixer": _attn(6, 2, 32, 16, 0.2, _rot(16, 10000.0, WAVE)), "mlp": _mlp(56, 0.75)},
    _L1_LAT,
    dict(_L1_RET, weights_of=0),
    dict(_L1_LAT, weights_of=2),
])
# 4 layers, width 128, no cap on the logits, nothing shared: latent attention first, with keys and values of the
# tensor-core sizes (rank 48 + 16 turned = rows of 64, 4 heads) and a window of 9 (less than a page of 8 + 1); attention with
# one kv head for 4 query heads of 64 / 64, all channels turned, plain frequencies; retention with nothing turned; latent
# attention with a window of 50 and plain frequencies.
L2 = _config(300, 128, 1e-6, None, [
    {"type": "latent_attention", "mixer": _latent(4, 32, 16, 32, 48, 0.18, 9, _rot(16, 50000.0, RAMP)), "mlp": _mlp(48, 2.0)},
    {"type": "attention", "mixer": _attn(4, 1, 64, 64, 0.125, _rot(64, 10000.0)), "mlp": _mlp(48, 2.0)},
    {"type": "retention", "mixer": _ret(2, 32, 64, [0.9375, 0.75], _rot(0, 1.0)), "mlp": _mlp(64, 1.0)},
    {"type": "latent_attention", "mixer": _latent(2, 24, 16, 40, 112, 0.2, 50, _rot(16, 300.0)), "mlp": _mlp(48, 2.0)},
])
# 3 layers, width 256: attention with as many kv heads as query heads and values larger than keys, run twice; retention
# with heads of 64 x 32 and all channels turned.
_L3_ATT = {"type": "attention", "mixer": _attn(4, 4, 16, 32, 0.3, _rot(8, 500.0, WAVE)), "mlp": _mlp(72, 1.75)}
L3 = _config(160, 256, 1e-6, 30.0, [
    _L3_ATT,
    {"type": "retention", "mixer": _ret(4, 64, 32, [0.984375, 0.9921875, 0.99609375, 0.998046875], _rot(64, 1000000.0)), "mlp": None},
    dict(_L3_ATT, weights_of=0),
])
# 2 layers of retention alone: a model without a single cached key (no page is ever taken); odd sizes (heads of 12 x 20).
L4 = _config(120, 80, 1e-6, 8.0, [
    {"type": "retention", "mixer": _ret(5, 12, 20, [0.875, 0.9, 0.95, 0.99, 0.999], _rot(12, 10000.0)), "mlp": _mlp(36, 2.5)},
    {"type": "retention", "mixer": _ret(2, 40, 8, [0.96875, 0.6], _rot(20, 77.0)), "mlp": _mlp(20, 1.5)},
])

# 4 layers of awkward sizes, none a multiple of 8: width 100, vocabulary 77; attention of 3 heads on one kv head,
# keys of 24 with 6 turned channels, values of 20; latent attention of 5 heads of 12 + 6 over rank 18, values of 10, a
# window of 7 (less than half a page) and plain frequencies; retention of 3 heads of 10 x 14 with 4 turned channels; a
# feed-forward of 50; the attention layer once more.  Every kernel takes its general path here.
_L5_ATT = {"type": "attention", "mixer": _attn(3, 1, 24, 20, 0.21, _rot(6, 300.0, WAVE)), "mlp": _mlp(50, 1.25)}
L5 = _config(77, 100, 1e-5, 9.0, [
    _L5_ATT,
    {"type": "latent_attention", "mixer": _latent(5, 12, 6, 10, 18, 0.24, 7, _rot(6, 2000.0)), "mlp": _mlp(50, 1.25)},
    {"type": "retention", "mixer": _ret(3, 10, 14, [0.9, 0.96875, 0.75], _rot(4, 50.0)), "mlp": _mlp(30, 2.0)},
    dict(_L5_ATT, weights_of=0),
])

TINY = {"L1": (L1, 21, 16), "L2": (L2, 22, 8), "L3": (L3, 23, 16), "L4": (L4, 24, 16), "L5": (L5, 25, 16)}      # config, weight seed, page size

GAIN = 10.0         # what the matrices of the layers are multiplied by
SINK_GAIN = 60.0    # ... the learned sinks
EMBED_GAIN = 25.0   # ... the embedding: the stream must leave the linear middle of the norm's tanh


def make_model_dir(tmp_dir, name: str, storage_dtype: str = "float32") -> str:
    """Random weights from the engine's random mode, the layers' matrices multiplied by ``GAIN`` and the
    sinks by ``SINK_GAIN``, the embedding by ``EMBED_GAIN``, stored in ``storage_dtype``."""
    import torch

    from qwen25vl_lite.weights import write_random_model
    from qwen25vl_lite.weights.safetensors_io import write_safetensors

    from plain.decoder import read_safetensors

    cfg, seed, _ = TINY[name]
    folder = write_random_model(os.path.join(str(tmp_dir), f"tiny-{name}-{storage_dtype}"), cfg, seed, "float32", prefix="")
    path = os.path.join(folder, "model.safetensors")
    tensors = read_safetensors(path)
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[storage_dtype]

    def named():
        for key, value in tensors.items():
            t = torch.from_numpy(np.array(value, copy=True))
            if key.startswith("l") and t.dim() >= 2:
                t = t * GAIN
            elif key.endswith(".sink"):
                t = t * SINK_GAIN
            elif key == "embed":
                t = t * EMBED_GAIN
            yield key, t.to(dtype)

    write_safetensors(path, named(), metadata={"format": "pt"})
    return folder
