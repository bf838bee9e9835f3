"""Tiny configurations of the Rirulix design for the tests, and the helper that writes them as model
folders with random weights.

The four differ in every size and option: widths, vocabularies, norm groups (1, 3, 4), layer
orders, head counts and groupings (grouped, one kv head, as many kv heads as query heads), key and
value sizes (equal and not), windows (none, shorter than a page, across pages) with 0 to 5 kept
first tokens, value mixing on some layers or none, experts and choices per token (1 to 3), a shared
expert or none, layers without a feed-forward, convolutions of 2 to 4 taps, 1 to 4 gate blocks.

The engine's random weights (N(0, 0.02) matrices) are made larger here, so that attention is
peaked, gates leave their middle and the experts' clamps are reached: a key too many or too few, a
lost state or a wrong expert then moves the logits far beyond rounding.
"""

from __future__ import annotations

import os

import numpy as np

ARCH = "Rirulix"


def _attn(heads, kv, dim, vdim, scale, window, keep, v_mix):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    return m


def _moe(experts, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


def _config(vocab, width, max_positions, groups, eps, layers):
    return {"architecture": ARCH, "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": eps, "groups": groups}, "layers": layers}


# 6 layers, width 96, 3 norm groups; window 24 (a page and a half of 16) with 3 kept tokens, window 40
# with none, a layer that sees everything, window 17 with 5 kept; values of 16 under keys of 32; a
# layer of as many kv heads as query heads with values larger than keys; two layers without a
# feed-forward; 2 of 6 experts with a shared one, 2 of 6 without, 1 of 4.
R1 = _config(211, 96, 512, 3, 1e-5, [
    {"type": "rglru", "mixer": {"width": 64, "blocks": 4, "conv": 3}, "mlp": _moe(6, 2, 40, 1.5, (56, 0.75))},
    {"type": "attention", "mixer": _attn(6, 2, 32, 16, 0.2, 24, 3, True), "mlp": None},
    {"type": "attention", "mixer": _attn(6, 2, 32, 16, 0.15, 40, 0, True), "mlp": _moe(6, 2, 40, 1.5)},
    {"type": "attention", "mixer": _attn(4, 4, 16, 32, 0.3, None, 0, False), "mlp": _moe(4, 1, 24, 2.5, (32, 1.0))},
    {"type": "rglru", "mixer": {"width": 96, "blocks": 1, "conv": 2}, "mlp": None},
    {"type": "attention", "mixer": _attn(6, 2, 32, 16, 0.2, 17, 5, True), "mlp": _moe(6, 2, 40, 1.5, (56, 0.75))},
])
# 4 layers, width 128, plain norm (1 group); keys and values of 64 (the tensor-core sizes), one kv head
# for 4 query heads; window 50 with 1 kept token and window 9 (less than a page) with 2; no value
# mixing anywhere; 3 of 5 experts; a convolution of 4 taps.
R2 = _config(300, 128, 768, 1, 1e-6, [
    {"type": "attention", "mixer": _attn(4, 1, 64, 64, 0.125, 50, 1, False), "mlp": _moe(5, 3, 48, 2.0, (64, 1.0))},
    {"type": "rglru", "mixer": {"width": 128, "blocks": 2, "conv": 4}, "mlp": _moe(5, 3, 48, 2.0)},
    {"type": "attention", "mixer": _attn(4, 1, 64, 64, 0.125, 9, 2, False), "mlp": _moe(5, 3, 48, 2.0, (64, 1.0))},
    {"type": "rglru", "mixer": {"width": 64, "blocks": 1, "conv": 2}, "mlp": _moe(5, 3, 48, 2.0)},
])
# 3 layers, width 256, 4 norm groups; keys of 128 with values of 64, then keys and values of 64 with
# 6 query heads, value mixing between them; windows beyond a hundred tokens; 8 experts of which 1.
R3 = _config(160, 256, 1024, 4, 1e-6, [
    {"type": "attention", "mixer": _attn(4, 2, 128, 64, 0.09, 130, 6, True), "mlp": _moe(8, 1, 72, 1.75, (88, 1.25))},
    {"type": "rglru", "mixer": {"width": 192, "blocks": 3, "conv": 4}, "mlp": _moe(8, 1, 72, 1.75, (88, 1.25))},
    {"type": "attention", "mixer": _attn(6, 2, 64, 64, 0.11, 200, 7, True), "mlp": _moe(8, 1, 72, 1.75, (88, 1.25))},
])

# 3 layers of the recurrence alone: a model without a single cached key (no page is ever taken); every
# expert is used by every token, so bfloat16 has no choice to flip.
R4 = _config(120, 80, 400, 5, 1e-6, [
    {"type": "rglru", "mixer": {"width": 48, "blocks": 3, "conv": 2}, "mlp": _moe(3, 3, 20, 1.5, (12, 0.5))},
    {"type": "rglru", "mixer": {"width": 112, "blocks": 1, "conv": 5}, "mlp": None},
    {"type": "rglru", "mixer": {"width": 80, "blocks": 5, "conv": 1}, "mlp": _moe(2, 2, 36, 2.5)},
])

TINY = {"R1": (R1, 11, 16), "R2": (R2, 12, 8), "R3": (R3, 13, 16), "R4": (R4, 14, 16)}      # config, weight seed, page size

GAIN = 5.0       # what the matrices of the layers are multiplied by


def make_model_dir(tmp_dir, name: str, storage_dtype: str = "float32") -> str:
    """Random weights from the engine's random mode, the layers' matrices multiplied by ``GAIN`` (the
    embedding, the position table and the head stay as drawn), stored in ``storage_dtype``."""
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
            if key.startswith("l") and t.dim() >= 2 and not key.endswith((".ra", ".ri", ".conv", ".router")):
                t = t * GAIN
            yield key, t.to(dtype)

    write_safetensors(path, named(), metadata={"format": "pt"})
    return folder
