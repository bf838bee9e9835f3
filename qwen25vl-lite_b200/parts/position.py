"""Multimodal rotary position encoding (MRoPE) of the Qwen2.5-VL text decoder.

Formulas (reference src/qwen25vl_lite/rope.py): ``inv_freq[j] = theta^(-2j/D)`` (:26-33);
the angle of rotary channel j is ``pos[axis(j)] * inv_freq[j]`` in float32 (:48-68) where
the three sections of ``mrope_section`` assign the channels to the axes t, h, w (:71-96);
pairs are (j, j + D/2) (:36-40).  Plain text has the same index on all three axes, and a
decoded token sits at ``tokens computed + rope_delta`` (:238-247).
"""

from __future__ import annotations

from typing import Sequence, Tuple

import numpy as np
import torch

from ..ops import kernels
from .base import PositionEncoding, register_position_encoding


def prompt_positions(num_tokens: int, image_spans: Sequence[Tuple[int, int, int, int]] = ()):
    """Positions [3, num_tokens] of a prompt and its ``rope_delta``.

    ``image_spans`` are ``(start, t, h, w)`` with the grid in merged units: the span covers
    t*h*w tokens from index ``start``.  This restates the reference's ``get_rope_index``
    (rope.py:137-235) for prompts whose image tokens are given by place instead of by id
    (the vision tower that would fill them is not part of this engine): a text run puts
    cursor + i on all axes and advances the cursor by its length; an image run at cursor c
    gets (c + t_idx, c + row, c + col) in t-major, row-major order (rope.py:99-126, interval
    1) and advances the cursor by max(h, w); rope_delta = max(pos) + 1 - num_tokens."""
    cols = []
    cursor = 0
    at = 0
    for start, t, h, w in sorted(image_spans):
        if start < at or start + t * h * w > num_tokens:
            raise ValueError(f"image span {(start, t, h, w)} overlaps another or leaves the prompt")
        run = np.arange(start - at, dtype=np.int64) + cursor
        cols.append(np.stack([run, run, run]))
        cursor += start - at
        grid = np.stack(np.meshgrid(np.arange(t), np.arange(h), np.arange(w), indexing="ij")).reshape(3, -1)
        cols.append(grid.astype(np.int64) + cursor)
        cursor += max(h, w)
        at = start + t * h * w
    run = np.arange(num_tokens - at, dtype=np.int64) + cursor
    cols.append(np.stack([run, run, run]))
    pos = np.concatenate(cols, axis=1)
    delta = int(pos.max()) + 1 - num_tokens if num_tokens else 0
    return pos, delta


@register_position_encoding("mrope")
class MRope(PositionEncoding):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    axes = 3

    def __init__(self, head_dim: int, theta: float, sections: Sequence[int]):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.sections = tuple(int(s) for s in sections)
        if sum(self.sections) * 2 != self.head_dim:
            raise ValueError(f"mrope sections {self.sections} must sum to head_dim/2 = {self.head_dim // 2}")
        self.axes = len(self.sections)
        self.inv_freq = None
        self.axis = None

    def load(self, tensors, device, dtype):
        idx = torch.arange(0, self.head_dim, 2, dtype=torch.float32)
        self.inv_freq = (1.0 / (self.theta ** (idx / self.head_dim))).to(torch.float32).to(device)
        axis = []
        for a, n in enumerate(self.sections):
            axis += [a] * n
        self.axis = torch.tensor(axis, dtype=torch.int32, device=device)

    # plain text: token i of a request sits at i + offset on every axis, which lets the step
    # function fill the positions of a whole decode batch at once
    default_is_linear = True

    def default_positions(self, start: int, count: int, offset: int):
        run = np.arange(start + offset, start + offset + count, dtype=np.int64)
        return np.broadcast_to(run, (self.axes, count))

    def rope_tables(self):
        """(inv_freq float32 [D/2], axis int32 [D/2]) for kernels that rotate by themselves."""
        return self.inv_freq, self.axis

    def prompt_positions(self, num_tokens: int, image_spans):
        """Positions [3, num_tokens] of a prompt whose image runs are ``(start, t, h, w)``."""
        return prompt_positions(num_tokens, image_spans)[0]

    def rotate_and_store(self, ctx, qkv, nq, nkv, head_dim, kv):
        """kv: the pages and slots of the stop's cache group, or None to store nothing."""
        if head_dim != self.head_dim:
            raise ValueError(f"mrope built for head size {self.head_dim}, mixer has {head_dim}")
        angles = None
        if ctx.dtype == torch.bfloat16:
            # the angles are the same for every layer of the step that shares the tables: the first
            # one to ask computes them (the 32-bit path computes them in place, in every layer)
            key = ("rope_angles", self.inv_freq.data_ptr(), self.axis.data_ptr())
            angles = ctx.shared.get(key)
            if angles is None:
                angles = ctx.shared[key] = kernels.rope_angles(ctx.positions, self.inv_freq, self.axis)
        if kv is None:
            kernels.rope_store(qkv, ctx.positions, self.inv_freq, self.axis, None, None, None, nq, nkv, head_dim, 1, angles)
        else:
            kernels.rope_store(qkv, ctx.positions, self.inv_freq, self.axis, kv.k_pages, kv.v_pages, kv.kv_slot,
                               nq, nkv, head_dim, kv.page_size, angles)


@register_position_encoding("token_index")
class TokenIndex(PositionEncoding):
    """A token's position is its index in the request, on one axis, and nothing is done to queries
    and keys: a model whose positions enter elsewhere (a learned vector at the embedding, a bias on
    the attention scores).  ``rotate_and_store`` only writes the step's keys and values."""

    graph_safe = True
    axes = 1
    default_is_linear = True

    def __init__(self, limit=None):
        """``limit``: how many positions the model can place (a table of learned vectors ends there)."""
        self.limit = None if limit is None else int(limit)

    def default_positions(self, start: int, count: int, offset: int):
        return np.arange(start + offset, start + offset + count, dtype=np.int64)[None, :]

    def rotate_and_store(self, ctx, qkv, nq, nkv, head_dim, kv):
        if kv is not None:
            kernels.rope_store(qkv, None, None, None, kv.k_pages, kv.v_pages, kv.kv_slot, nq, nkv, head_dim, kv.page_size)


def rotary_frequencies(dims: int, base: float, scaling=None):
    """(frequencies [dims / 2] in float64, magnitude) of a rotary encoding: ``f_i = base^(-2i/dims)``,
    optionally scaled for contexts beyond the length the model was trained at.  ``scaling`` is None or
    a dict with ``kind``:

    * ``"wavelength"`` (the rule of Llama 3.1): with wavelength ``l = 2 pi / f``, ``f`` is kept where
      ``l < original / high``, divided by ``factor`` where ``l > original / low``, and in between
      ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``; magnitude 1;
    * ``"ramp"`` (YaRN: Peng, Quesnelle, Fan, Shippole, "YaRN: Efficient Context Window Extension of
      Large Language Models"): with ``pair(t) = dims ln(original / (2 pi t)) / (2 ln base)``, the pair
      that turns t times within the original length, ``lo = max(floor(pair(fast)), 0)``,
      ``hi = min(ceil(pair(slow)), dims - 1)`` and ``r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``,
      the frequency is ``r_i f / factor + (1 - r_i) f``; cos and sin are multiplied by
      ``0.1 ln(factor) + 1``."""
    import math

    half = dims // 2
    freqs = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return np.asarray(freqs, dtype=np.float64), 1.0
    kind = scaling.get("kind")
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if kind == "wavelength":
        low, high = float(scaling["low"]), float(scaling["high"])
        out = []
        for f in freqs:
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                out.append(f)
            elif wavelength > original / low:
                out.append(f / factor)
            else:
                s = (original / wavelength - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        return np.asarray(out, dtype=np.float64), 1.0
    if kind == "ramp":
        pair = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))
        lo = max(math.floor(pair(float(scaling["fast"]))), 0)
        hi = min(math.ceil(pair(float(scaling["slow"]))), dims - 1)
        out = []
        for i, f in enumerate(freqs):
            r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / factor * r + f * (1.0 - r))
        return np.asarray(out, dtype=np.float64), 0.1 * math.log(factor) + 1.0
    raise ValueError(f"unknown rotary scaling kind {kind!r}; known: wavelength, ramp")


@register_position_encoding("rotary")
class Rotary(PositionEncoding):
    """Rotary positions on one axis for the first ``dims`` channels of a head (the rest pass), with
    either pairing of channels: ``layout`` ``"interleaved"`` turns channel 2i with 2i + 1,
    ``"halves"`` channel i with i + dims / 2; the pair (u, v) at position p becomes
    ``(u cos a - v sin a, v cos a + u sin a)``, ``a = p f_i``.  ``scaling``: see
    :func:`rotary_frequencies`.  Positions and angles are float32 in both dtypes; a step's angles
    are computed once and shared by every layer with the same table.

    A mixer applies it itself where its layout wants it: ``angles(ctx)`` gives the step's table
    [N, dims / 2, 2] of (cos, sin), ``rotate(ctx, src, dst, width)`` turns [N, heads, width] views."""

    graph_safe = True
    axes = 1
    default_is_linear = True

    def __init__(self, dims: int, base: float, layout: str = "interleaved", scaling=None):
        self.dims, self.base, self.layout = int(dims), float(base), layout
        if self.dims < 0 or self.dims % 2:
            raise ValueError(f"a rotary encoding turns an even number of channels, got {dims}")
        if layout not in kernels.ROTARY_LAYOUTS:
            raise ValueError(f"unknown rotary layout {layout!r}; known: {sorted(kernels.ROTARY_LAYOUTS)}")
        self.scaling = dict(scaling) if scaling else None
        freqs, self.magnitude = rotary_frequencies(self.dims, self.base, self.scaling)
        self._freqs = freqs.astype(np.float32)
        self.inv_freq = None

    def load(self, tensors, device, dtype):
        self.inv_freq = torch.from_numpy(self._freqs).to(device)

    def default_positions(self, start: int, count: int, offset: int):
        return np.arange(start + offset, start + offset + count, dtype=np.int64)[None, :]

    def angles(self, ctx):
        """(cos, sin) of the step's positions, float32 [N, dims / 2, 2]; None when nothing turns."""
        if self.dims == 0:
            return None
        key = ("rotary_angles", id(self))
        table = ctx.shared.get(key)
        if table is None:
            table = ctx.shared[key] = kernels.rotary_angles(ctx.positions[0], self.inv_freq, self.magnitude)
        return table

    def rotate(self, ctx, src, dst, width: int):
        """[N, heads, >= width] views: ``width`` channels of every head of ``src`` go to ``dst`` (which
        may be ``src``), the first ``dims`` of them turned."""
        if self.dims > width:
            raise ValueError(f"the encoding turns {self.dims} channels, the head part has {width}")
        if self.dims == 0 and dst is src:
            return
        kernels.rotary_apply(src, dst, src.shape[1], width, self.angles(ctx) if self.dims else
                             torch.empty((src.shape[0], 0, 2), dtype=torch.float32, device=src.device), self.layout)
