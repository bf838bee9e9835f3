"""Grouped-query softmax attention over the paged cache.

Reference (src/qwen25vl_lite/text.py:69-185): biased q/k/v projections, no bias on o
(:80-83); position encoding on q and k (:118); the step's k, v go into the pages before
the whole context is read back (:125-147); scores scaled by D^-1/2 (:78), query at
absolute index a sees keys j <= a (src/qwen25vl_lite/attention.py:366-372); query head h
reads kv head h // (nq / nkv) (attention.py:143-148).  ``window`` additionally hides keys
j <= a - window; the reference parses a window (src/qwen25vl_lite/config.py:93-94) but
never applies one.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import attention as attention_ops
from ..ops import kernels
from ..ops.linear import Linear
from .base import KVCacheNeed, Mixer, TensorSpec, register_mixer


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position,
                 qkv_bias: bool = True, out_bias: bool = False, window: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head size {head_dim} is not supported: the kernels take multiples of 16 up to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.position = position
        self.qkv_bias, self.out_bias = bool(qkv_bias), bool(out_bias)
        self.window = None if not window else int(window)
        self.scale = float(head_dim) ** -0.5
        self.rows_per_token = num_heads // num_kv_heads      # query heads that share one kv head
        self.graph_safe = True                               # forward is a fixed sequence of launches
        self.qkv_proj = None
        self.o_proj = None

    def tensor_specs(self):
        q, kv, h = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.hidden_size
        specs = [TensorSpec("q_proj.weight", (q, h)), TensorSpec("k_proj.weight", (kv, h)),
                 TensorSpec("v_proj.weight", (kv, h)), TensorSpec("o_proj.weight", (h, q))]
        if self.qkv_bias:
            specs += [TensorSpec("q_proj.bias", (q,), "bias"), TensorSpec("k_proj.bias", (kv,), "bias"),
                      TensorSpec("v_proj.bias", (kv,), "bias")]
        if self.out_bias:
            specs.append(TensorSpec("o_proj.bias", (h,), "bias"))
        return tuple(specs)

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def load(self, tensors, device, dtype):
        w = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0)
        b = None
        if self.qkv_bias:
            b = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]], dim=0)
            b = b.to(device=device, dtype=torch.float32).contiguous()
        self.qkv_proj = Linear(w.to(device=device, dtype=dtype).contiguous(), b)
        ob = tensors["o_proj.bias"].to(device=device, dtype=torch.float32).contiguous() if self.out_bias else None
        self.o_proj = Linear(tensors["o_proj.weight"].to(device=device, dtype=dtype).contiguous(), ob)

    accepts_deferred_norm = True     # forward takes a DeferredNorm as its input
    accepts_residual = True          # forward can add its result into the residual stream itself

    def plan_key(self):
        """Mixers with equal keys read the same work lists, which are then built once a step."""
        return ("gqa_attention", self.rows_per_token, self.num_kv_heads, bool(self.window))

    def plan_step(self, host):
        """The attention kernels' work lists for a step of this shape (int32 arrays by name)."""
        places = 2 * attention_ops.kernels.sm_count() // self.num_kv_heads      # two CTAs of the tcgen05 kernel fit an SM
        return attention_ops.plan_step(host, self.rows_per_token, self.window or 0, places)

    def forward(self, ctx, h, stop, residual=None):
        """Returns the update of the residual stream, or None after adding it into ``residual``."""
        qkv = self.qkv_proj(h)
        out = attention_ops.attend(ctx, ctx.plan(self), qkv, ctx.kv(stop), self.position, self.num_heads,
                                   self.num_kv_heads, self.head_dim, self.window, self.scale, stop.owns_cache)
        return self.o_proj(out, residual=residual)


@register_mixer("biased_window_attention")
class BiasedWindowAttention(Mixer):
    """Grouped-query softmax attention without rotation, whose positions enter as a bias on the
    scores: ``score = (q . k) * scale - r1[h] * ln(1 + r2[h] * (i - j))`` with two learned numbers per
    query head (``distance_bias``).  A sliding ``window`` beside which the first ``keep_first`` tokens
    of the request stay visible at their true distances (``j <= i and (i - j < window or j <
    keep_first)``; no window: all ``j <= i``).  Keys have ``head_dim`` channels, values
    ``value_dim``; q, k, v and the output projection carry biases.

    ``value_mix``: ``"source"`` offers this layer's values to the layers after it; ``"follower"``
    replaces its own by ``(1 - m) v + m v_source`` (m the layer's learned scalar ``vmix``, v_source the
    source layer's values of the same token) before they are cached and read.  Both kinds hold the
    scalar in a checkpoint; the source does not use it.  ``value_mix_key`` names the source among the
    tensors that the layers of one forward pass share."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: Optional[int] = None,
                 scale: Optional[float] = None, window: Optional[int] = None, keep_first: int = 0, distance_bias: bool = True,
                 value_mix: Optional[str] = None, value_mix_key: str = "first_values", position=None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads")
        if value_mix not in (None, "source", "follower"):
            raise ValueError(f"value_mix is None, 'source' or 'follower', got {value_mix!r}")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.value_dim = self.head_dim if value_dim is None else int(value_dim)
        if not 0 < self.value_dim <= 256 or self.head_dim <= 0:
            raise ValueError(f"key size {head_dim} / value size {value_dim} is not supported: values take up to 256 channels")
        self.scale = float(head_dim) ** -0.5 if scale is None else float(scale)
        self.window = None if not window else int(window)
        self.keep_first = int(keep_first) if self.window else 0
        self.distance_bias = bool(distance_bias)
        self.value_mix, self.value_mix_key = value_mix, value_mix_key
        self.qkv_proj = self.o_proj = self.r1 = self.r2 = None
        self.mix = 0.0

    def tensor_specs(self):
        q, k, v, h = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.num_kv_heads * self.value_dim, self.hidden_size
        specs = [TensorSpec("q", (q, h)), TensorSpec("q.b", (q,), "bias"), TensorSpec("k", (k, h)), TensorSpec("k.b", (k,), "bias"),
                 TensorSpec("v", (v, h)), TensorSpec("v.b", (v,), "bias")]
        # a layer that mixes nothing has no use for the scalar; a checkpoint that holds one all the same is accepted
        specs.append(TensorSpec("vmix", (), "fraction", optional=self.value_mix is None))
        if self.distance_bias:
            specs += [TensorSpec("r1", (self.num_heads,), "positive"), TensorSpec("r2", (self.num_heads,), "positive")]
        specs += [TensorSpec("o", (h, self.num_heads * self.value_dim)), TensorSpec("o.b", (h,), "bias")]
        return tuple(specs)

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, self.window, self.value_dim, self.keep_first)

    def load(self, tensors, device, dtype):
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        w = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0)
        b = torch.cat([tensors["q.b"], tensors["k.b"], tensors["v.b"]], dim=0)
        self.qkv_proj = Linear(w.to(device=device, dtype=dtype).contiguous(), f32(b))
        self.o_proj = Linear(tensors["o"].to(device=device, dtype=dtype).contiguous(), f32(tensors["o.b"]))
        if self.distance_bias:
            self.r1, self.r2 = f32(tensors["r1"]), f32(tensors["r2"])
        if self.value_mix == "follower":
            self.mix = float(tensors["vmix"].to(torch.float32))

    def plan_key(self):
        return ("biased_window_attention", self.num_heads // self.num_kv_heads, self.window or 0, self.keep_first)

    def plan_step(self, host):
        return attention_ops.plan_biased(host, self.num_heads // self.num_kv_heads, self.window or 0, self.keep_first)

    def forward(self, ctx, h, stop):
        nq, nkv, dk, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        qkv = self.qkv_proj(h)
        kv = ctx.kv(stop)
        other = None
        if self.value_mix == "follower":
            other = ctx.shared.get(self.value_mix_key)
            if other is None:
                raise RuntimeError("a layer mixes in the values of a source layer, but none ran before it in this pass")
        if stop.owns_cache:
            kernels.kv_store_mix(qkv, other, self.mix, kv.k_pages, kv.v_pages, kv.kv_slot, nq, nkv, dk, dv, kv.page_size)
        if self.value_mix == "source":
            ctx.shared[self.value_mix_key] = qkv[:, (nq + nkv) * dk:]
        out = attention_ops.attend_biased(ctx, ctx.plan(self), qkv, kv, nq, nkv, dk, dv, self.window, self.keep_first,
                                          self.scale, self.r1, self.r2)
        return self.o_proj(out)
