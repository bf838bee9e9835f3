"""Gated linear recurrent mixer: the recurrent block of Griffin (De, Smith, Fernando, Botev et al.,
"Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language Models") with
its real-gated linear recurrent unit.

Two branches of ``width`` channels from one product: ``y = gelu_tanh(Wy h + by)`` and
``xin = Wx h + bx``, the latter through a causal per-channel convolution of ``conv`` taps to u.  The
channels are cut into ``blocks`` equal parts; in each, two gates from square matrices,
``r = sigmoid(Ra u + ba)`` and ``i = sigmoid(Ri u + bi)``.  Then per channel
``a = exp(-gain * r * softplus(lam))`` and ``S_t = a S_(t-1) + sqrt(1 - a^2) * i * u`` from S = 0, and
the mixer returns ``Wo (S * y)``.

What is float32 in both dtypes: u, the gates and their products (plain FMA chains, so that a
token's gates do not depend on the batch), the decay, S.  The request's state is S and the last
``conv - 1`` inputs of the convolution, one float32 tensor [conv, width] per slot, zero at
admission (the zeros before the start), carried from step to step.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import Linear
from .base import Mixer, StateNeed, TensorSpec, register_mixer


@register_mixer("rglru")
class RGLRU(Mixer):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, hidden_size: int, width: int, blocks: int, conv: int, gain: float = 8.0, position=None):
        self.hidden_size, self.width, self.blocks, self.conv = int(hidden_size), int(width), int(blocks), int(conv)
        self.gain = float(gain)
        if self.blocks < 1 or self.width % self.blocks:
            raise ValueError(f"{width} channels cannot be cut into {blocks} equal blocks")
        if not 1 <= self.conv <= 16:
            raise ValueError(f"the convolution takes 1 to 16 taps, got {conv}")
        self.in_proj = self.out_proj = None

    def tensor_specs(self):
        h, w, b = self.hidden_size, self.width, self.blocks
        bw = w // b
        return (TensorSpec("y", (w, h)), TensorSpec("y.b", (w,), "bias"), TensorSpec("x", (w, h)), TensorSpec("x.b", (w,), "bias"),
                TensorSpec("conv", (w, self.conv), "matrix_wide"), TensorSpec("conv.b", (w,), "bias"),
                TensorSpec("ra", (b, bw, bw), "matrix_wide"), TensorSpec("ra.b", (b, bw), "bias"),
                TensorSpec("ri", (b, bw, bw), "matrix_wide"), TensorSpec("ri.b", (b, bw), "bias"),
                TensorSpec("lam", (w,), "bias"), TensorSpec("o", (h, w)))

    def state_need(self):
        return StateNeed((self.conv, self.width), "float32")

    def load(self, tensors, device, dtype):
        f32 = lambda name: tensors[name].to(device=device, dtype=torch.float32).contiguous()
        w = torch.cat([tensors["y"], tensors["x"]], dim=0).to(device=device, dtype=dtype).contiguous()
        b = torch.cat([tensors["y.b"], tensors["x.b"]], dim=0).to(device=device, dtype=torch.float32).contiguous()
        self.in_proj = Linear(w, b)
        self.out_proj = Linear(tensors["o"].to(device=device, dtype=dtype).contiguous())
        self.conv_w, self.conv_b = f32("conv"), f32("conv.b")
        self.ra, self.ra_b, self.ri, self.ri_b, self.lam = f32("ra"), f32("ra.b"), f32("ri"), f32("ri.b"), f32("lam")

    def forward(self, ctx, h, stop):
        n, w = h.shape[0], self.width
        yx = self.in_proj(h)                                    # [N, 2 width]: the y branch, then the convolution's input
        u = torch.empty((n, w), dtype=torch.float32, device=h.device)
        kernels.rglru_conv(yx, w, self.conv_w, self.conv_b, stop.state, ctx.token_seq, ctx.cu_q, ctx.slot_ids, u)
        a, bx = torch.empty_like(u), torch.empty_like(u)
        kernels.rglru_gates(u, self.ra, self.ra_b, self.ri, self.ri_b, self.lam, self.gain, a, bx)
        out = torch.empty((n, w), dtype=ctx.dtype, device=h.device)
        kernels.rglru_scan(a, bx, yx, 0, w, stop.state, ctx.cu_q, ctx.slot_ids, out, ctx.n_seqs, ctx.max_q_len)
        return self.out_proj(out)
