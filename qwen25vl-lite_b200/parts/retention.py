"""Retention: linear attention with a fixed decay per head and neither softmax nor denominator
(Sun, Dong, Huang, Ma, Xia, Xue, Wang, Wei, "Retentive Network: A Successor to Transformer for Large
Language Models").

``q = Wq h``, ``k = Wk h`` (heads x dim), ``v = Wv h`` (heads x value_dim), no biases.  The layer's
position encoding turns q and k; then k is multiplied by ``dim^(-1/2)``.  Per head, from S = 0,

    S_t = decay_h S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t,

each head's o is divided by its root mean square (no weight), the heads are concatenated, multiplied
by ``silu(Wg h)`` and projected by ``Wo``.

What is float32 in both dtypes: the rotation, k's scale, S, o, the unit norm and the gate's product.
A request's state is S, one float32 tensor [heads, dim, value_dim] per slot, zero at admission and
carried from step to step, so a run of tokens may be cut anywhere.  Single tokens and short runs are
walked token by token; a long run is cut into chunks that are computed in parallel (``csrc/retention.cu``).
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..ops import kernels
from ..ops.linear import Linear
from .base import Mixer, StateNeed, TensorSpec, register_mixer


@register_mixer("retention")
class Retention(Mixer):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_residual = True          # the output projection can add into the residual stream itself

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay: Sequence[float], norm_eps: float,
                 position=None):
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.decay_values = tuple(float(d) for d in decay)
        if len(self.decay_values) != self.num_heads:
            raise ValueError(f"{self.num_heads} heads need {self.num_heads} decays, got {len(self.decay_values)}")
        self.norm_eps = float(norm_eps)
        self.position = position
        if position is not None and position.dims > self.head_dim:
            raise ValueError(f"the position encoding turns {position.dims} channels, a head has {head_dim}")
        self.in_proj = self.o_proj = self.decay = None

    def tensor_specs(self):
        h, qk, v = self.hidden_size, self.num_heads * self.head_dim, self.num_heads * self.value_dim
        return (TensorSpec("q", (qk, h)), TensorSpec("k", (qk, h)), TensorSpec("v", (v, h)), TensorSpec("g", (v, h)),
                TensorSpec("o", (h, v)))

    def state_need(self):
        return StateNeed((self.num_heads, self.head_dim, self.value_dim), "float32")

    def load(self, tensors, device, dtype):
        w = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0)
        self.in_proj = Linear(w.to(device=device, dtype=dtype).contiguous())
        self.o_proj = Linear(tensors["o"].to(device=device, dtype=dtype).contiguous())
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)

    def plan_key(self):
        return ("retention",)                 # the chunks of a step's long runs do not depend on a layer's sizes

    def plan_step(self, host):
        chunks, runs, short = kernels.plan_retention(host.q_lens)
        return {"chunks": np.asarray(chunks, dtype=np.int32).reshape(-1), "runs": np.asarray(runs, dtype=np.int32).reshape(-1),
                "short": np.asarray([1] if short and chunks else [], dtype=np.int32)}

    def forward(self, ctx, h, stop, residual=None):
        H, D, Dv = self.num_heads, self.head_dim, self.value_dim
        plan = ctx.plan(self)
        x = self.in_proj(h)                                          # [N, q | k | v | g]
        angles = self.position.angles(ctx) if self.position is not None else None
        layout = self.position.layout if self.position is not None else "halves"
        out = torch.empty((h.shape[0], H * Dv), dtype=x.dtype, device=x.device)
        kernels.retention(x, 0, H * D, 2 * H * D, 2 * H * D + H * Dv, angles, layout, self.decay, stop.state, ctx.cu_q, ctx.slot_ids,
                          out, ctx.n_seqs, ctx.max_q_len, H, D, Dv, float(D) ** -0.5, self.norm_eps, plan.get("chunks"), plan.get("runs"),
                          scan_too=plan.get("chunks") is None or plan.get("short") is not None)
        return self.o_proj(out, residual=residual)
