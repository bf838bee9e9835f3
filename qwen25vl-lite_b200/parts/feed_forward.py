"""SwiGLU feed-forward: ``down(silu(gate x) * up x)``, no biases
(reference src/qwen25vl_lite/text.py:56-66).  gate and up are held as one matrix so one
product feeds the activation; in the decode kernel the activation is its epilogue."""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels, linear
from ..ops.linear import DeferredNorm, Linear
from .base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_deferred_norm = True     # forward takes a DeferredNorm as its input
    accepts_residual = True          # forward can add its result into the residual stream itself

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.gate_up_proj = None
        self.down_proj = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return (TensorSpec("gate_proj.weight", (i, h)), TensorSpec("up_proj.weight", (i, h)),
                TensorSpec("down_proj.weight", (h, i)))

    def load(self, tensors, device, dtype):
        gate, up = tensors["gate_proj.weight"].to(device), tensors["up_proj.weight"].to(device)
        self.paired = self.intermediate_size % 8 == 0
        if self.paired:
            # rows in groups of 16: 8 gate features, then their 8 up features, so that the
            # weight-streaming kernel can form silu(gate) * up in its epilogue
            h = self.hidden_size
            gu = torch.stack([gate.reshape(-1, 8, h), up.reshape(-1, 8, h)], dim=1).reshape(2 * self.intermediate_size, h)
        else:
            gu = torch.cat([gate, up], dim=0)
        self.gate_up_proj = Linear(gu.to(dtype=dtype).contiguous())
        self.down_proj = Linear(tensors["down_proj.weight"].to(device=device, dtype=dtype).contiguous())

    def forward(self, ctx, h, residual=None):
        """Returns the update of the residual stream, or None after adding it into ``residual``."""
        act = torch.empty((h.shape[0], self.intermediate_size), dtype=ctx.dtype, device=h.device)
        w = self.gate_up_proj.weight
        deferred = isinstance(h, DeferredNorm)
        if self.paired and deferred and kernels.gemm_skinny_norm_supports(h.x, w):
            kernels.gemm_skinny_norm(h.x, h.weight, h.eps, w, None, act, kernels.SKINNY_SWIGLU)
        else:
            if deferred:
                h = h.materialize()
            if self.paired and kernels.gemm_skinny_supports(h, w):
                kernels.gemm_skinny(h, w, None, act, kernels.SKINNY_SWIGLU)
            elif self.paired and linear.use_tcgen05(h, w, fused_epilogue=True):
                kernels.gemm_tcgen05(h, w, None, act, kernels.SKINNY_SWIGLU)
            else:
                kernels.silu_mul(self.gate_up_proj(h), act, self.paired)
        return self.down_proj(act, residual=residual)


TCGEN05_MIN_WIDTH = 2048        # from this width on the grouped products of long steps run on tcgen05


@register_feed_forward("routed_glu")
class RoutedGLU(FeedForward):
    """A mixture of ``experts`` small gated feed-forwards of which each token uses ``top``, plus an
    optional shared one that every token uses.

    Router: ``z = Wr h`` in float32, scores ``sigmoid(z)``; the ``top`` largest are chosen and weigh
    in with their scores as they are (not renormalised).  The weight multiplies the expert's
    *input*: the routed part is the sum of ``expert(s_e * h)``.  An expert has no biases:
    ``g = min(Wg a, limit)``, ``u = clamp(Wu a, -limit, limit)``, ``Wd (g * sigmoid(alpha g) * (u + 1))``.
    The shared expert has the same form with sizes and limit of its own; its result is multiplied
    by ``sigmoid(wsg . h)``, one number per token.

    The pairs of a step are sorted by expert on the device and two grouped products walk them
    (``csrc/moe.cu``; in long bfloat16 steps of wide models the grouped mode of ``csrc/gemm_tcgen05.cu``);
    the host reads nothing back, so a step of single tokens can be captured."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, limit: float, alpha: float = 1.702,
                 shared_size: Optional[int] = None, shared_limit: Optional[float] = None):
        self.hidden_size, self.experts, self.top, self.expert_size = int(hidden_size), int(experts), int(top), int(expert_size)
        self.limit, self.alpha = float(limit), float(alpha)
        self.shared_size = None if not shared_size else int(shared_size)
        self.shared_limit = self.limit if shared_limit is None else float(shared_limit)
        if not 1 <= self.top <= min(self.experts, 16) or self.experts > 256:
            raise ValueError(f"the router takes up to 256 experts and chooses 1 to 16 of them, got {experts} and {top}")

    def tensor_specs(self):
        h, f = self.hidden_size, self.expert_size
        specs = []
        for e in range(self.experts):
            specs += [TensorSpec(f"e{e}.gate", (f, h)), TensorSpec(f"e{e}.up", (f, h)), TensorSpec(f"e{e}.down", (h, f))]
        specs.append(TensorSpec("router", (self.experts, h), "matrix_wide"))
        if self.shared_size:
            s = self.shared_size
            specs += [TensorSpec("shared.gate", (s, h)), TensorSpec("shared.up", (s, h)), TensorSpec("shared.down", (h, s)),
                      TensorSpec("shared.sg", (1, h))]
        return tuple(specs)

    def load(self, tensors, device, dtype):
        # an expert's gate rows and then its up rows, expert after expert: the layout that one grouped product reads whole
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0)
                                      for e in range(self.experts)]).to(device=device, dtype=dtype).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).to(device=device, dtype=dtype).contiguous()
        self.router = tensors["router"].to(device=device, dtype=torch.float32).contiguous()
        self.shared_gate = self.shared_gate_up = self.shared_down = None
        if self.shared_size:
            gu = torch.cat([tensors["shared.gate"], tensors["shared.up"]], dim=0)
            self.shared_gate_up = Linear(gu.to(device=device, dtype=dtype).contiguous())
            self.shared_down = Linear(tensors["shared.down"].to(device=device, dtype=dtype).contiguous())
            self.shared_gate = tensors["shared.sg"].reshape(-1).to(device=device, dtype=torch.float32).contiguous()

    def forward(self, ctx, h):
        n, top, experts = h.shape[0], self.top, self.experts
        pairs = n * top
        # rows of a tile of the grouped products, from the step's shape alone: 16 while an expert gets up to 16
        # rows on average (the product is then a stream of weights), 64 beyond, and in bfloat16 128 once an
        # expert gets 128 rows on average: on tcgen05 where the width and the sizes allow it, else mma.sync
        many = pairs >= 128 * experts and ctx.dtype == torch.bfloat16
        # measured, a 2,048-token prompt of six layers: width 2,048: 4.73 ms with mma.sync, 3.67 ms with tcgen05; width
        # 2,560: 6.59 and 5.70 ms; width 1,024 (a tile's walk over K is then short against its epilogue): 2.68 and 2.86 ms
        tcgen05 = (many and self.hidden_size >= TCGEN05_MIN_WIDTH
                   and kernels.gemm_tcgen05_grouped_supports(ctx.dtype, self.hidden_size, self.expert_size))
        tile = 16 if pairs <= 16 * experts else (128 if many else 64)
        rows = kernels.moe_max_rows(pairs, experts, tile)
        dev = h.device
        shared = None
        if self.shared_size:
            act = torch.empty((n, self.shared_size), dtype=ctx.dtype, device=dev)
            kernels.glu_clamped(self.shared_gate_up(h), act, self.shared_limit, self.alpha)
            shared = self.shared_down(act)
        # counts | cursor (zero) | plan | row of every pair | pair of every row
        n_plan = 2 + experts + rows // tile
        ints = torch.zeros(2 * experts + n_plan + pairs + rows, dtype=torch.int32, device=dev)
        counts, cursor = ints[:experts], ints[experts:2 * experts]
        plan = ints[2 * experts:2 * experts + n_plan]
        pair_row = ints[2 * experts + n_plan:2 * experts + n_plan + pairs]
        row_pair = ints[2 * experts + n_plan + pairs:]
        topk_idx = torch.empty((n, top), dtype=torch.int32, device=dev)
        topk_w = torch.empty((n, top), dtype=torch.float32, device=dev)
        sg = torch.empty(n, dtype=torch.float32, device=dev) if self.shared_size else None
        kernels.moe_route(h, self.router, self.shared_gate, top, topk_idx, topk_w, sg, counts)
        kernels.moe_sort(topk_idx, counts, cursor, plan, row_pair, pair_row, experts, tile)
        act = torch.empty((rows, self.expert_size), dtype=ctx.dtype, device=dev)
        y = torch.empty((rows, self.hidden_size), dtype=torch.float32, device=dev)
        if tcgen05:
            # long steps: the sorted rows, weighted; gate and up of every expert as one grouped product on tcgen05
            # (which finds its tiles in the plan on the device), the activation, and down the same way
            sorted_rows = torch.empty((rows, self.hidden_size), dtype=ctx.dtype, device=dev)
            kernels.moe_gather(h, row_pair, topk_w, top, sorted_rows)
            gate_up = torch.empty((rows, 2 * self.expert_size), dtype=ctx.dtype, device=dev)
            kernels.gemm_tcgen05_grouped(sorted_rows, self.w_gate_up, gate_up, plan)
            kernels.glu_clamped(gate_up, act, self.limit, self.alpha)
            kernels.gemm_tcgen05_grouped(act, self.w_down, y, plan)
        else:
            kernels.moe_gate_up(h, self.w_gate_up, act, plan, row_pair, topk_w, top, self.limit, self.alpha, tile)
            kernels.moe_down(act, self.w_down, y, plan, row_pair, pairs, top, tile)
        out = torch.empty((n, self.hidden_size), dtype=ctx.dtype, device=dev)
        kernels.moe_combine(y, pair_row, sg, shared, out, top)
        return out


@register_feed_forward("clamped_glu")
class ClampedGLU(FeedForward):
    """A dense gated feed-forward with clamped branches, no biases: ``g = min(Wg h, limit)``,
    ``u = clamp(Wu h, -limit, limit)``, ``Wd (g * sigmoid(alpha g) * (u + 1))``: the form of one expert of
    ``routed_glu``, used by every token.  gate and up are one product, and in bfloat16 the unit is that
    product's epilogue: in the weight-streaming kernel for steps of up to 8 rows, in the tcgen05 product for
    long steps; between the two a kernel of its own follows the library's product."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_residual = True          # the down projection can add into the residual stream itself

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.alpha = float(limit), float(alpha)
        self.gate_up_proj = self.down_proj = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return (TensorSpec("gate", (i, h)), TensorSpec("up", (i, h)), TensorSpec("down", (h, i)))

    def load(self, tensors, device, dtype):
        gate, up = tensors["gate"].to(device), tensors["up"].to(device)
        # bfloat16: rows in groups of 16 (8 gate features, then their 8 up features), so that the products' kernels
        # can form the unit in their epilogue, as for ``swiglu``
        self.paired = dtype == torch.bfloat16 and self.intermediate_size % 8 == 0
        if self.paired:
            h = self.hidden_size
            gu = torch.stack([gate.reshape(-1, 8, h), up.reshape(-1, 8, h)], dim=1).reshape(2 * self.intermediate_size, h)
        else:
            gu = torch.cat([gate, up], dim=0)
        self.gate_up_proj = Linear(gu.to(dtype=dtype).contiguous())
        self.down_proj = Linear(tensors["down"].to(device=device, dtype=dtype).contiguous())
        self.constants = torch.tensor([self.limit, self.alpha], dtype=torch.float32, device=device)     # what the fused epilogue reads

    def forward(self, ctx, h, residual=None):
        act = torch.empty((h.shape[0], self.intermediate_size), dtype=ctx.dtype, device=h.device)
        w = self.gate_up_proj.weight
        if self.paired and kernels.gemm_skinny_supports(h, w):
            kernels.gemm_skinny(h, w, self.constants, act, kernels.SKINNY_GLU)
        elif self.paired and linear.use_tcgen05(h, w, fused_epilogue=True):
            kernels.gemm_tcgen05(h, w, self.constants, act, kernels.SKINNY_GLU)
        else:
            kernels.glu_clamped(self.gate_up_proj(h), act, self.limit, self.alpha, self.paired)
        return self.down_proj(act, residual=residual)
