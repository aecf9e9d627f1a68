"""SwiGLU feed-forward: ``residual += (silu(h Wg^T) * (h Wu^T)) Wd^T`` with
``silu(z) = z / (1 + exp(-z))`` (cleanroom-transformer/src/cpu_backend.c:247-251,
ops_common.h:56; shapes shapes.c:34-36).  Gate and up weights are concatenated row-wise so
that one matrix product (with the activation in its epilogue where the tensor-core kernel
applies) makes both.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FEED_FORWARDS, FeedForward, ParamSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        # the tensors' names below the part's prefix: (gate, up, down)
        self.names = tuple(spec.get("tensor_names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        self.w_gate_up = None
        self.w_down = None

    def params(self) -> List[ParamSpec]:
        return [
            ParamSpec(self.names[0], (self.inter, self.hidden)),
            ParamSpec(self.names[1], (self.inter, self.hidden)),
            ParamSpec(self.names[2], (self.hidden, self.inter)),
        ]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors[self.names[0]], tensors[self.names[1]]
        if g.dtype != u.dtype:
            raise ValueError("swiglu: gate and up projections are stored in different dtypes")
        pack = self.ctx.ops.pack_weight
        self.w_gate_up = pack(torch.cat([g, u], dim=0).contiguous(), swiglu=True)
        self.w_down = pack(tensors[self.names[2]].contiguous())

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    folds_norms = True
    can_overwrite = True        # forward(..., accumulate=False) writes its result instead of adding it

    def forward(self, h, residual, step, prepared=None, prepare=None, accumulate: bool = True):
        ops, ws, T = self.ctx.ops, self.ctx.workspace, step.num_tokens
        cap = self.ctx.max_step_tokens
        act = ws.buffer("swiglu.act", (cap, self.inter), self.ctx.dtype)[:T]
        ops.linear_swiglu(h, self.w_gate_up, act, ws, cap, scale=prepared)
        return ops.linear(act, self.w_down, residual, accumulate=accumulate, prepare=prepare if accumulate else None)


@FEED_FORWARDS.register("gated_gelu")
class GatedGelu(FeedForward):
    """``residual += Wd (gelu(Wg h) * (Wu h))`` with the tanh form of gelu, ``gelu(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715
    z^3)))``.  Gate and up weights are one matrix product with a 32-bit result; the activation reads it unrounded."""

    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.names = tuple(spec.get("tensor_names", ("gate", "up", "down")))
        self.w_gate_up = self.w_down = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec(self.names[0], (self.inter, self.hidden)), ParamSpec(self.names[1], (self.inter, self.hidden)),
                ParamSpec(self.names[2], (self.hidden, self.inter))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors[self.names[0]], tensors[self.names[1]]
        if g.dtype != u.dtype:
            raise ValueError("gated_gelu: gate and up projections are stored in different dtypes")
        rows = [g, u]
        pad = (-2 * self.inter) % 8
        if pad:
            rows.append(torch.zeros(pad, self.hidden, dtype=g.dtype, device=g.device))
        pack = self.ctx.ops.pack_weight
        self.w_gate_up = pack(torch.cat(rows, dim=0).contiguous())
        self.w_down = pack(tensors[self.names[2]].contiguous())

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, h, residual, step, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        first = self.w_gate_up.shape[0]
        gu = ws.buffer(f"gated_gelu.gate_up.{first}", (cap, first), torch.float32)[:T]
        ops.linear(h, self.w_gate_up, gu)
        act = ws.buffer("gated_gelu.act", (cap, self.inter), self.ctx.dtype)[:T]
        ops.gelu_unit(gu, act, "tanh_gated")
        ops.linear(act, self.w_down, residual, accumulate=accumulate)
