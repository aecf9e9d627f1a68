"""Mixture of experts with a clamped gated unit, and an optional shared expert.

Router: ``z = W_router h`` in 32-bit; the ``top`` experts with the largest logits are chosen per
token and weighted by the softmax over the chosen logits alone.  Expert (no biases):
``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``, ``y = g sigmoid(alpha g) (u + 1)``,
output ``W_down y``; ``alpha`` is 1.702 unless the spec says otherwise.  The layer's result is the
weighted sum of the chosen experts' outputs, plus the shared expert's (same form, own sizes and
limit), which runs for every token.

Options beside that form.  ``router`` "scores": scores are the softmax over ALL router outputs; the choice goes by
``score + correction`` (tensor ``correction``), only among the outputs of the ``keep`` best of ``groups`` equal runs of
neighbours (a run's score: its largest choice score; the others count as minus infinity); the weights are the chosen
outputs' scores, without the correction, divided by their sum ``+ 1e-20``.  ``identity`` n: the router's last n outputs are
identity experts, which hand the token's input back (times the weight) and have no tensors.  ``unit`` "gelu": an expert is
``W_down gelu(W_up h)`` with the exact (erf) gelu, no gate matrix.  ``shared_gate``: the shared expert's result is multiplied
by ``sigmoid(W_sg h)``, one number per token (tensor ``shared.sg`` ``[1, width]``).

Tensors below the part's prefix: ``router``, ``e<i>.gate|up|down``, ``shared.gate|up|down``.  The
experts' matrices are stacked at load time; the routed products gather their rows on the device
from a plan that a kernel makes, so a step reads nothing back and decode steps can be captured.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FEED_FORWARDS, FeedForward, ParamSpec


@FEED_FORWARDS.register("moe")
class MixtureOfExperts(FeedForward):
    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_experts = int(p["num_experts"])
        self.top = int(p["top"])
        self.ff = int(p["expert_size"])
        self.limit = float(p.get("limit", 0.0))
        self.alpha = float(p.get("alpha", 1.702))
        self.shared_ff = int(p.get("shared_size") or 0)
        self.shared_limit = float(p.get("shared_limit", self.limit))
        self.router = p.get("router", "top_logits")
        self.unit = p.get("unit", "clamped_glu")
        if self.router not in ("top_logits", "scores") or self.unit not in ("clamped_glu", "gelu"):
            raise ValueError(f"moe: router {self.router!r} ('top_logits' or 'scores'), unit {self.unit!r} ('clamped_glu' or 'gelu')")
        self.identity = int(p.get("identity") or 0)
        self.groups, self.keep = int(p.get("groups") or 1), int(p.get("keep") or 1)
        self.shared_gate = bool(p.get("shared_gate", False))
        self.n_outputs = self.n_experts + self.identity
        if (self.identity or self.groups > 1) and self.router != "scores":
            raise ValueError("moe: identity experts and groups belong to the router 'scores'")
        if self.n_outputs % self.groups or not 1 <= self.keep <= self.groups or self.top > self.n_outputs // self.groups * self.keep:
            raise ValueError(f"moe: {self.n_outputs} router outputs in {self.groups} groups, {self.keep} kept, top {self.top}")
        if not 1 <= self.top <= self.n_outputs:
            raise ValueError(f"moe: top {self.top} of {self.n_outputs} experts")
        self.correction = None
        self.gate_col = None
        self.w_router = self.w_gate = self.w_up = self.w_down = self.ws_gate_up = self.ws_down = None

    def params(self) -> List[ParamSpec]:
        W, F = self.hidden, self.ff
        glu = self.unit == "clamped_glu"
        out = [ParamSpec("router", (self.n_outputs, W))]
        if self.router == "scores":
            out.append(ParamSpec("correction", (self.n_outputs,), kind="vector", init="zeros"))
        for e in range(self.n_experts):
            out += ([ParamSpec(f"e{e}.gate", (F, W))] if glu else []) + [ParamSpec(f"e{e}.up", (F, W)), ParamSpec(f"e{e}.down", (W, F))]
        if self.shared_ff:
            S = self.shared_ff
            out += ([ParamSpec("shared.gate", (S, W))] if glu else []) + [ParamSpec("shared.up", (S, W)), ParamSpec("shared.down", (W, S))]
            if self.shared_gate:
                out.append(ParamSpec("shared.sg", (1, W)))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t, E = tensors, self.n_experts
        self.w_router = t["router"].to(torch.float32).contiguous()
        glu = self.unit == "clamped_glu"
        self.w_gate = torch.stack([t[f"e{e}.gate"] for e in range(E)]).contiguous() if glu else None
        self.w_up = torch.stack([t[f"e{e}.up"] for e in range(E)]).contiguous()
        self.w_down = torch.stack([t[f"e{e}.down"] for e in range(E)]).contiguous()
        if self.router == "scores":
            self.correction = t["correction"].reshape(-1).to(torch.float32).contiguous()
        if self.shared_ff:
            pack = self.ctx.ops.pack_weight
            rows = ([t["shared.gate"]] if glu else []) + [t["shared.up"]]
            if self.shared_gate:
                # the per-token gate is one more row of the shared expert's first product (zero rows up to 16 bytes)
                self.gate_col = sum(r.shape[0] for r in rows)
                rows.append(t["shared.sg"].reshape(1, self.hidden))
                pad = (-(self.gate_col + 1)) % 8
                if pad:
                    rows.append(torch.zeros(pad, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
            self.ws_gate_up = pack(torch.cat(rows, dim=0).contiguous())
            self.ws_down = pack(t["shared.down"].contiguous())

    def weight_bytes(self) -> int:
        # what a decode step of one token reads: the router, `top` experts, the shared expert
        per = (3 if self.w_gate is not None else 2) * self.ff * self.hidden * self.w_up.element_size()
        shared = sum(w.numel() * w.element_size() for w in (self.ws_gate_up, self.ws_down)) if self.shared_ff else 0
        return self.w_router.numel() * 4 + self.top * per + shared

    def forward(self, h, residual, step, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        experts = ws.buffer("moe.experts", (cap, self.top), torch.int32)[:T]
        weights = ws.buffer("moe.weights", (cap, self.top), torch.float32)[:T]
        if self.router == "scores":
            ops.moe_route_scores(h, self.w_router, self.correction, self.top, self.groups, self.keep, experts, weights)
        else:
            ops.moe_route(h, self.w_router, self.top, experts, weights)
        if self.unit == "gelu":
            ops.moe_experts(h, experts, weights, self.w_up, None, self.w_down, 0.0, 0.0, residual, accumulate, ws, cap,
                            tag=".gelu", identity=self.identity > 0)
        else:
            ops.moe_experts(h, experts, weights, self.w_gate, self.w_up, self.w_down, self.limit, self.alpha, residual, accumulate, ws, cap)
        if self.shared_ff:
            S = self.shared_ff
            first = self.ws_gate_up.shape[0]
            gu = ws.buffer(f"moe.shared_first.{first}", (cap, first), torch.float32)[:T]
            ops.linear(h, self.ws_gate_up, gu)
            act = ws.buffer("moe.shared_act", (cap, S), self.ctx.dtype)[:T]
            if self.unit == "gelu":
                # sigmoid(W_sg h) * (W_down act) = W_down (sigmoid(W_sg h) * act): the gate multiplies the rows the product reads
                ops.gelu_unit(gu, act, "erf", row_gate=self.gate_col)
            else:
                ops.glu_clamp(gu[:, : 2 * S], act, self.shared_limit, self.alpha)
            ops.linear(act, self.ws_down, residual, accumulate=True)
