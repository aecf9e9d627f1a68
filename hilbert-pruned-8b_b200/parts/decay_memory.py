"""A matrix memory with a fixed decay per head (linear attention with exponential forgetting).

Per token, from the mixer's input ``h``: ``q = act(Wq h)``, ``k = act(Wk h)`` (heads x d),
``v = act(Wv h)`` (heads x dv), laid out head by head, ``act`` = silu.  Per head
``S_t = decay_h S_(t-1) + k_t v_t^T`` and ``o_t = S_t^T q_t``, with no other scale.  The heads'
``o`` are concatenated, divided TOGETHER by their root mean square, multiplied by a weight and by
``sigmoid(Wg h)``, and projected by ``Wo``.  ``S`` starts at zero, is 32-bit and is the
sequence's state; q, k, v stay 32-bit from the projection's accumulator to the recurrence.  The
four input projections are one matrix product with a 32-bit result.  ``output_scale`` multiplies
the mixer's result (applied, in 32-bit, to what the output product reads).

Options beside that form: ``activation`` "none"; ``position`` (a rotary part: the first dimensions of every
head of q and k are turned by the token's angles, after the activation); ``k_scale`` multiplies k after the
rotation; ``norm`` "heads" divides each head's ``o`` by its own root mean square instead of the whole row's;
``norm_weight`` False leaves the norm's weight out (no such tensor then); ``gate`` "silu" multiplies by
``silu(Wg h)`` instead of the sigmoid.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import MIXERS, POSITION_ENCODINGS, Mixer, ParamSpec, StateNeed


@MIXERS.register("decay_memory")
class DecayMemory(Mixer):
    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.d = int(p["head_dim"])
        self.dv = int(p["v_head_dim"])
        self.decay_values = [float(x) for x in p["decay"]]
        if len(self.decay_values) != self.heads:
            raise ValueError(f"decay_memory: {len(self.decay_values)} decays for {self.heads} heads")
        self.eps = float(p["eps"])
        self.activation = p.get("activation", "silu")
        self.output_scale = float(p.get("output_scale", 1.0))
        pos = p.get("position")
        self.position = ctx.shared_part(POSITION_ENCODINGS, pos) if pos is not None else None
        self.k_scale = float(p.get("k_scale", 1.0))
        self.norm = p.get("norm", "row")
        if self.norm not in ("row", "heads"):
            raise ValueError(f"decay_memory: norm {self.norm!r} ('row' or 'heads')")
        self.has_norm_weight = bool(p.get("norm_weight", True))
        self.gate = p.get("gate", "sigmoid")
        if self.gate not in ("sigmoid", "silu"):
            raise ValueError(f"decay_memory: gate {self.gate!r} ('sigmoid' or 'silu')")
        H, d, dv = self.heads, self.d, self.dv
        self.gate_at = 2 * H * d + H * dv
        self.proj_width = self.gate_at + H * dv
        self.proj_ld = (self.proj_width + 7) // 8 * 8
        self.w_in = self.w_o = self.norm_weight = self.decay = None

    def params(self) -> List[ParamSpec]:
        H, d, dv, W = self.heads, self.d, self.dv, self.hidden
        out = [ParamSpec("q", (H * d, W)), ParamSpec("k", (H * d, W)), ParamSpec("v", (H * dv, W)), ParamSpec("g", (H * dv, W)),
               ParamSpec("o", (W, H * dv))]
        if self.has_norm_weight:
            out.append(ParamSpec("norm", (H * dv,), kind="vector", init="ones"))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = tensors
        rows = [t["q"], t["k"], t["v"], t["g"]]
        if len({r.dtype for r in rows}) != 1:
            raise ValueError("decay_memory: the input projections are stored in different dtypes")
        if self.proj_ld > self.proj_width:
            rows.append(torch.zeros(self.proj_ld - self.proj_width, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        pack = self.ctx.ops.pack_weight
        self.w_in = pack(torch.cat(rows, dim=0).contiguous())
        self.w_o = pack(t["o"].contiguous())
        self.norm_weight = t["norm"].reshape(-1).to(torch.float32).contiguous() if self.has_norm_weight else None
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rows[0].device)

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.heads * self.d * self.dv,), torch.float32)

    def forward(self, h, residual, step, cache, state, append: bool, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        H, d, dv = self.heads, self.d, self.dv
        proj = ws.buffer("decay_memory.proj", (cap, self.proj_ld), torch.float32)[:T]
        ops.linear(h, self.w_in, proj)
        o = ws.buffer("decay_memory.o", (cap, H * dv), torch.float32)[:T]
        table, rot = None, 0
        if self.position is not None:
            rotation = self.position.rotation_table(step)
            if rotation is None:
                raise ValueError("decay_memory: this mixer needs a position encoding that is a table of rotations")
            table, rot = rotation
        ops.decay_memory(proj, self.decay, state, step, o, H, d, dv, self.activation, table=table, rot=rot, k_scale=self.k_scale)
        gated = ws.buffer("decay_memory.gated", (cap, H * dv), self.ctx.dtype)[:T]
        ops.gated_norm(o, proj[:, self.gate_at: self.gate_at + H * dv], self.norm_weight, self.eps, gated, self.output_scale,
                       group=dv if self.norm == "heads" else None, gate_kind=self.gate)
        ops.linear(gated, self.w_o, residual, accumulate=accumulate)
