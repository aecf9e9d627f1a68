"""Mixers built on a recurrent matrix memory per head whose decay depends on the token (the ``head_scan`` kernel).

``state_space_heads`` (the state-space duality form).  ``inner = heads * head_dim``, N = ``state``, G = ``groups``.
``W_in h = [z (inner) | x (inner) | B (G N) | C (G N) | dt (heads)]``.  x, B and C together pass a causal convolution per
channel (``conv`` ``[channels, taps]``, last column the current token's, bias ``conv.b``, zeros before the sequence's
start) and silu.  ``dt = softplus(dt + dt_bias)`` per head, unclamped.  Per head h (which reads group ``h // (heads / G)``):
``S <- exp(-exp(A_log_h) dt) S + dt B x^T`` (S is N x head_dim), ``y = S^T C + D_h x``.  The heads' y, side by side, times
``silu(z)``, then divided by the root mean square of each of ``norm_groups`` equal parts of the row, times ``norm``, then
``W_o``: the gate comes BEFORE the norm.  State per sequence, 32-bit, zero at the start: the convolution's last
``taps - 1`` inputs and S.

``gated_linear_attention``.  ``q = W_q h * dim^-1/2`` and ``k = W_k h`` (heads x dim), ``v = W_v h`` (heads x vdim); a decay
per key channel ``alpha = sigmoid(W_a2 (W_a1 h) + a2.b) ^ (1 / tau)``.  Per head ``S <- diag(alpha) S + k v^T``, ``o = S^T q``.
Each head's o is divided by its root mean square over vdim and multiplied by ``norm`` (size vdim, shared by the heads); the
heads side by side times ``silu(W_g h)``, then ``W_o``.  State: S, 32-bit, zero at the start.

32-bit: the projections' results as the convolution and the recurrence read them, step sizes, decays and their
logarithms, S, the recurrence's output, gates and norms.  What the output products read is in the activations' dtype.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import MIXERS, Mixer, ParamSpec, StateNeed


def _padded(rows: List[torch.Tensor], width: int, multiple: int = 8) -> torch.Tensor:
    """The matrices one below the other, with zero rows up to a multiple of ``multiple`` rows."""
    total = sum(r.shape[0] for r in rows)
    pad = (-total) % multiple
    if pad:
        rows = rows + [torch.zeros(pad, width, dtype=rows[0].dtype, device=rows[0].device)]
    return torch.cat(rows, dim=0).contiguous()


@MIXERS.register("state_space_heads")
class StateSpaceHeads(Mixer):
    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.head_dim = int(p["num_heads"]), int(p["head_dim"])
        self.n_state, self.groups = int(p["state"]), int(p.get("groups", 1))
        self.taps = int(p["conv"])
        self.norm_groups = int(p.get("norm_groups", 1))
        self.eps = float(p["eps"])
        self.inner = self.heads * self.head_dim
        if self.heads % self.groups:
            raise ValueError("state_space_heads: heads must be a multiple of groups")
        if self.inner % self.norm_groups:
            raise ValueError("state_space_heads: the row does not divide into norm_groups equal parts")
        if self.taps < 1:
            raise ValueError("state_space_heads: at least one convolution tap")
        self.conv_width = self.inner + 2 * self.groups * self.n_state
        self.proj_width = self.inner + self.conv_width + self.heads
        self.proj_ld = (self.proj_width + 7) // 8 * 8
        self.conv_state = (self.taps - 1) * self.conv_width
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm_weight = None

    def params(self) -> List[ParamSpec]:
        H, W = self.heads, self.hidden
        return [ParamSpec("in", (self.proj_width, W)), ParamSpec("conv", (self.conv_width, self.taps)),
                ParamSpec("conv.b", (self.conv_width,), kind="vector", init="zeros"), ParamSpec("dt_bias", (H,), kind="vector", init="zeros"),
                ParamSpec("A_log", (H,), kind="vector", init="zeros"), ParamSpec("D", (H,), kind="vector", init="ones"),
                ParamSpec("norm", (self.inner,), kind="vector", init="ones"), ParamSpec("o", (W, self.inner))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t, pack = tensors, self.ctx.ops.pack_weight
        f32 = lambda x: x.reshape(-1).to(torch.float32).contiguous()
        self.w_in = pack(_padded([t["in"]], self.hidden))
        self.w_o = pack(t["o"].contiguous())
        self.conv_w = t["conv"].reshape(self.conv_width, self.taps).to(torch.float32).contiguous()
        self.conv_b, self.dt_bias, self.a_log, self.d_skip, self.norm_weight = (f32(t[n]) for n in ("conv.b", "dt_bias", "A_log", "D", "norm"))

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o)) + 4 * (self.conv_w.numel() + self.conv_width + self.inner + 3 * self.heads)

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.conv_state + self.inner * self.n_state,), torch.float32)

    def forward(self, h, residual, step, cache, state, append: bool, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        I, GN = self.inner, self.groups * self.n_state
        proj = ws.buffer("state_space_heads.proj", (cap, self.proj_ld), torch.float32)[:T]
        ops.linear(h, self.w_in, proj)
        xbc = ws.buffer("state_space_heads.xbc", (cap, self.conv_width), torch.float32)[:T]
        ops.conv_act(proj[:, I: I + self.conv_width], self.conv_w, self.conv_b, state[:, : self.conv_state], step, xbc, "silu")
        y = ws.buffer("state_space_heads.y", (cap, I), torch.float32)[:T]
        dt_at = I + self.conv_width
        ops.head_scan(xbc[:, :I], xbc[:, I: I + GN], xbc[:, I + GN:], proj[:, dt_at: dt_at + self.heads], self.dt_bias,
                      state[:, self.conv_state:], step, y, self.heads, self.groups, self.head_dim, self.n_state, a_log=self.a_log,
                      skip=self.d_skip, z=proj[:, :I], workspace=ws)
        normed = ws.buffer("state_space_heads.normed", (cap, I), self.ctx.dtype)[:T]
        ops.gated_norm(y, None, self.norm_weight, self.eps, normed, group=I // self.norm_groups if self.norm_groups > 1 else None)
        ops.linear(normed, self.w_o, residual, accumulate=accumulate)


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.d, self.dv = int(p["num_heads"]), int(p["head_dim"]), int(p["v_head_dim"])
        self.tau = float(p["tau"])
        if not self.tau > 0.0:
            raise ValueError("gated_linear_attention: tau must be positive")
        self.eps = float(p["eps"])
        self.rank = int(p["decay_rank"])
        H, d, dv = self.heads, self.d, self.dv
        self.k_at, self.v_at, self.g_at = H * d, 2 * H * d, 2 * H * d + H * dv
        self.a_at = self.g_at + H * dv
        self.proj_width = self.a_at + self.rank
        self.proj_ld = (self.proj_width + 7) // 8 * 8
        self.w_in = self.w_a2 = self.w_o = self.a_bias = self.norm_weight = None

    def params(self) -> List[ParamSpec]:
        H, d, dv, W, R = self.heads, self.d, self.dv, self.hidden, self.rank
        return [ParamSpec("q", (H * d, W)), ParamSpec("k", (H * d, W)), ParamSpec("v", (H * dv, W)), ParamSpec("g", (H * dv, W)),
                ParamSpec("a1", (R, W)), ParamSpec("a2", (H * d, R)), ParamSpec("a2.b", (H * d,), kind="vector", init="zeros"),
                ParamSpec("norm", (dv,), kind="vector", init="ones"), ParamSpec("o", (W, H * dv))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t, pack = tensors, self.ctx.ops.pack_weight
        rows = [t["q"], t["k"], t["v"], t["g"], t["a1"]]
        if len({r.dtype for r in rows}) != 1:
            raise ValueError("gated_linear_attention: the input projections are stored in different dtypes")
        self.w_in = pack(_padded(rows, self.hidden))
        # the decay's second product reads the 32-bit low-rank values where the first product left them (the general product
        # takes a column range of a wider 32-bit matrix; its inner size is the small rank)
        self.w_a2 = t["a2"].contiguous()
        self.w_o = pack(t["o"].contiguous())
        self.a_bias = t["a2.b"].reshape(-1).to(torch.float32).contiguous()
        self.norm_weight = t["norm"].reshape(-1).to(torch.float32).repeat(self.heads).contiguous()     # one weight for every head

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_a2, self.w_o))

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.heads * self.d * self.dv,), torch.float32)

    def forward(self, h, residual, step, cache, state, append: bool, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        H, d, dv = self.heads, self.d, self.dv
        proj = ws.buffer("gated_linear_attention.proj", (cap, self.proj_ld), torch.float32)[:T]
        ops.linear(h, self.w_in, proj)
        low = proj[:, self.a_at: self.a_at + self.rank]
        a_raw = ws.buffer("gated_linear_attention.decay", (cap, H * d), torch.float32)[:T]
        ops.linear(low, self.w_a2, a_raw)
        o = ws.buffer("gated_linear_attention.o", (cap, H * dv), torch.float32)[:T]
        ops.head_scan(proj[:, self.v_at: self.v_at + H * dv], proj[:, self.k_at: self.k_at + H * d], proj[:, : H * d], a_raw, self.a_bias,
                      state, step, o, H, H, dv, d, inv_tau=1.0 / self.tau, q_scale=float(d) ** -0.5, workspace=ws)
        gated = ws.buffer("gated_linear_attention.gated", (cap, H * dv), self.ctx.dtype)[:T]
        ops.gated_norm(o, proj[:, self.g_at: self.g_at + H * dv], self.norm_weight, self.eps, gated, group=dv if H > 1 else None, gate_kind="silu")
        ops.linear(gated, self.w_o, residual, accumulate=accumulate)
