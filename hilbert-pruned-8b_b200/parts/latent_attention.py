"""Attention whose keys and values are made from one small latent per token.

Per token, from the mixer's input ``h``: ``q = Wq h`` (heads x [d unrotated | dr rotated]); ``Wdkv h`` has
``rank + dr`` rows: the first ``rank``, divided by their root mean square and multiplied by a weight, are the
latent ``c``; the last ``dr`` are one key part that every head shares and that is rotated by position, as
are the queries' last ``dr`` dimensions (pairs ``(2i, 2i + 1)`` of the first ``rotary_dim`` of them).  Head
h's unrotated key is ``Wuk_h c`` and its value ``Wuv_h c``; its score for a key is ``(q_u . k_u + q_r . k_r)
* scale``; causal softmax; the head's result times ``sigmoid(Wg h)_h`` (``head_gate``); output projection.

Only ``c`` and the rotated key part are cached.  The up projections are folded around the attention
instead of being applied to the cache: with ``q'_h = [Wuk_h^T q_u | q_r]`` the score is ``q'_h . [c | k_r]``
and the head's result is ``Wuv_h (sum_s p_s c_s)``, which is attention with ONE key/value head whose key row
is ``[c | k_r]`` and whose value row is ``c``, between two small products per head.  The attention itself is
the library's softmax attention over a paged cache group (``softmax_attention``), with 32-bit results.

That folded form is what a step of few tokens runs (decoding: the cache is read once, for all heads).  A bfloat16
step that brings many tokens writes the keys and values of every head out instead, for its sequences from their
first token on, into a scratch cache of the ordinary paged layout with as many key/value heads as heads: key
``[Wuk_h c | k_r]`` of ``d + dr`` numbers, value ``Wuv_h c``, each padded with zeros to a head size the tensor-core
prompt kernel is built for (``written_out``).  The products of the attention are then several times smaller than
with ``rank + dr`` numbers per key, and the two per-head products become one ordinary matrix product.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import MIXERS, POSITION_ENCODINGS, CacheNeed, Mixer, ParamSpec
from .sink_attention import softmax_attention


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.d = int(p["head_dim"])                 # unrotated query/key dimensions per head
        self.dr = int(p["rotary_head_dim"])         # rotated ones
        self.dv = int(p["v_head_dim"])
        self.rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.head_gate = bool(p.get("head_gate", False))
        pos = p.get("position")
        self.position = ctx.shared_part(POSITION_ENCODINGS, pos) if pos is not None else None
        self.graph_safe = getattr(self.position, "graph_safe", True)
        H = self.heads
        self.q_width = H * (self.d + self.dr)
        self.down_at = self.q_width
        self.gate_at = self.down_at + self.rank + self.dr
        self.proj_width = self.gate_at + (H if self.head_gate else 0)
        self.proj_ld = (self.proj_width + 7) // 8 * 8
        self.key_dim = self.rank + self.dr
        # head sizes of the written-out form (multiples of 64, as the prompt kernel wants them)
        self.flat_d = (self.d + self.dr + 63) // 64 * 64
        self.flat_dv = (self.dv + 63) // 64 * 64
        self.write_out = True                 # tests switch it off to run every step in the folded form
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.c_weight = self.w_ukv = self.w_o_flat = None

    def params(self) -> List[ParamSpec]:
        H, W = self.heads, self.hidden
        out = [ParamSpec("q", (self.q_width, W)), ParamSpec("dkv", (self.rank + self.dr, W)),
               ParamSpec("dkv.norm", (self.rank,), kind="vector", init="ones"), ParamSpec("uk", (H * self.d, self.rank)),
               ParamSpec("uv", (H * self.dv, self.rank)), ParamSpec("o", (W, H * self.dv))]
        if self.head_gate:
            out.append(ParamSpec("g", (H, W)))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t, H = tensors, self.heads
        rows = [t["q"], t["dkv"]] + ([t["g"]] if self.head_gate else [])
        if len({r.dtype for r in rows}) != 1:
            raise ValueError("latent_attention: the input projections are stored in different dtypes")
        if self.proj_ld > self.proj_width:
            rows.append(torch.zeros(self.proj_ld - self.proj_width, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        pack = self.ctx.ops.pack_weight
        self.w_in = pack(torch.cat(rows, dim=0).contiguous())
        self.w_o = pack(t["o"].contiguous())
        # per head [inputs, outputs]: the key up-projection is stored that way already (it is applied transposed, to the query)
        self.w_uk = t["uk"].reshape(H, self.d, self.rank).contiguous()
        self.w_uv = t["uv"].reshape(H, self.dv, self.rank).transpose(1, 2).contiguous()
        self.c_weight = t["dkv.norm"].reshape(-1).to(torch.float32).contiguous()
        # the written-out form: [Wuk; Wuv] as one matrix, and the output projection with zero columns where values are padded
        self.w_ukv = pack(torch.cat([t["uk"], t["uv"]], dim=0).contiguous())
        if self.flat_dv == self.dv:
            self.w_o_flat = self.w_o
        else:
            o = torch.zeros(self.hidden, H, self.flat_dv, dtype=t["o"].dtype, device=t["o"].device)
            o[:, :, : self.dv] = t["o"].reshape(self.hidden, H, self.dv)
            self.w_o_flat = pack(o.reshape(self.hidden, H * self.flat_dv).contiguous())

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_uk, self.w_uv, self.w_o))

    def cache_need(self) -> CacheNeed:
        return CacheNeed(1, self.key_dim, None, v_head_dim=self.rank)

    def forward(self, h, residual, step, cache, state, append: bool, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        H, d, dr, dv, rank = self.heads, self.d, self.dr, self.dv, self.rank
        proj = ws.buffer("latent_attention.proj", (cap, self.proj_ld), torch.float32)[:T]
        ops.linear(h, self.w_in, proj)
        table, rot = None, 0
        if self.position is not None and dr:
            rotation = self.position.rotation_table(step)
            if rotation is None:
                raise ValueError("latent_attention: this mixer needs a position encoding that is a table of rotations")
            table, rot = rotation
        gate = proj[:, self.gate_at: self.gate_at + H] if self.head_gate else None
        if self.written_out(step):
            self._forward_written_out(proj, table, rot, gate, residual, step, cache, append, accumulate)
            return
        q = ws.buffer("latent_attention.q", (cap, H * self.key_dim), self.ctx.dtype)[:T]
        ops.latent_prepare(proj, H, d, dr, rank, self.down_at, self.c_weight, self.eps, table, rot, q, cache, step, append)
        ops.head_linear(proj, d + dr, self.w_uk, q, self.key_dim, d, rank)
        mixed = ws.buffer("latent_attention.mixed", (cap, H * rank), torch.float32)[:T]
        softmax_attention(self.ctx, q, H, 1, self.key_dim, rank, cache, step, self.scale, None, 0, mixed)
        attn = ws.buffer("latent_attention.out", (cap, H * dv), self.ctx.dtype)[:T]
        ops.head_linear(mixed, rank, self.w_uv, attn, dv, rank, dv, gate=gate)
        ops.linear(attn, self.w_o, residual, accumulate=accumulate)

    def written_out(self, step) -> bool:
        """Whether this step writes every head's keys and values out and runs the tensor-core prompt kernel on them."""
        return bool(self.write_out and self.ctx.dtype == torch.bfloat16 and self.ctx.ops.attention_sink_prefill_wanted(
            step, self.heads, self.heads, self.flat_d, self.flat_dv, self.ctx.dtype))

    def _forward_written_out(self, proj, table, rot, gate, residual, step, cache, append: bool, accumulate: bool) -> None:
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        H, d, dr, dv, rank, D, DV = self.heads, self.d, self.dr, self.dv, self.rank, self.flat_d, self.flat_dv
        q = ws.buffer("latent_attention.q_flat", (cap, H * D), torch.bfloat16)[:T]
        ops.latent_prepare(proj, H, d, dr, rank, self.down_at, self.c_weight, self.eps, table, rot, q, cache, step, append, whole_heads=D)
        pages = sum((n + 63) // 64 for n in step.host_len)
        width = (step.max_len + 63) // 64
        rows = ws.buffer("latent_attention.flat_c", (pages * 64, rank), torch.bfloat16)
        scratch_table = ws.buffer("latent_attention.flat_pages", (step.num_seqs, width), torch.int32)
        ops.latent_gather(cache, step, rank, rows, scratch_table)
        kv = ws.buffer("latent_attention.flat_kv", (pages * 64, H * (d + dv)), torch.bfloat16)
        ops.linear(rows, self.w_ukv, kv)
        flat = _WrittenOut(ws.buffer("latent_attention.flat_k", (pages, H, 64, D), torch.bfloat16),
                           ws.buffer("latent_attention.flat_v", (pages, H, 64, DV), torch.bfloat16), len(step.page_tables))
        ops.latent_scatter(kv, cache, step, H, d, dr, dv, rank, flat.k, flat.v)
        step.page_tables.append(scratch_table)              # the scratch cache is one more group of this step
        try:
            attn = ws.buffer("latent_attention.out_flat", (cap, H * DV), torch.bfloat16)[:T]
            softmax_attention(self.ctx, q, H, H, D, DV, flat, step, self.scale, None, 0, attn, gate=gate)
        finally:
            step.page_tables.pop()
        ops.linear(attn, self.w_o_flat, residual, accumulate=accumulate)


class _WrittenOut:
    """The scratch cache of one step: keys ``[pages, heads, 64, d]``, values ``[pages, heads, 64, dv]`` and the index of its
    page table among the step's."""

    def __init__(self, k, v, group: int):
        self.k, self.v, self.group = k, v, group
