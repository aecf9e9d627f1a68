"""Grouped-query attention with a sliding window that keeps the sequence's first tokens, and
the options that go with it here: biases on the projections, queries and keys divided by their
root mean square after the rotation (or, ``qk_norm_weight``, divided by it and multiplied by a weight
of the head's size, shared by the heads, BEFORE the rotation), key and value heads of different sizes,
softmax weights mixed between the heads, values mixed with those of an earlier layer, and
(``head_gate``) each head's result multiplied by ``sigmoid(Wg h)_head``, one number per token and head,
before the output projection.  ``out_bias`` (default: as ``bias``) says whether the output projection has
a bias too.  ``chunk`` (instead of a window): positions are cut into runs of ``chunk`` from the sequence's start and a query
sees only the keys of its own run.  ``sink``: a learned number per head (tensor ``sink``) whose exponential is one more
term of the softmax's sum, with no key and no value.  ``v_from_k``: no value projection; the values are the keys as
projected (bias included, before norm and rotation).  ``rotary_pairs`` "interleaved": the rotation turns the pairs
``(2i, 2i + 1)`` instead of ``(i, i + rot/2)``.

Per token: ``q, k, v = Wq h + bq, Wk h + bk, Wv h + bv``; the position encoding turns q and k;
``q`` and ``k`` of every head are divided by ``sqrt(mean(x^2) + eps)`` (``qk_unit_norm``); with
``v_mix = "mix"`` the values become ``(1 - l) v + l v_first`` where ``v_first`` are the values that
the layer with ``v_mix = "first"`` made for the same token (same ``v_mix_key``); ``k`` and the
mixed ``v`` go to the cache.  Query at position p sees key s if ``s <= p`` and (``p - s < window``
or ``s < keep_first``).  ``P_g`` = softmax over the visible keys of ``q_g . k * scale``; with a
``talk`` matrix T head h uses ``sum_g T[h, g] P_g`` on the values of its own key/value head,
which is computed as the same mix of the sums ``P_g V`` for every value head.  The output
projection's bias rides along as one more column of its weight (the attention output carries a
column of ones), so the product adds it on the way into the residual stream.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import MIXERS, POSITION_ENCODINGS, CacheNeed, Mixer, ParamSpec

_BIAS_PAD = 8       # columns added to the output projection: the bias and zeros up to 16 bytes of bfloat16


@MIXERS.register("sink_attention")
class SinkAttention(Mixer):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.v_dim = int(p.get("v_head_dim") or self.head_dim)
        self.window: Optional[int] = p.get("window")
        self.chunk = int(p.get("chunk") or 0)
        if self.chunk and (self.window is not None or p.get("keep_first")):
            raise ValueError("attention: chunks come without a window and kept first tokens")
        self.sink = bool(p.get("sink", False))
        self.v_from_k = bool(p.get("v_from_k", False))
        self.interleaved = p.get("rotary_pairs", "halves") == "interleaved"
        if p.get("rotary_pairs", "halves") not in ("halves", "interleaved"):
            raise ValueError(f"attention: rotary_pairs {p.get('rotary_pairs')!r} ('halves' or 'interleaved')")
        self.keep_first = int(p.get("keep_first") or 0)
        self.scale = float(p["scale"]) if p.get("scale") is not None else float(self.head_dim) ** -0.5
        self.bias = bool(p.get("bias", False))
        self.qk_unit_norm = bool(p.get("qk_unit_norm", False))
        self.qk_norm_weight = bool(p.get("qk_norm_weight", False))
        if self.qk_unit_norm and self.qk_norm_weight:
            raise ValueError("attention: queries and keys get one norm, behind the rotation or in front of it")
        self.head_gate = bool(p.get("head_gate", False))
        self.out_bias = bool(p.get("out_bias", p.get("bias", False)))
        self.eps = float(p.get("eps", 1e-6))
        self.talk = bool(p.get("talk", False))
        self.v_mix = p.get("v_mix")                      # None | "first" | "mix"
        if self.v_mix not in (None, "first", "mix"):
            raise ValueError(f"attention: v_mix {self.v_mix!r} (None, 'first' or 'mix')")
        self.v_mix_key = "v_first:" + str(p.get("v_mix_key", ""))
        if self.heads % self.kv_heads:
            raise ValueError("attention: heads must be a multiple of kv heads")
        if self.v_from_k and (self.v_dim != self.head_dim or self.v_mix is not None):
            raise ValueError("attention: values that are the keys have the keys' size and are not mixed")
        pos = p.get("position")
        self.position = ctx.shared_part(POSITION_ENCODINGS, pos) if pos is not None else None
        self.graph_safe = getattr(self.position, "graph_safe", True)
        self.q_width, self.k_width, self.v_width = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.kv_heads * self.v_dim
        self.gate_at = self.q_width + self.k_width + (0 if self.v_from_k else self.v_width)
        self.proj_width = self.gate_at + (self.heads if self.head_gate else 0)
        self.proj_ld = (self.proj_width + 7) // 8 * 8
        self.out_width = self.heads * self.v_dim
        self.w_qkv = self.w_o = self.b_qkv = self.talk_matrix = self.v_lambda = self.norm_weights = self.sink_logits = None
        self.use_heads_kernel = True          # tests switch it off to run the general kernel instead

    def params(self) -> List[ParamSpec]:
        W = self.hidden
        out = [ParamSpec("q", (self.q_width, W)), ParamSpec("k", (self.k_width, W))]
        out += [] if self.v_from_k else [ParamSpec("v", (self.v_width, W))]
        out.append(ParamSpec("o", (W, self.out_width)))
        if self.bias:
            out += [ParamSpec("q.b", (self.q_width,), kind="vector", init="zeros"), ParamSpec("k.b", (self.k_width,), kind="vector", init="zeros")]
            out += [] if self.v_from_k else [ParamSpec("v.b", (self.v_width,), kind="vector", init="zeros")]
        if self.sink:
            out.append(ParamSpec("sink", (self.heads,), kind="vector", init="zeros"))
        if self.out_bias:
            out.append(ParamSpec("o.b", (W,), kind="vector", init="zeros"))
        if self.qk_norm_weight:
            out += [ParamSpec("q.norm", (self.head_dim,), kind="vector", init="ones"), ParamSpec("k.norm", (self.head_dim,), kind="vector", init="ones")]
        if self.head_gate:
            out.append(ParamSpec("g", (self.heads, W)))
        if self.talk:
            out.append(ParamSpec("talk", (self.heads, self.heads)))
        if self.v_mix is not None:
            # the layer that only provides the first values stores the scalar too and never reads it
            out.append(ParamSpec("vmix", (), kind="vector", init="zeros", optional=self.v_mix == "first"))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = tensors
        q, k, o = t["q"], t["k"], t["o"]
        v = None if self.v_from_k else t["v"]
        if q.dtype != k.dtype or (v is not None and v.dtype != q.dtype):
            raise ValueError("attention: q, k and v projections are stored in different dtypes")
        rows = [q, k] + ([] if v is None else [v]) + ([t["g"]] if self.head_gate else [])
        if len({r.dtype for r in rows}) != 1:
            raise ValueError("attention: the input projections are stored in different dtypes")
        if self.proj_ld > self.proj_width:
            rows.append(torch.zeros(self.proj_ld - self.proj_width, self.hidden, dtype=q.dtype, device=q.device))
        pack = self.ctx.ops.pack_weight
        self.w_qkv = pack(torch.cat(rows, dim=0).contiguous())
        if self.bias:
            biases = [t["q.b"].reshape(-1), t["k.b"].reshape(-1)] + ([] if v is None else [t["v.b"].reshape(-1)])
            self.b_qkv = torch.cat(biases).to(torch.float32).contiguous()
        if self.sink:
            self.sink_logits = t["sink"].reshape(-1).to(torch.float32).contiguous()
        if self.qk_norm_weight:
            self.norm_weights = tuple(t[n].reshape(-1).to(torch.float32).contiguous() for n in ("q.norm", "k.norm"))
        if self.out_bias:
            extra = torch.zeros(self.hidden, _BIAS_PAD, dtype=o.dtype, device=o.device)
            extra[:, 0] = t["o.b"].reshape(-1).to(o.dtype)
            o = torch.cat([o, extra], dim=1)
        self.w_o = pack(o.contiguous())
        if self.talk:
            self.talk_matrix = t["talk"].reshape(-1).to(torch.float32).contiguous()
        if self.v_mix == "mix":
            self.v_lambda = t["vmix"].reshape(1).to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o))

    def cache_need(self) -> CacheNeed:
        # a chunk is stored like a window of its length: no later token sees a key that lies a whole chunk back
        return CacheNeed(self.kv_heads, self.head_dim, self.chunk if self.chunk else self.window, v_head_dim=self.v_dim,
                         keep_first=self.keep_first if self.window is not None else 0)

    can_overwrite = True        # forward(..., accumulate=False) writes its result instead of adding it

    def forward(self, h, residual, step, cache, state, append: bool, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        H, G, d, dv = self.heads, self.kv_heads, self.head_dim, self.v_dim
        proj = ws.buffer("sink_attention.proj", (cap, self.proj_ld), torch.float32)[:T]
        ops.linear(h, self.w_qkv, proj)
        table, rot = None, 0
        if self.position is not None:
            rotation = self.position.rotation_table(step)
            if rotation is None:
                raise ValueError("attention: this mixer needs a position encoding that is a table of rotations")
            table, rot = rotation
        v_first, v_mode = None, 0
        if self.v_mix is not None:
            v_first = ws.buffer(self.v_mix_key, (cap, self.v_width), torch.float32)[:T]
            if self.v_mix == "first":
                step.shared[self.v_mix_key] = v_first
                v_mode = 1
            else:
                if step.shared.get(self.v_mix_key) is None:
                    raise ValueError("attention: values are to be mixed with those of a layer that has not run in this step")
                v_mode = 2
        q = ws.buffer("sink_attention.q", (cap, self.q_width), self.ctx.dtype)[:T]
        ops.qkv_prepare(proj, self.b_qkv, table, rot, H, G, d, dv, self.qk_unit_norm, self.eps, q, cache, step, append,
                        self.v_lambda, v_first, v_mode, norm_weights=self.norm_weights, interleaved=self.interleaved, v_from_k=self.v_from_k)
        ones = _BIAS_PAD if self.out_bias else 0
        gate = proj[:, self.gate_at: self.gate_at + H] if self.head_gate else None
        attn = ws.buffer("sink_attention.out", (cap, self.out_width + ones), self.ctx.dtype)[:T]
        softmax_attention(self.ctx, q, H, G, d, dv, cache, step, self.scale, self.window, self.keep_first, attn, ones=ones, gate=gate,
                          talk_matrix=self.talk_matrix if self.talk else None, use_heads_kernel=self.use_heads_kernel,
                          chunk=self.chunk, sink=self.sink_logits)
        ops.linear(attn, self.w_o, residual, accumulate=accumulate)


def softmax_attention(ctx, q, H: int, G: int, d: int, dv: int, cache, step, scale: float, window: Optional[int], keep_first: int, out,
                      ones: int = 0, gate=None, talk_matrix=None, use_heads_kernel: bool = True, chunk: int = 0, sink=None) -> None:
    """Softmax attention of the step's queries ``q [tokens, H * d]`` over the cached keys and values of ``cache`` (``G``
    key/value heads of sizes ``d`` and ``dv``), by whichever kernel takes the step: ``out [tokens, H * dv + ones]`` (the
    dtype of the products, or 32-bit) receives the normalised results, mixed between the heads by ``talk_matrix``, each
    head's times ``sigmoid(gate[t, head])``, and ``ones`` more columns (a one, then zeros).  ``chunk`` (instead of a window) and
    ``sink`` (float32 ``[H]``) as the kernels take them.  Any part that has put its keys
    and values into a paged cache group can call it."""
    ops, ws, T, cap = ctx.ops, ctx.workspace, step.num_tokens, ctx.max_step_tokens
    talk = talk_matrix is not None
    longest = min(step.max_len, chunk) if chunk else step.max_len if window is None else min(step.max_len, window + keep_first)
    plan = ops.attention_heads_plan(T, H, G, d, dv, ctx.dtype, longest) if use_heads_kernel else None
    if use_heads_kernel and ops.attention_sink_prefill_wanted(step, H, G, d, dv, ctx.dtype):
        # many tokens: 64 query tokens of a sequence share a block's keys and values (flash-style, tensor cores)
        all_values = talk and G > 1
        n_val = G if all_values else 1
        partial = ws.buffer(f"sink_attention.partial_general.{H * n_val * dv}", (cap, H * n_val * dv), torch.float32)[:T]
        ops.attention_sink_prefill(q, H, G, d, dv, cache, step, partial, scale, window, keep_first, all_values, chunk=chunk, sink=sink)
        if n_val == G:
            ops.head_mix_splits(partial, None, talk_matrix, out, H, G, dv, 1, ones, gate=gate)
        else:
            ops.head_mix(partial, None, out, H, G, dv, n_val, ones, gate=gate)
    elif plan is not None:
        # one block per (token, key split) serves all heads; it mixes the heads itself when it can
        splits, writes_output = plan
        direct = gate is None and out.dtype == ctx.dtype          # the kernel can write this output itself
        if writes_output and direct:
            ops.attention_heads(q, H, G, d, dv, cache, step, scale, window, keep_first, 1, mix=talk_matrix, out=out, ones=ones,
                                chunk=chunk, sink=sink)
        else:
            # tokens x splits at most: the same buffer for every step, a captured graph holds its address.  Only steps of few
            # tokens are split when the kernel writes the output of the others itself; else every token of a step has a row.
            rows = (ops.ATTENTION_HEADS_MAX_ROWS if direct and ops.attention_heads_whole(H, G, d, dv, ctx.dtype)
                    else max(cap, ops.ATTENTION_HEADS_MAX_ROWS))
            partial = ws.buffer("sink_attention.partial", (rows, H * G * dv), torch.float32)
            ml = ws.buffer("sink_attention.ml", (rows, H * 2), torch.float32)
            ops.attention_heads(q, H, G, d, dv, cache, step, scale, window, keep_first, splits, partial=partial, ml=ml, chunk=chunk, sink=sink)
            ops.head_mix_splits(partial, ml, talk_matrix, out, H, G, dv, splits, ones, gate=gate)
    else:
        all_values = talk and G > 1
        n_val = G if all_values else 1
        partial = ws.buffer(f"sink_attention.partial_general.{H * n_val * dv}", (cap, H * n_val * dv), torch.float32)[:T]
        ops.attention_sink(q, H, G, d, dv, cache, step, partial, scale, window, keep_first, all_values, chunk=chunk, sink=sink)
        ops.head_mix(partial, talk_matrix, out, H, G, dv, n_val, ones, gate=gate)
