"""A plain, slow Moponex decoder: the oracle of the tests.

One function per mechanism, written from the design's equations in torch on the CPU (float64
unless another dtype is asked for); it shares no code with the library.  ``PlainMoponex`` feeds a
whole sequence at once and recomputes everything from the first token: the recurrences are
token-by-token loops, attention goes through an explicit mask, the experts are evaluated for every
token and picked afterwards.

Notation: ``x`` residual stream, ``h`` a sublayer's normed input, ``S`` a recurrent state, ``m`` the
factor on every sublayer's result (``x <- x + m * sublayer(norm(x))``).  ``rnd`` rounds a tensor where the
library rounds in bfloat16 (what a matrix product reads, queries, cached keys and values); the identity
by default.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------ small pieces
def rms_norm(x, w, eps: float):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension (w None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def same(t):
    return t


def to_bf16(t):
    return t.to(torch.bfloat16).to(t.dtype)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


# ------------------------------------------------------------------------------------------------ embedding
def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Row of the pair table per token: a hash of (previous token, token); the table's last row for a first token."""
    return [buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets for i, t in enumerate(tokens)]


def embed(tokens: List[int], table, pair_table, pair_cfg: Optional[dict]):
    x = table[torch.tensor(tokens)]
    if pair_cfg is not None:
        rows = bigram_rows(tokens, int(pair_cfg["buckets"]), int(pair_cfg["mul_prev"]), int(pair_cfg["mul_cur"]))
        x = x + pair_table[torch.tensor(rows)]
    return x


# ------------------------------------------------------------------------------------------------ state-space mixer
def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (last column: the current token), b [C]: y[t] = b + sum_j w[:, j] x[t - taps + 1 + j]."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    y = b.expand(T, C).clone()
    for j in range(taps):
        y = y + padded[j: j + T] * w[:, j]
    return y


def head_state_scan(xs, B, C, dt, A, D):
    """xs [T, H, P], B and C [T, G, N], dt [T, H] (positive), A [H] (negative), D [H] -> y [T, H, P].
    Per head: S <- exp(A dt) S + dt B x^T (S is N x P), y = S^T C + D x; head h reads group h // (H / G)."""
    T, H, P = xs.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros(T, H, P, dtype=xs.dtype)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros(N, P, dtype=xs.dtype)
        for t in range(T):
            S = torch.exp(A[h] * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], xs[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * xs[t, h]
    return y


def mamba2_mixer(h, w: Dict[str, torch.Tensor], c: dict, eps: float, rnd=same):
    H, P, N, G = int(c["heads"]), int(c["vdim"]), int(c["state"]), int(c["groups"])
    inner = H * P
    T = h.shape[0]
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    xs = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner: inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    y = head_state_scan(xs, B, C, dt, -torch.exp(w["A_log"]), w["D"]).reshape(T, inner)
    y = y * silu(z)                                                  # the gate first, the norm after it
    parts = int(c["norm_groups"])
    y = rms_norm(y.reshape(T, parts, inner // parts), None, eps).reshape(T, inner) * w["norm"]
    return rnd(y) @ w["o"].T


# ------------------------------------------------------------------------------------------------ chunked attention with a sink
def rotate_pairs(t, positions, dims: int, base: float, factor: float):
    """t [T, heads, d]: the pairs (2i, 2i + 1), i < dims / 2, turned by positions * base^(-2i/dims) / factor."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims) / factor
    a = positions.to(torch.float64)[:, None] * f[None, :]
    cos, sin = torch.cos(a).to(t.dtype)[:, None, :], torch.sin(a).to(t.dtype)[:, None, :]
    out = t.clone()
    u, v = t[..., 0:dims:2], t[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def chunk_mask(T: int, size: Optional[int]):
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    mask = j <= i
    if size is not None:
        mask = mask & (i // size == j // size)
    return mask


def sink_softmax_attention(q, k, v, scale: float, mask, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv], sink [H] or None -> [T, H, dv].  The softmax's denominator holds
    exp(sink_h) once more; that term has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        if sink is not None:
            s = torch.cat([s, sink[hd].expand(T, 1)], dim=1)
        p = torch.softmax(s, dim=-1)
        out[:, hd] = p[:, :T] @ v[:, g]
    return out


def chunk_attention_mixer(h, w: Dict[str, torch.Tensor], c: dict, eps: float, positions, rnd=same):
    H, G, d = int(c["heads"]), int(c["kv_heads"]), int(c["dim"])
    T = h.shape[0]
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, d)
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, d)
    v = k                                                            # the values are the keys as projected
    q, k = rms_norm(q, w["q.norm"], eps), rms_norm(k, w["k.norm"], eps)
    rot = c.get("rot")
    if rot is not None and int(rot["dims"]) > 0:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate_pairs(q, positions, int(rot["dims"]), float(rot["base"]), factor)
        k = rotate_pairs(k, positions, int(rot["dims"]), float(rot["base"]), factor)
    size = (c.get("mask") or {}).get("size")
    o = sink_softmax_attention(rnd(q), rnd(k), rnd(v), float(c["scale"]), chunk_mask(T, size), w.get("sink"))
    return rnd(o.reshape(T, H * d)) @ w["o"].T


# ------------------------------------------------------------------------------------------------ gated linear attention
def channel_decay_memory(q, k, v, alpha):
    """q, k, alpha [T, H, d], v [T, H, dv] -> [T, H, dv]: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t."""
    T, H, d = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for hd in range(H):
        S = torch.zeros(d, v.shape[2], dtype=q.dtype)
        for t in range(T):
            S = alpha[t, hd][:, None] * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    return out


def gated_linear_mixer(h, w: Dict[str, torch.Tensor], c: dict, eps: float, rnd=same):
    H, d, dv = int(c["heads"]), int(c["dim"]), int(c["vdim"])
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).reshape(T, H, d)
    v = (h @ w["v"].T).reshape(T, H, dv)
    zed = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.pow(torch.sigmoid(zed), 1.0 / float(c["tau"])).reshape(T, H, d)
    o = rms_norm(channel_decay_memory(q, k, v, alpha), w["norm"], eps).reshape(T, H * dv)
    return rnd(o * silu(h @ w["g"].T)) @ w["o"].T


def parallel_mixer(h, w: Dict[str, torch.Tensor], c: dict, eps: float, positions, rnd=same):
    sub = lambda side: {n[len(side) + 1:]: t for n, t in w.items() if n.startswith(side + ".")}
    a = chunk_attention_mixer(h, sub("left"), c["left"], eps, positions, rnd)
    b = gated_linear_mixer(h, sub("right"), c["right"], eps, rnd)
    return 0.5 * (rms_norm(a, w["left.out"], eps) + rms_norm(b, w["right.out"], eps))


# ------------------------------------------------------------------------------------------------ feed-forwards
def dense_ff(h, w, rnd=same):
    return rnd(gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def route(h, w_router, correction, c: dict):
    """-> (chosen [T, top] expert numbers, weights [T, top]).  Softmax over all outputs; choice by score + correction
    inside the best groups; weights from the scores without the correction, divided by their sum."""
    r = c["router"]
    E, top = int(r["experts"]) + int(r.get("identity", 0)), int(r["top"])
    s = torch.softmax(h @ w_router.T, dim=-1)
    choice = s + correction
    groups = r.get("groups")
    if groups is not None:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = E // count
        best = choice.reshape(-1, count, per).max(-1).values
        kept = torch.topk(best, keep, dim=-1).indices
        allowed = torch.zeros(h.shape[0], count, dtype=torch.bool)
        allowed.scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    chosen = torch.topk(choice, top, dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h, w, c: dict, rnd=same):
    r = c["router"]
    real = int(r["experts"])
    chosen, weights = route(h, w["router"], w["correction"], c)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            if e >= real:
                out[t] += g * h[t]                                   # an identity expert hands its input back
            else:
                out[t] += g * (rnd(gelu_erf(h[t] @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T)
    if c.get("shared") is not None:
        # (the library multiplies the rows the second product reads by the gate: the same sum)
        out = out + rnd(torch.sigmoid(h @ w["shared.sg"].T) * gelu_erf(h @ w["shared.up"].T)) @ w["shared.down"].T
    return out


# ------------------------------------------------------------------------------------------------ the model
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
        data = f.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    out = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        a, b = m["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[m["dtype"]]).reshape(m["shape"]).clone()
    return out


class PlainMoponex:
    def __init__(self, cfg, tensors=None, dtype=torch.float64, round_to=None):
        """``cfg``: the configuration (a dict) with ``tensors`` (name -> tensor), or a model folder."""
        if tensors is None:
            folder = cfg
            with open(os.path.join(folder, "config.json")) as f:
                cfg = json.load(f)
            tensors = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.cfg = cfg
        self.dtype = dtype
        self.rnd = to_bf16 if round_to == torch.bfloat16 else same
        self.w = {n: t.to(dtype) for n, t in tensors.items()}

    def _sub(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {n[len(prefix):]: t for n, t in self.w.items() if n.startswith(prefix)}

    def logits(self, tokens: List[int], layers_out: Optional[list] = None):
        """[T, vocab] for the whole sequence; ``layers_out`` collects the stream after every layer."""
        c, w, rnd = self.cfg, self.w, self.rnd
        eps, m = float(c["norm"]["eps"]), float(c.get("residual_mult", 1.0))
        pair = (c.get("embedding") or {}).get("bigram")
        x = embed(tokens, w["embed"], w.get("bigram"), pair)
        positions = torch.arange(len(tokens))
        for i, layer in enumerate(c["layers"]):
            p = f"l{i}."
            h = rnd(rms_norm(x, w[p + "norm1"], eps))
            mw = self._sub(p + "mix.")
            if layer["type"] == "mamba2":
                y = mamba2_mixer(h, mw, layer["mixer"], eps, rnd)
            else:
                y = parallel_mixer(h, mw, layer["mixer"], eps, positions, rnd)
            x = x + m * y
            if layer.get("mlp") is not None:
                h = rnd(rms_norm(x, w[p + "norm2"], eps))
                fw = self._sub(p + "mlp.")
                y = dense_ff(h, fw, rnd) if layer["mlp"]["kind"] == "dense" else moe_ff(h, fw, layer["mlp"], rnd)
                x = x + m * y
            if layers_out is not None:
                layers_out.append(x.clone())
        return (rnd(rms_norm(x, w["final.norm"], eps)) @ w["embed"].T) * float(c.get("logit_scale", 1.0))
