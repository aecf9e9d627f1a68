"""A plain, slow Tonovik decoder: the oracle of the tests.

One function per mechanism, written from the design's equations in torch on the CPU (float64
unless another dtype is asked for); it shares no code with the library.  ``PlainTonovik`` feeds a
whole sequence at once and recomputes everything from the first token: attention through an
explicit mask, the matrix memory as a token-by-token loop, the latent attention with the keys and
values of every head written out (nothing is folded into the queries).

Notation: ``x`` residual stream (a sublayer reads it as it is; the layer norm sits on the
sublayer's OUTPUT), ``c`` the latent of the latent attention, ``S`` the matrix memory.  With
``round_to`` the values are rounded where the library rounds them in bfloat16 (what a matrix
product reads, cached keys, values and latents).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import torch


def layer_norm(x, w, b, eps: float):
    """(x - mean) / sqrt(var + eps) * w + b over the last dimension, var the mean squared deviation."""
    m = x.mean(-1, keepdim=True)
    d = x - m
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w + b


def rms_unit(x, eps: float):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(dims: int, base: float, scaling: Optional[dict] = None):
    """(f [dims / 2] in 64-bit, amplitude).  ``scaling`` = {factor, original, fast, slow}: the YaRN blend."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if scaling is None:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])
    at = lambda turns: dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(at(float(scaling["fast"]))), 0)
    hi = min(math.ceil(at(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(t, positions, dims: int, freq, amplitude: float, interleaved: bool):
    """t [T, heads, d]: the first ``dims`` dimensions of each head turned by positions * freq.  Pairs are
    (i, i + dims/2), or (2i, 2i + 1) when ``interleaved``; the rest of the head passes unchanged."""
    a = positions.to(torch.float64)[:, None] * freq[None, :]               # [T, dims/2]
    cos, sin = (torch.cos(a) * amplitude).to(t.dtype)[:, None, :], (torch.sin(a) * amplitude).to(t.dtype)[:, None, :]
    out = t.clone()
    if interleaved:
        u, v = t[..., 0:dims:2], t[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        half = dims // 2
        u, v = t[..., :half], t[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


def masked_softmax_attention(q, k, v, scale: float, window: Optional[int]):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; query i sees j <= i (and i - j < window)."""
    T, H, _ = q.shape
    G = k.shape[1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    mask = j <= i
    if window is not None:
        mask = mask & (i - j < window)
    out = torch.empty(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def retention(q, k, v, decay):
    """q, k [T, H, d], v [T, H, dv], decay [H]: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, S_(-1) = 0."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=q.dtype)
    out = torch.empty(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def swiglu(h, wg, wu, wd, r=lambda t: t):
    return r(silu(h @ wg.T) * (h @ wu.T)) @ wd.T


class PlainTonovik:
    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float64, round_to=None):
        self.cfg, self.dtype = cfg, dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.round_to = round_to

    def r(self, t):
        return t if self.round_to is None else t.to(self.round_to).to(self.dtype)

    # ------------------------------------------------------------------ mixers
    def window_branch(self, h, positions, m, name, eps):
        w, r = self.w, self.r
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        T = h.shape[0]
        hr = r(h)
        q = (hr @ w[name + "q"].T + w[name + "q.b"]).reshape(T, H, d)
        k = (hr @ w[name + "k"].T + w[name + "k.b"]).reshape(T, G, d)
        v = (hr @ w[name + "v"].T + w[name + "v.b"]).reshape(T, G, dv)
        q = rms_unit(q, eps) * w[name + "q.norm"]
        k = rms_unit(k, eps) * w[name + "k.norm"]
        f, amp = rotary_frequencies(m["rot"]["dims"], m["rot"]["base"])
        q, k = rotate(q, positions, m["rot"]["dims"], f, amp, False), rotate(k, positions, m["rot"]["dims"], f, amp, False)
        o = masked_softmax_attention(r(q), r(k), r(v), m["scale"], m["mask"]["size"])
        gate = torch.sigmoid(hr @ w[name + "g"].T)                      # [T, H]
        return r((o * gate[:, :, None]).reshape(T, H * dv)) @ w[name + "o"].T

    def retention_branch(self, h, positions, m, name, eps):
        w, r = self.w, self.r
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        T = h.shape[0]
        hr = r(h)
        q, k = (hr @ w[name + "q"].T).reshape(T, H, d), (hr @ w[name + "k"].T).reshape(T, H, d)
        v = (hr @ w[name + "v"].T).reshape(T, H, dv)
        f, amp = rotary_frequencies(m["rot"]["dims"], m["rot"]["base"])
        q, k = rotate(q, positions, m["rot"]["dims"], f, amp, False), rotate(k, positions, m["rot"]["dims"], f, amp, False)
        k = k * d ** -0.5
        o = retention(q, k, v, torch.tensor(m["decay"], dtype=self.dtype))
        o = rms_unit(o, eps).reshape(T, H * dv) * silu(hr @ w[name + "g"].T)
        return r(o) @ w[name + "o"].T

    def parallel(self, h, positions, m, name, eps):
        return (m["left_scale"] * self.window_branch(h, positions, m["left"], name + "left.", eps)
                + m["right_scale"] * self.retention_branch(h, positions, m["right"], name + "right.", eps))

    def latent_attention(self, h, positions, m, name, eps):
        w, r = self.w, self.r
        H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        T = h.shape[0]
        hr = r(h)
        q = (hr @ w[name + "q"].T).reshape(T, H, d + dr)
        down = hr @ w[name + "dkv"].T
        c = r(rms_unit(down[:, :rank], eps) * w[name + "dkv.norm"])
        f, amp = rotary_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
        k_rot = rotate(down[:, None, rank:], positions, m["rot"]["dims"], f, amp, True)        # [T, 1, dr]
        q_rot = rotate(q[:, :, d:], positions, m["rot"]["dims"], f, amp, True)
        k_flat = (c @ w[name + "uk"].T).reshape(T, H, d)
        v = (c @ w[name + "uv"].T).reshape(T, H, dv)
        qq = torch.cat([q[:, :, :d], q_rot], dim=-1)
        kk = torch.cat([k_flat, r(k_rot).expand(T, H, dr)], dim=-1)
        o = masked_softmax_attention(r(qq), kk, v, m["scale"], None)
        gate = torch.sigmoid(hr @ w[name + "g"].T)
        return r((o * gate[:, :, None]).reshape(T, H * dv)) @ w[name + "o"].T

    # ------------------------------------------------------------------ the stack
    def forward(self, tokens: List[int], return_layers: bool = False):
        cfg, w, r = self.cfg, self.w, self.r
        eps = float(cfg["norm"]["eps"])
        ids = torch.tensor(tokens, dtype=torch.long)
        positions = torch.arange(len(tokens))
        x = w["embed"][ids] * float(cfg["embedding"]["scale"])
        layers = []
        for i, l in enumerate(cfg["layers"]):
            p = f"l{i}."
            if l["type"] == "parallel":
                y = self.parallel(x, positions, l["mixer"], p + "mix.", eps)
            elif l["type"] == "latent_attention":
                y = self.latent_attention(x, positions, l["mixer"], p + "mix.", eps)
            else:
                raise ValueError(l["type"])
            x = x + layer_norm(y, w[p + "norm1"], w[p + "norm1.b"], eps)
            if l.get("mlp") is not None:
                y = swiglu(r(x), w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"], r)
                x = x + layer_norm(y, w[p + "norm2"], w[p + "norm2.b"], eps)
            layers.append(x.clone())
        logits = r(layer_norm(x, w["final.norm"], w["final.norm.b"], eps)) @ w["head"].T
        return (logits, torch.stack(layers)) if return_layers else logits

    def logits(self, tokens: List[int]):
        return self.forward(tokens).to(torch.float64)


def latent_heads(q, c, k_rot, uk, uv, scale: float):
    """The latent attention with every head's keys and values written out: q [T, H, d + dr] (rotated part last, already
    turned), c [T, rank], k_rot [T, dr] (turned), uk [H * d, rank], uv [H * dv, rank] -> [T, H, dv]."""
    T, H, _ = q.shape
    d, dv = uk.shape[0] // H, uv.shape[0] // H
    k = torch.cat([(c @ uk.T).reshape(T, H, d), k_rot[:, None, :].expand(T, H, k_rot.shape[1])], dim=-1)
    return masked_softmax_attention(q, k, (c @ uv.T).reshape(T, H, dv), scale, None)


def generate_greedy(model: PlainTonovik, prompt, n: int) -> List[int]:
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(torch.argmax(model.forward(seq)[-1])))
    return seq[len(prompt):]


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """A reader of its own (8-byte length, JSON header, data), so that the oracle shares none with the library."""
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[lo:hi]), dtype=kinds[e["dtype"]]).reshape(e["shape"]).clone()
    return out


def load_folder(folder: str, dtype=torch.float64, round_to=None) -> PlainTonovik:
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return PlainTonovik(cfg, read_safetensors(os.path.join(folder, "model.safetensors")), dtype, round_to)
