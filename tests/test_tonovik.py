"""The Tonovik decoder against the plain implementation (tests/plain_tonovik.py): every mechanism alone (the layer
norm on a sublayer's output, the window attention with its norms, rotation and gates, the matrix memory with a
fixed decay, the attention over cached latents), then the engine: whole prompts, token-by-token decoding, prompts
in portions down to two tokens, unequal batches with slots and pages used again, long decoding, greedy
generation through the library's entry point and the replay program."""
import math

import pytest
import torch

import tonovik_tools as tv
import trace_tools as tt
from conftest import require_gpu
from plain_tonovik import (PlainTonovik, latent_heads, layer_norm, masked_softmax_attention, retention, rms_unit, rotary_frequencies,
                           rotate, silu)

DTYPES = ["float32", "bfloat16"]
NAMES = ["mixed", "edges", "wide"]
DEV = "cuda:0"


# --------------------------------------------------------------------------- helpers
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config, {"exact" | dtype: plain model}): in 64-bit; in 32-bit; in 64-bit but rounding to bfloat16
    where the library does"""
    out = {}
    for i, (name, cfg) in enumerate(tv.CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("tonovik_" + name))
        tensors = tv.write_model(d, cfg, 40 + i)
        out[name] = (d, cfg, {"exact": PlainTonovik(cfg, tensors), "float32": PlainTonovik(cfg, tensors, dtype=torch.float32),
                              "bfloat16": PlainTonovik(cfg, tensors, round_to=torch.bfloat16)})
    return out


def _engine(folder, dtype, max_tokens, **kw):
    from hilbert_pruned_8b_b200.engine.step import Engine
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, **kw)


def _err(x, exact):
    return (x - exact).abs().max().item() / max(1.0, exact.abs().max().item())


def _spread(x, exact, scale):
    """Root mean square over the vocabulary of the difference, its mean taken off, over ``scale``."""
    d = (x - exact).double()
    return (d - d.mean()).pow(2).mean().sqrt().item() / scale


def _reference(plain, requests, dtype=None):
    """(request, position) -> (the exact logits; the two errors, ``_err`` and ``_spread``, of a plain model that rounds as
    ``dtype`` does).  ``_spread`` is in units of the root mean square of all the exact logits (each row's mean taken off)."""
    exact = {rid: plain["exact"].logits(toks) for rid, toks in requests.items()}
    rows = torch.cat([e.double() - e.double().mean(dim=-1, keepdim=True) for e in exact.values()])
    scale = max(rows.pow(2).mean().sqrt().item(), 1e-30)
    ref = {}
    for rid, toks in requests.items():
        rounded = plain[dtype].logits(toks) if dtype is not None else exact[rid]
        for p in range(len(toks)):
            ref[(rid, p)] = (exact[rid][p], _err(rounded[p], exact[rid][p]), _spread(rounded[p], exact[rid][p], scale), scale)
    return ref


# The bound.  Every position's logits are compared with the 64-bit plain model's.  In this design a layer norm sits on each
# sublayer's OUTPUT, so where that output happens to have little spread the norm multiplies whatever rounding error it
# carries: a few positions of a random model are ill-conditioned, and there a plain model that only rounds (to 32-bit; or
# what the matrix products read and the cache holds to bfloat16) is itself far from the exact one.
# 32-bit: the largest difference over the largest logit (or 1) is at most three times what the plain 32-bit model shows at
# that position, or three times that model's median, or 1e-4, at EVERY position.
# bfloat16: which positions a rounding hits hard differs between two programs that round in different places, so the
# library's errors are compared with the plain rounding model's as a population (root mean square over the vocabulary):
# at most 3 % of the positions (or one) above three times the plain model's error there (or its median), the median and
# the ninth decile within 1.5 times the plain model's, the largest within three times its largest.  A wrong key, window
# or state moves the logits by tens of per cent at most positions of these models, and the 32-bit runs of the same
# schedules hold every single position.
def _compare(got, ref, dtype, what):
    assert got, "nothing was compared"
    for key, g in got.items():
        assert torch.isfinite(g).all(), f"{what}: non-finite logits at {key}"
    if dtype == "float32":
        noise = sorted(ref[key][1] for key in got)
        typical = noise[len(noise) // 2]
        for key, g in got.items():
            exact, rounding = ref[key][:2]
            bound = max(3.0 * max(rounding, typical), 1e-4)
            err = _err(g, exact)
            assert err <= bound, f"{what}: float32 logits differ at request {key[0]} position {key[1]}: {err:.3e} (bound {bound:.3e})"
        return
    keys = list(got)
    noise = [ref[k][2] for k in keys]
    errs = [_spread(got[k], ref[k][0], ref[k][3]) for k in keys]
    n, ns, es = len(keys), sorted(noise), sorted(errs)
    typical = ns[n // 2]
    over = [(e / (3.0 * max(x, typical)), k) for k, e, x in zip(keys, errs, noise) if e > 3.0 * max(x, typical)]
    assert len(over) <= max(1, (3 * n) // 100), f"{what}: bfloat16 logits differ at {len(over)} of {n} positions, most at {max(over)}"
    assert es[-1] <= 3.0 * max(ns[-1], 3.0 * typical), f"{what}: largest bfloat16 error {es[-1]:.3e}, the plain rounding model's {ns[-1]:.3e}"
    if n >= 40:
        assert es[n // 2] <= 1.5 * typical, f"{what}: median bfloat16 error {es[n // 2]:.3e}, the plain rounding model's {typical:.3e}"
        assert es[(9 * n) // 10] <= 1.5 * ns[(9 * n) // 10], f"{what}: ninth decile {es[(9 * n) // 10]:.3e} against {ns[(9 * n) // 10]:.3e}"


def _requests(cfg, lengths, seed):
    return {f"r{i}": tt.random_tokens(n, cfg["vocab"], seed + i) for i, n in enumerate(lengths)}


# --------------------------------------------------------------------------- without a GPU
def test_config_round_trip_and_weight_table():
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.config import ConfigError, config_class_for
    from hilbert_pruned_8b_b200.engine.model import weight_table
    for cfg in tv.CONFIGS.values():
        assert config_class_for(cfg) is hb.TonovikConfig
        c = hb.TonovikConfig.from_dict(cfg)
        assert hb.TonovikConfig.from_dict(c.to_dict()) == c
        table = weight_table(c.model_spec(), "")
        for i, layer in enumerate(cfg["layers"]):
            assert f"l{i}.norm1" in table and f"l{i}.norm1.b" in table
            assert (f"l{i}.norm2.b" in table) == (layer["mlp"] is not None) == (f"l{i}.mlp.gate" in table)
            assert (f"l{i}.mix.left.q.b" in table) == (layer["type"] == "parallel") == (f"l{i}.mix.right.g" in table)
            assert (f"l{i}.mix.dkv.norm" in table) == (layer["type"] == "latent_attention")
            assert f"l{i}.mix.right.norm" not in table and f"l{i}.mix.left.o.b" not in table
        assert table["final.norm.b"].shape == (cfg["width"],) and table["head"].shape == (cfg["vocab"], cfg["width"])
    table = weight_table(hb.TonovikConfig.from_dict(tv.MIXED).model_spec(), "")
    m0, m1 = tv.MIXED["layers"][0]["mixer"], tv.MIXED["layers"][1]["mixer"]
    assert table["l0.mix.q"].shape == (m0["heads"] * (m0["dim"] + m0["rot_dim"]), 64)
    assert table["l0.mix.dkv"].shape == (m0["kv_rank"] + m0["rot_dim"], 64) and table["l0.mix.uv"].shape == (m0["heads"] * m0["vdim"], m0["kv_rank"])
    assert table["l0.mix.g"].shape == (m0["heads"], 64) and table["l1.mix.left.g"].shape == (m1["left"]["heads"], 64)
    assert table["l1.mix.left.k"].shape == (m1["left"]["kv_heads"] * m1["left"]["dim"], 64) and table["l1.mix.left.q.norm"].shape == (m1["left"]["dim"],)
    assert table["l1.mix.right.g"].shape == (m1["right"]["heads"] * m1["right"]["vdim"], 64)
    good = tv.with_mlp(tv.parallel((2, 1, 4, 4, 5, 4), (2, 4, 4, (0.5, 0.5), 4)), None)

    def changed(path, value):
        import copy
        layer = copy.deepcopy(good)
        d = layer["mixer"]
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = value
        return {**tv.MIXED, "layers": [layer]}
    for bad in ({**tv.MIXED, "layers": []}, {**tv.MIXED, "width": 0}, {k: v for k, v in tv.MIXED.items() if k != "norm"},
                {**tv.MIXED, "layers": [{"type": "conv", "mixer": {}, "mlp": None}]},
                changed(("left", "kv_heads"), 3), changed(("right", "decay"), [0.5]), changed(("left", "rot", "dims"), 6),
                changed(("left", "rot", "dims"), 3), changed(("left", "mask", "size"), 0), changed(("right", "decay"), [0.5, 1.5]),
                {**tv.MIXED, "layers": [tv.with_mlp(tv.latent(2, 4, 4, 4, 8, dims=6), None)]},
                {**tv.MIXED, "layers": [dict(tv.with_mlp(tv.latent(2, 4, 4, 4, 8), None), mlp={"kind": "moe", "ff": 8})]}):
        with pytest.raises(ConfigError):
            hb.TonovikConfig.from_dict(bad)
    hb.TonovikConfig.from_dict({**tv.MIXED, "layers": [good]})


def test_plain_mechanisms_agree_with_their_definitions():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    # layer norm: zero mean, unit mean square before weight and bias
    x, w, b = r(3, 10) * 4 + 2, r(10), r(10)
    y = (layer_norm(x, w, b, 0.0) - b) / w
    assert y.mean(-1).abs().max() < 1e-12 and ((y * y).mean(-1) - 1).abs().max() < 1e-12
    # the memory equals the explicit sums
    q, k, v, lam = r(7, 2, 3), r(7, 2, 3), r(7, 2, 5), torch.tensor([0.8, 1.0], dtype=torch.float64)
    out = retention(q, k, v, lam)
    for h in range(2):
        want = sum(lam[h] ** (6 - s) * (q[6, h] @ k[s, h]) * v[s, h] for s in range(7))
        assert torch.allclose(out[6, h], want)
    # rotation: pairs (i, i + dims/2) or (2i, 2i + 1), the rest untouched; a score depends on the distance only
    f, amp = rotary_frequencies(4, 100.0)
    assert amp == 1.0 and torch.allclose(f, torch.tensor([1.0, 0.1], dtype=torch.float64))
    t = r(1, 1, 6)
    a = 5 * f
    for inter, pairs in ((False, ((0, 2), (1, 3))), (True, ((0, 1), (2, 3)))):
        got = rotate(t, torch.tensor([5]), 4, f, 1.0, inter)[0, 0]
        for i, (u, vv) in enumerate(pairs):
            assert torch.allclose(got[u], t[0, 0, u] * torch.cos(a[i]) - t[0, 0, vv] * torch.sin(a[i]))
            assert torch.allclose(got[vv], t[0, 0, vv] * torch.cos(a[i]) + t[0, 0, u] * torch.sin(a[i]))
        assert torch.equal(got[4:], t[0, 0, 4:])
    qq, kk = r(1, 1, 4), r(1, 1, 4)
    s1 = (rotate(qq, torch.tensor([9]), 4, f, 1.0, True) * rotate(kk, torch.tensor([4]), 4, f, 1.0, True)).sum()
    s2 = (rotate(qq, torch.tensor([105]), 4, f, 1.0, True) * rotate(kk, torch.tensor([100]), 4, f, 1.0, True)).sum()
    assert torch.allclose(s1, s2)
    # YaRN: dims 8, base 100, original 64: dim(t) = 8 ln(64 / (2 pi t)) / (2 ln 100); fast 4 -> lo 0, slow 1 -> hi 3
    f, amp = rotary_frequencies(8, 100.0, {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0})
    base = torch.pow(torch.tensor(100.0, dtype=torch.float64), -torch.arange(4, dtype=torch.float64) / 4)
    lo, hi = max(math.floor(8 * math.log(64 / (8 * math.pi)) / (2 * math.log(100))), 0), min(math.ceil(8 * math.log(64 / (2 * math.pi)) / (2 * math.log(100))), 7)
    assert (lo, hi) == (0, 3)
    ramp = torch.clamp(torch.arange(4, dtype=torch.float64) / 3, 0, 1)
    assert torch.allclose(f, base / 4 * ramp + base * (1 - ramp)) and abs(amp - (0.1 * math.log(4.0) + 1)) < 1e-15
    # window: query 10 with a window of 4 sees 7..10
    q, k, v = r(12, 2, 3), r(12, 1, 3), r(12, 1, 2)
    out = masked_softmax_attention(q, k, v, 0.7, 4)
    p = torch.softmax(torch.stack([q[10, 1] @ k[j, 0] for j in range(7, 11)]) * 0.7, 0)
    assert torch.allclose(out[10, 1], (p[:, None] * v[7:11, 0]).sum(0))
    # the latent attention's folded form: scores against [c | k_r] with the key up-projection applied to the query
    T, H, d, dr, dv, rank = 6, 2, 3, 2, 4, 5
    q, c, kr, uk, uv = r(T, H, d + dr), r(T, rank), r(T, dr), r(H * d, rank), r(H * dv, rank)
    want = latent_heads(q, c, kr, uk, uv, 0.4)
    qf = torch.cat([torch.einsum("thd,hdr->thr", q[:, :, :d], uk.view(H, d, rank)), q[:, :, d:]], -1)
    mixed = masked_softmax_attention(qf, torch.cat([c, kr], -1)[:, None, :], c[:, None, :], 0.4, None)
    assert torch.allclose(torch.einsum("thr,hvr->thv", mixed, uv.view(H, dv, rank)), want)


# --------------------------------------------------------------------------- mechanisms on the GPU
def _context(dtype, cap=512):
    from hilbert_pruned_8b_b200.engine.workspace import Workspace
    from hilbert_pruned_8b_b200.kernels.ops import Ops
    from hilbert_pruned_8b_b200.parts import BuildContext
    dev = torch.device(DEV)
    return BuildContext(device=dev, dtype=dtype, ops=Ops(dev), workspace=Workspace(dev), max_step_tokens=cap)


def _mixer_spec(layer, width):
    """The part description the configuration makes for one layer's mixer (for a parallel layer: its two branches)."""
    import hilbert_pruned_8b_b200 as hb
    spec = hb.TonovikConfig.from_dict(tv.config(width, 16, [tv.with_mlp(layer, None)])).model_spec().layers[0].parts["mixer"]
    if layer["type"] == "parallel":
        return [b["mixer"] for b in spec.params["branches"]]
    return spec


def _portions(total, sizes):
    """Per round the new tokens of every sequence that still has some: [(live indices, new tokens, tokens done)]."""
    done, out = [0] * len(total), []
    for portion in sizes:
        live = [i for i in range(len(total)) if done[i] < total[i]]
        if not live:
            break
        new = [min(portion, total[i] - done[i]) for i in live]
        out.append((live, new, list(done)))
        for i, n in zip(live, new):
            done[i] += n
    assert done == list(total), "the portions do not cover the sequences"
    return out


class _MixerRun:
    """One mixer with a cache of its own: feeds rows of inputs, sequence by sequence and portion by portion."""

    def __init__(self, c, spec, weights, tokens=64 * 24):
        from hilbert_pruned_8b_b200.cache.manager import CacheManager
        from hilbert_pruned_8b_b200.parts import MIXERS
        self.c, self.mixer = c, MIXERS.build(spec, c)
        assert sorted(p.name for p in self.mixer.params()) == sorted(weights), sorted(p.name for p in self.mixer.params())
        self.mixer.bind({k: (v.to(c.dtype) if v.dim() == 2 else v).to(DEV) for k, v in weights.items()})
        need, state = self.mixer.cache_need(), self.mixer.state_need()
        self.cache = CacheManager({0: need} if need is not None else {}, {0: state} if state is not None else {}, tokens, c.device, c.dtype)
        self.has_cache, self.has_state = need is not None, state is not None

    def feed(self, hs, sizes):
        """hs: one [tokens, width] tensor per sequence; returns the mixer's outputs in the same shapes (float64, CPU)."""
        from hilbert_pruned_8b_b200.engine.batch import StepEntry, build_step
        c, cache = self.c, self.cache
        seqs = [cache.open() for _ in hs]
        got = [[] for _ in hs]
        for live, new, done in _portions([h.shape[0] for h in hs], sizes):
            entries = [StepEntry(seqs[i], [0] * n, []) for i, n in zip(live, new)]
            cache.reserve([(seqs[i], seqs[i].length + n) for i, n in zip(live, new)])
            step = build_step(entries, cache, c.workspace, c.device)
            hin = torch.cat([hs[i][done[i]: done[i] + n] for i, n in zip(live, new)]).to(c.dtype).to(DEV).contiguous()
            out = torch.full((hin.shape[0], hs[0].shape[1]), 7.0, device=DEV)
            self.mixer.forward(hin, out, step, cache.view(0) if self.has_cache else None, cache.state_view(0) if self.has_state else None,
                               True, accumulate=False)
            oc, at = out.cpu().double(), 0
            for i, n in zip(live, new):
                got[i].append(oc[at: at + n])
                cache.commit(seqs[i], seqs[i].length + n)
                at += n
        c.ops.check_errors()
        for s in seqs:
            cache.close(s)
        assert all(g.pool.num_free == g.pool.size for g in cache.groups)
        return [torch.cat(g) for g in got]


def _plain_for(weights, dtype):
    return PlainTonovik(None, {"m." + k: v for k, v in weights.items()}, round_to=torch.bfloat16 if dtype == torch.bfloat16 else None)


def _assert_close(got, want, dtype, what):
    for i, (g, w) in enumerate(zip(got, want)):
        err = (g - w).abs().max(1).values / w.abs().max().clamp(min=1.0)
        assert err.max() < (1e-4 if dtype == torch.float32 else 3e-2), f"{what}: sequence {i} position {int(err.argmax())}: {float(err.max()):.3e}"


def _bf16(t):
    return t.to(torch.bfloat16).double()


@pytest.mark.gpu
def test_layer_norm_alone_on_an_output_and_on_a_weighted_sum():
    require_gpu()
    c = _context(torch.float32)
    ops = c.ops
    g = torch.Generator().manual_seed(1)
    for width in (1, 2, 72, 257, 2500, 9000):
        y, y2 = (torch.randn(19, width, generator=g) * 3 + 1.5).cuda(), torch.randn(19, width, generator=g).cuda()
        x = torch.randn(19, width, generator=g).cuda()
        w, b = torch.randn(width, generator=g).cuda(), torch.randn(width, generator=g).cuda()
        eps = 1e-5
        out = torch.empty_like(y)
        ops.layernorm(y, w, b, eps, out)
        assert (out.double() - layer_norm(y.double(), w.double(), b.double(), eps)).abs().max() < 2e-5
        rows = torch.tensor([18, 0, 5], dtype=torch.int32, device=DEV)
        some = torch.empty(3, width, dtype=torch.bfloat16, device=DEV)
        ops.layernorm(y, w, b, eps, some, rows)
        assert (some.double() - layer_norm(y[rows.long()].double(), w.double(), b.double(), eps)).abs().max() < 6e-2
        x1, copy = x.clone(), torch.empty(19, width, dtype=torch.bfloat16, device=DEV)
        ops.layernorm_add(y, w, b, eps, x1, copy=copy)
        want = x.double() + layer_norm(y.double(), w.double(), b.double(), eps)
        assert (x1.double() - want).abs().max() < 2e-5 and torch.equal(copy, x1.to(torch.bfloat16))
        x2 = x.clone()
        ops.layernorm_add(y, w, b, eps, x2, y2=y2, sa=1.2, sb=-0.7)
        want = x.double() + layer_norm(1.2 * y.double() - 0.7 * y2.double(), w.double(), b.double(), eps)
        assert (x2.double() - want).abs().max() < 2e-5
    # a row of equal values has no deviation: the bias alone remains
    flat = torch.full((2, 40), 3.25, device=DEV)
    w, b = torch.randn(40, generator=g).cuda(), torch.randn(40, generator=g).cuda()
    out = torch.empty_like(flat)
    ops.layernorm(flat, w, b, 1e-5, out)
    assert (out - b).abs().max() < 1e-6
    ops.check_errors()


def _selection(rows, width, at):
    """[rows, width] with ones at (i, at + i): the projection that cuts columns at .. at + rows out of the input."""
    m = torch.zeros(rows, width)
    m[torch.arange(rows), at + torch.arange(rows)] = 1.0
    return m


WINDOWS = [(4, 2, 16, 8, 20, 8), (1, 1, 8, 12, 1, 0), (3, 3, 4, 4, 1000, 4), (4, 2, 64, 40, 33, 32), (2, 1, 32, 64, 100, 16), (5, 1, 64, 128, 140, 64),
           (2, 2, 128, 64, 64, 128), (2, 1, 128, 128, 65, 2), (6, 2, 24, 40, 63, 24)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,size,rot", WINDOWS)
def test_window_attention_sees_exactly_its_window(H, G, d, dv, size, rot, dtype):
    """A prompt of 300 tokens, then tokens one by one, a second, shorter sequence beside it.  The projections cut q, k, v and
    the gates out of the input (their matrices hold ones and zeros), so the test writes them directly: for some queries one key
    is made to stand out, the oldest token inside the window, the newest one outside it, a token on a page border.  The output
    then shows at once whether that key was seen."""
    require_gpu()
    layer = tv.parallel((H, G, d, dv, size, rot), (1, 2, 2, (0.5,), 0))
    spec = _mixer_spec(layer, 8)[0]
    m = layer["mixer"]["left"]
    width = H * d + G * d + G * dv + H
    spec.params["hidden_size"] = width
    g = torch.Generator().manual_seed(H * 100 + size)
    wts = {"q": _selection(H * d, width, 0), "k": _selection(G * d, width, H * d), "v": _selection(G * dv, width, H * d + G * d),
           "g": _selection(H, width, H * d + G * d + G * dv), "o": torch.randn(width, H * dv, generator=g) / (H * dv) ** 0.5,
           "q.b": torch.randn(H * d, generator=g) * 0.2, "k.b": torch.randn(G * d, generator=g) * 0.2, "v.b": torch.randn(G * dv, generator=g) * 0.5,
           "q.norm": torch.rand(d, generator=g) + 0.5, "k.norm": torch.rand(d, generator=g) + 0.5}
    wts = {k: v.to(torch.bfloat16).float() for k, v in wts.items()}
    n, n2 = 420, 97
    h = torch.randn(n, width, generator=g)
    probes = {299: 299 - size + 1, 300: 300 - size, 301: 301 - size + 1, 383: 320, 384: 383, 385: 385 - size, 411: 411 - size + 1}
    if rot < d:         # the unrotated dimensions carry the probe: their product does not depend on the distance
        for p, key in probes.items():
            if 0 <= key < n:
                kk = h[key, H * d: H * d + G * d].view(G, d) + wts["k.b"].view(G, d)
                kk[:, rot:] *= 6.0
                h[key, H * d: H * d + G * d] = (kk - wts["k.b"].view(G, d)).reshape(-1)
                kn = rms_unit(kk.double(), 1e-5) * wts["k.norm"].double()
                for hh in range(H):
                    qq = torch.zeros(d, dtype=torch.float64)
                    qq[rot:] = kn[hh // (H // G), rot:] / wts["q.norm"].double()[rot:]
                    h[p, hh * d: (hh + 1) * d] = (qq * 8.0).float() - wts["q.b"][hh * d: (hh + 1) * d]
    hs = [h, h[:n2].clone()]
    c = _context(dtype)
    got = _MixerRun(c, spec, wts).feed(hs, [300] + [1] * 200)
    plain = _plain_for(wts, dtype)
    want = [plain.window_branch(x.double(), torch.arange(x.shape[0]), m, "m.", 1e-5) for x in hs]
    _assert_close(got, want, dtype, "window attention")
    assert (got[1] - got[0][:n2]).abs().max() < (1e-4 if dtype == torch.float32 else 3e-2) * want[0].abs().max()
    # the same in portions of two and three tokens and one that fills the step
    got = _MixerRun(c, spec, wts).feed(hs, [2, 3, 2, 130, 2, 161] + [5] * 30)
    _assert_close(got, want, dtype, "window attention in portions")


def _random_weights(mixer_params, g, gain=1.0):
    out = {}
    for p in mixer_params:
        shape = tuple(p.shape)
        if p.name.endswith("norm"):
            t = torch.rand(shape, generator=g) + 0.5
        elif len(shape) == 1:
            t = torch.randn(shape, generator=g) * 0.3
        else:
            t = torch.randn(shape, generator=g) * gain / shape[1] ** 0.5
        out[p.name] = t.to(torch.bfloat16).float()
    return out


def _params_of(spec):
    from hilbert_pruned_8b_b200.parts import MIXERS
    return MIXERS.build(spec, _context(torch.float32, 8)).params()


MEMORIES = [(2, 8, 16, (0.7, 0.98), 4), (1, 40, 33, (1.0,), 40), (3, 64, 70, (0.0, 0.5, 1.0), 0), (2, 128, 32, (0.9995, 0.95), 64),
            (4, 32, 96, (0.9375, 0.99, 0.997, 0.9995), 16), (2, 2, 2, (0.25, 0.75), 2)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,d,dv,decay,rot", MEMORIES)
def test_decayed_memory_with_rotation_in_portions_equals_the_recurrence(heads, d, dv, decay, rot, dtype):
    """Two sequences of unequal lengths in portions of 1, 2, ... and of hundreds of tokens against the token-by-token loop:
    decays of one (nothing is forgotten: the first token still counts after hundreds) and of zero (only the token itself)."""
    require_gpu()
    W = 72
    layer = tv.parallel((1, 1, 2, 2, 4, 0), (heads, d, dv, decay, rot))
    spec = _mixer_spec(layer, W)[1]
    g = torch.Generator().manual_seed(d + rot)
    wts = _random_weights(_params_of(spec), g, gain=2.0)
    hs = [torch.randn(n, W, generator=g) for n in (460, 23)]
    hs[0][0] *= 5.0                                    # a first token that a lost state would miss
    c = _context(dtype)
    plain = _plain_for(wts, dtype)
    want = [plain.retention_branch(x.double(), torch.arange(x.shape[0]), layer["mixer"]["right"], "m.", 1e-5) for x in hs]
    got = _MixerRun(c, spec, wts).feed(hs, [1, 2, 1, 5, 70, 33, 1, 1, 64, 200, 2, 3, 77])
    _assert_close(got, want, dtype, "decayed memory")
    # the same state slots again, by other sequences: they start from zeros
    run = _MixerRun(c, spec, wts)
    run.feed(hs, [500])
    got = run.feed(hs[::-1], [300, 1, 1, 158])
    _assert_close(got, want[::-1], dtype, "decayed memory, slots used again")


LATENTS = [(4, 16, 8, 8, 24, None, None), (1, 8, 2, 8, 5, (1.5, 16, 2.0, 1.0), None), (3, 12, 4, 20, 40, None, None), (2, 4, 6, 4, 16, None, 4),
           (8, 64, 32, 96, 160, (2.0, 256, 32.0, 1.0), None), (4, 32, 64, 32, 64, (4.0, 128, 16.0, 1.0), None), (16, 16, 32, 16, 96, None, None),
           (2, 128, 64, 128, 192, (8.0, 64, 4.0, 2.0), None), (2, 24, 0, 8, 16, None, None)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dr,dv,rank,scaling,dims", LATENTS)
def test_latent_attention_finds_a_far_key(H, d, dr, dv, rank, scaling, dims, dtype):
    """The mixer with the up projections folded around its one cached key head, against keys and values of every head
    written out.  The input projections cut q, the latent and the gates out of the input, so that the test writes them: some
    queries are aligned with one key hundreds of tokens back, with the sequence's first key, with a key on a page border."""
    require_gpu()
    layer = tv.latent(H, d, dr, dv, rank, base=5000.0, scaling=scaling, dims=dims)
    spec = _mixer_spec(layer, 8)
    m = layer["mixer"]
    width = H * (d + dr) + rank + dr + H
    spec.params["hidden_size"] = width
    g = torch.Generator().manual_seed(H * 10 + rank)
    wts = {"q": _selection(H * (d + dr), width, 0), "dkv": _selection(rank + dr, width, H * (d + dr)), "g": _selection(H, width, H * (d + dr) + rank + dr),
           "dkv.norm": torch.rand(rank, generator=g) + 0.5, "uk": torch.randn(H * d, rank, generator=g) / rank ** 0.5,
           "uv": torch.randn(H * dv, rank, generator=g) / rank ** 0.5, "o": torch.randn(width, H * dv, generator=g) / (H * dv) ** 0.5}
    wts = {k: v.to(torch.bfloat16).float() for k, v in wts.items()}
    n, n2 = 700, 66
    h = torch.randn(n, width, generator=g)
    probes = {699: 3, 650: 0, 600: 63, 601: 64, 640: 320, 641: 641, 500: 499}
    for p, key in probes.items():
        cc = rms_unit(h[key, H * (d + dr): H * (d + dr) + rank].double(), 1e-5) * wts["dkv.norm"].double()
        for hh in range(H):
            ku = wts["uk"].double().view(H, d, rank)[hh] @ cc
            h[p, hh * (d + dr): hh * (d + dr) + d] = (ku / ku.norm() * 14.0 / m["scale"] / ku.norm()).float()      # score 14 above the others
    hs = [h, h[:n2].clone()]
    c = _context(dtype, cap=768)
    plain = _plain_for(wts, dtype)
    want = [plain.latent_attention(x.double(), torch.arange(x.shape[0]), m, "m.", 1e-5) for x in hs]
    got = _MixerRun(c, spec, wts).feed(hs, [590] + [1] * 110)
    _assert_close(got, want, dtype, "latent attention")
    got = _MixerRun(c, spec, wts).feed(hs, [2, 3, 61, 2, 700])
    _assert_close(got, want, dtype, "latent attention in portions")


@pytest.mark.gpu
@pytest.mark.parametrize("H,d,dr,dv,rank", [(4, 32, 32, 64, 64), (3, 64, 32, 64, 160), (2, 100, 28, 40, 48), (2, 128, 64, 128, 96), (5, 160, 64, 72, 64),
                                            (2, 8, 8, 200, 32)])
def test_latent_attention_with_keys_and_values_written_out_equals_the_folded_form(H, d, dr, dv, rank):
    """bfloat16 steps of many tokens write every head's keys and values out for the tensor-core prompt kernel (head sizes
    padded to 64, 128, 192 or 256 for keys and 64 or 128 for values; larger ones stay folded): the same results as the folded
    form, for prompts that start a sequence and for portions that go on in one, beside a second, shorter sequence."""
    require_gpu()
    layer = tv.latent(H, d, dr, dv, rank, scaling=(2.0, 64, 8.0, 1.0))
    W = 96
    spec = _mixer_spec(layer, W)
    g = torch.Generator().manual_seed(rank + d)
    wts = _random_weights(_params_of(spec), g, gain=2.0)
    hs = [torch.randn(n, W, generator=g) for n in (333, 70)]
    c = _context(torch.bfloat16)
    want = [_plain_for(wts, torch.bfloat16).latent_attention(x.double(), torch.arange(x.shape[0]), layer["mixer"], "m.", 1e-5) for x in hs]
    sizes = [130, 1, 1, 62, 3, 16, 200]
    run = _MixerRun(c, spec, wts)
    calls = []
    plain_call = c.ops._call
    c.ops._call = lambda name, *a: (calls.append(name), plain_call(name, *a))[1]
    try:
        got = run.feed(hs, sizes)
    finally:
        c.ops._call = plain_call
    fits = (d + dr + 63) // 64 * 64 <= 256 and (dv + 63) // 64 * 64 <= 128
    assert (calls.count("hb_latent_scatter") == 4) == fits and (calls.count("hb_attention_sink_prefill") == 4) == fits
    _assert_close(got, want, torch.bfloat16, "written out")
    folded = _MixerRun(c, spec, wts)
    folded.mixer.write_out = False
    ref = folded.feed(hs, sizes)
    for a, b in zip(got, ref):
        assert (a - b).abs().max() < 2e-2 * max(1.0, b.abs().max().item())


@pytest.mark.gpu
def test_rotation_tables_with_yarn():
    require_gpu()
    import types
    from hilbert_pruned_8b_b200.config import PartSpec
    from hilbert_pruned_8b_b200.parts import POSITION_ENCODINGS
    c = _context(torch.float32, 8)
    pos = torch.tensor([0, 1, 77, 1500, 9000], dtype=torch.int32, device=DEV)
    for dims, base, scaling in ((32, 20000.0, (3.0, 1024, 32.0, 1.0)), (8, 100.0, (4.0, 64, 4.0, 1.0)), (2, 10.0, (1.5, 16, 2.0, 1.0)), (64, 1e6, None)):
        sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
        params = {"head_dim": dims + 4, "rotary_dim": dims, "theta": base, "frequencies_in_64_bit": True}
        if sc:
            params["yarn"] = sc
        rope = POSITION_ENCODINGS.build(PartSpec("rotary", params), c)
        f, amp = rotary_frequencies(dims, base, sc)
        assert (torch.from_numpy(rope.inv_freq_host).double() - f).abs().max() <= 1e-7 * f.max()
        table, rot = rope.rotation_table(types.SimpleNamespace(positions=pos, num_tokens=5, shared={}))
        ang = torch.from_numpy(rope.inv_freq_host)[None, :] * pos.cpu().float()[:, None]         # 32-bit angles
        assert rot == dims and (table[..., 0].cpu().double() - torch.cos(ang.double()) * amp).abs().max() < 8e-7
        assert (table[..., 1].cpu().double() - torch.sin(ang.double()) * amp).abs().max() < 8e-7


# --------------------------------------------------------------------------- the engine
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(models, name, dtype):
    require_gpu()
    folder, cfg, plain = models[name]
    reqs = _requests(cfg, [1, 2, 7, 70, 150], 100)
    steps, peak = tt.trace_whole(reqs)
    eng = _engine(folder, dtype, peak)
    _compare(tt.run_in_process(eng, steps), _reference(plain, reqs, dtype), dtype, "whole")
    assert all(g.pool.num_free == g.pool.size for g in eng.cache.groups) and eng.cache.slots.num_held == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_the_residual_stream_after_every_layer(models, name):
    """Layer by layer in 32-bit: the first layer that differs names the mechanism."""
    require_gpu()
    from hilbert_pruned_8b_b200.engine.batch import StepEntry
    folder, cfg, plain = models[name]
    toks = tt.random_tokens(90, cfg["vocab"], 150)
    eng = _engine(folder, "float32", 128)
    seen = []
    for b in eng.model.blocks:
        def wrapped(x, *a, _orig=b.forward, **kw):
            r = _orig(x, *a, **kw)
            seen.append(x.detach().double().cpu())
            return r
        b.forward = wrapped
    seq = eng.open_sequence()
    eng.step_chunked([StepEntry(seq, toks, [len(toks) - 1])])
    eng.close_sequence(seq)
    _, layers = plain["exact"].forward(toks, return_layers=True)
    assert len(seen) == len(cfg["layers"])
    for i, (got, want) in enumerate(zip(seen, layers)):
        assert (got - want).abs().max() < 1e-4 * max(1.0, want.abs().max().item()), f"layer {i} ({cfg['layers'][i]['type']})"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_tokens_one_by_one(models, name, dtype):
    """The decoded tokens carry windows over the prompt's end and over page borders."""
    require_gpu()
    folder, cfg, plain = models[name]
    reqs = _requests(cfg, [3, 60, 190], 200)
    steps, peak = tt.trace_tail(reqs, tail=75)
    eng = _engine(folder, dtype, peak)
    _compare(tt.run_in_process(eng, steps), _reference(plain, reqs, dtype), dtype, "tail")
    assert eng.graph_replays > 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompts_in_portions(models, name, dtype):
    """A prompt cut into portions of 2, 3, 1, 64, 5 ... tokens, and cut by the engine itself when a step brings more tokens
    than it takes at once."""
    require_gpu()
    folder, cfg, plain = models[name]
    toks = tt.random_tokens(170, cfg["vocab"], 300)
    steps, at = [], 0
    for n in (2, 3, 1, 64, 5, 2, 40, 2, 51):
        steps.append({"step": len(steps), "entries": [{"id": "p", "tokens": toks[at: at + n], "want": list(range(n))}],
                      "end": ["p"] if at + n == len(toks) else []})
        at += n
    assert at == len(toks)
    ref = _reference(plain, {"p": toks}, dtype)
    _compare(tt.run_in_process(_engine(folder, dtype, 192), steps), ref, dtype, "portions")
    whole = [{"step": 0, "entries": [{"id": "p", "tokens": toks, "want": list(range(len(toks)))}], "end": ["p"]}]
    _compare(tt.run_in_process(_engine(folder, dtype, 192, max_step_tokens=48), whole), ref, dtype, "cut by the engine")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_slots_and_pages_used_again(models, name, dtype):
    require_gpu()
    folder, cfg, plain = models[name]
    v = cfg["vocab"]
    batches = [{f"a{i}": (tt.random_tokens(n, v, 400 + i), p) for i, (n, p) in enumerate([(90, 70), (12, 1), (150, 129), (40, 39)])},
               {f"b{i}": (tt.random_tokens(n, v, 500 + i), p) for i, (n, p) in enumerate([(30, 2), (100, 64), (5, 5)])}]
    steps, peak = tt.trace_batches(batches)
    eng = _engine(folder, dtype, peak)
    reqs = {rid: t for b in batches for rid, (t, _) in b.items()}
    _compare(tt.run_in_process(eng, steps), _reference(plain, reqs, dtype), dtype, "batches")
    assert eng.graph_replays > 0
    assert all(g.pool.num_free == g.pool.size for g in eng.cache.groups) and eng.cache.slots.num_held == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_decoding(models, name):
    """Hundreds of single-token steps through the captured graphs: windows slide off their pages, which are given back,
    while the latents of every token stay."""
    require_gpu()
    folder, cfg, plain = models[name]
    toks = tt.random_tokens(460, cfg["vocab"], 600)
    steps = [{"step": 0, "entries": [{"id": "l", "tokens": toks[:4], "want": [3]}], "end": []}]
    for p in range(4, len(toks)):
        steps.append({"step": len(steps), "entries": [{"id": "l", "tokens": [toks[p]], "want": [0]}],
                      "end": ["l"] if p == len(toks) - 1 else []})
    eng = _engine(folder, "float32", 512)
    got = tt.run_in_process(eng, steps)
    ref = _reference(plain, {"l": toks}, "float32")
    _compare(got, {k: ref[k] for k in got}, "float32", "long decoding")
    assert eng.graph_replays > 400


def _greedy(plain, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(plain.logits(toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "edges"])
def test_greedy_generation_through_the_library(models, name):
    """hb.load(...).generate(...): the scheduler's batches, the sampler and the captured decode steps."""
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    folder, cfg, plain = models[name]
    prompts = [tt.random_tokens(n, cfg["vocab"], 800 + i) for i, n in enumerate([1, 9, 45, 3, 66])]
    llm = hb.load(folder, dtype="float32", max_tokens=64 * 8, max_batch=3)       # two batches: slots are used again
    res = llm.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    for r, p in zip(res, prompts):
        assert r.tokens == _greedy(plain["exact"], p, 10), f"prompt of {len(p)} tokens"
    assert llm.generator.stats.batches == 2
    assert all(g.pool.num_free == g.pool.size for g in llm.engine.cache.groups)


@pytest.mark.gpu
def test_replay_program(models, tmp_path):
    require_gpu()
    folder, cfg, plain = models["mixed"]
    batches = [{f"t{i}": (tt.random_tokens(n, cfg["vocab"], 900 + i), p) for i, (n, p) in enumerate([(70, 66), (9, 2)])}]
    steps, peak = tt.trace_batches(batches, want_all=False)
    reqs = {rid: t for rid, (t, _) in batches[0].items()}
    for dtype in DTYPES:
        ref = _reference(plain, reqs, dtype)
        got = tt.run_program(folder, dtype, steps, peak, str(tmp_path / dtype), cfg["vocab"])
        _compare(got, {k: ref[k] for k in got}, dtype, "trace_run")
