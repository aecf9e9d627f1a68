"""The Moponex decoder against the plain implementation (tests/plain_moponex.py): every mechanism alone (the hashed pair
embedding, the factor on a sublayer's result with the next norm, the normed sum of two branches, the recurrent memory per
head in its two forms, the chunked attention with its sink, the score router with groups and identity experts, the gelu
units), then the engine: whole prompts, token-by-token decoding, prompts in portions down to two tokens, unequal batches
with slots and pages used again, long decoding, greedy generation through the library's entry point and the replay program."""
import copy
import math

import pytest
import torch

import moponex_tools as mp
import trace_tools as tt
from conftest import require_gpu
from plain_moponex import (PlainMoponex, bigram_rows, causal_conv, channel_decay_memory, chunk_attention_mixer, chunk_mask, dense_ff,
                           gated_linear_mixer, gelu_erf, gelu_tanh, head_state_scan, mamba2_mixer, moe_ff, parallel_mixer, rms_norm, rotate_pairs,
                           route, sink_softmax_attention, to_bf16)
from test_tonovik import _MixerRun, _compare, _context, _reference, _requests

DTYPES = ["float32", "bfloat16"]
NAMES = ["mixed", "edges", "wide"]
DEV = "cuda:0"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config, {"exact" | dtype: plain model})"""
    out = {}
    for i, (name, cfg) in enumerate(mp.CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("moponex_" + name))
        tensors = mp.write_model(d, cfg, 70 + i, state_rank=(name != "mixed"))
        out[name] = (d, cfg, {"exact": PlainMoponex(cfg, tensors), "float32": PlainMoponex(cfg, tensors, dtype=torch.float32),
                              "bfloat16": PlainMoponex(cfg, tensors, round_to=torch.bfloat16)})
    return out


def _engine(folder, dtype, max_tokens, **kw):
    from hilbert_pruned_8b_b200.engine.step import Engine
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, **kw)


# --------------------------------------------------------------------------- without a GPU
def test_config_round_trip_weight_table_and_sizes_from_shapes(tmp_path):
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.config import ConfigError, config_class_for
    from hilbert_pruned_8b_b200.engine.model import weight_table
    for cfg in mp.CONFIGS.values():
        assert config_class_for(cfg) is hb.MoponexConfig
        c = hb.MoponexConfig.from_dict(cfg)
        assert hb.MoponexConfig.from_dict(c.to_dict()) == c
        table = weight_table(c.model_spec(), "")
        assert ("bigram" in table) == ("embedding" in cfg)
        for i, layer in enumerate(cfg["layers"]):
            assert f"l{i}.norm1" in table and (f"l{i}.norm2" in table) == (layer["mlp"] is not None)
            assert (f"l{i}.mix.left.sink" in table) == (layer["type"] == "parallel") == (f"l{i}.mix.right.a2.b" in table) == (f"l{i}.mix.left.out" in table)
            assert (f"l{i}.mix.A_log" in table) == (layer["type"] == "mamba2")
            assert f"l{i}.mix.left.v" not in table and f"l{i}.mix.left.o.b" not in table
            if layer["mlp"] and layer["mlp"]["kind"] == "moe":
                r = layer["mlp"]["router"]
                assert table[f"l{i}.mlp.router"].shape == (r["experts"] + r["identity"], cfg["width"])
                assert f"l{i}.mlp.e{r['experts'] - 1}.up" in table and f"l{i}.mlp.e{r['experts']}.up" not in table and f"l{i}.mlp.e0.gate" not in table
                assert (f"l{i}.mlp.shared.sg" in table) == (layer["mlp"]["shared"] is not None)
    table = weight_table(hb.MoponexConfig.from_dict(mp.MIXED).model_spec(), "")
    m0, m1 = mp.MIXED["layers"][0]["mixer"], mp.MIXED["layers"][1]["mixer"]
    inner, gn = m0["heads"] * m0["vdim"], m0["groups"] * m0["state"]
    assert table["l0.mix.in"].shape == (2 * inner + 2 * gn + m0["heads"], 64) and table["l0.mix.conv"].shape == (inner + 2 * gn, m0["conv"])
    assert table["l1.mix.left.k"].shape == (m1["left"]["kv_heads"] * m1["left"]["dim"], 64) and table["l1.mix.left.q.norm"].shape == (m1["left"]["dim"],)
    assert table["l1.mix.right.a1"].shape == (4, 64) and table["l1.mix.right.a2"].shape == (m1["right"]["heads"] * m1["right"]["dim"], 4)
    assert table["l1.mix.right.norm"].shape == (m1["right"]["vdim"],) and table["bigram"].shape == (62, 64)
    # a size that only a tensor's shape gives: without it the model cannot be described, with the shapes it can
    bare = copy.deepcopy(mp.MIXED)
    for layer in bare["layers"]:
        if layer["type"] == "parallel":
            del layer["mixer"]["right"]["decay_rank"]
    c = hb.MoponexConfig.from_dict(bare)
    with pytest.raises(ConfigError):
        c.model_spec()
    filled = c.with_tensor_shapes({"l1.mix.right.a1": (4, 64), "l3.mix.right.a1": (5, 64)})
    assert filled == hb.MoponexConfig.from_dict(mp.MIXED)
    with pytest.raises(ConfigError):
        hb.MoponexConfig.from_dict(mp.MIXED).with_tensor_shapes({"l1.mix.right.a1": (9, 64)})
    d = str(tmp_path / "m")
    mp.write_model(d, mp.MIXED, 3, state_rank=False)
    assert hb.load_config(d) == hb.MoponexConfig.from_dict(mp.MIXED)

    def changed(layer, path, value):
        layer = copy.deepcopy(layer)
        d = layer
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = value
        return {**mp.MIXED, "layers": [layer]}
    par, ssm = mp.MIXED["layers"][1], mp.MIXED["layers"][0]
    for bad in ({**mp.MIXED, "layers": []}, {**mp.MIXED, "width": 0}, {k: v for k, v in mp.MIXED.items() if k != "norm"},
                {**mp.MIXED, "layers": [{"type": "conv", "mixer": {}, "mlp": None}]},
                changed(par, ("mixer", "left", "kv_heads"), 3), changed(par, ("mixer", "left", "vdim"), 8), changed(par, ("mixer", "left", "rot", "dims"), 7),
                changed(par, ("mixer", "left", "rot", "dims"), 18), changed(par, ("mixer", "left", "mask", "size"), 0), changed(par, ("mixer", "right", "tau"), 0.0),
                changed(par, ("mlp", "router", "top"), 5), changed(par, ("mlp", "router", "groups", "count"), 3), changed(par, ("mlp", "router", "groups", "keep"), 5),
                changed(ssm, ("mixer", "groups"), 3), changed(ssm, ("mixer", "norm_groups"), 5), changed(ssm, ("mlp", "kind"), "glu")):
        with pytest.raises(ConfigError):
            hb.MoponexConfig.from_dict(bad)


def test_plain_mechanisms_agree_with_their_definitions():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    # the pair table's rows: the last row for a first token, the hash of (previous, token) after it
    assert bigram_rows([5, 9, 9], 7, 3, 2) == [7, (5 * 3 + 9 * 2) % 7, (9 * 3 + 9 * 2) % 7]
    # the convolution looks back taps - 1 tokens and sees zeros before the start
    x, w, b = r(5, 2), r(2, 3), r(2)
    y = causal_conv(x, w, b)
    assert torch.allclose(y[0], b + w[:, 2] * x[0]) and torch.allclose(y[4], b + w[:, 0] * x[2] + w[:, 1] * x[3] + w[:, 2] * x[4])
    # the state-space memory equals the explicit sums: y_t = sum_s prod_{s<r<=t} a_r dt_s (C_t . B_s) x_s + D x_t
    T, H, P, G, N = 6, 2, 3, 1, 4
    xs, B, C, dt, A, D = r(T, H, P), r(T, G, N), r(T, G, N), r(T, H).abs() + 0.1, -r(H).abs(), r(H)
    y = head_state_scan(xs, B, C, dt, A, D)
    for h in range(H):
        want = D[h] * xs[5, h] + sum(torch.exp(A[h] * dt[s + 1:, h].sum()) * dt[s, h] * (C[5, 0] @ B[s, 0]) * xs[s, h] for s in range(T))
        assert torch.allclose(y[5, h], want)
    # the memory with a decay per key channel: o_t = sum_s sum_c q_tc k_sc prod_{s<r<=t} alpha_rc v_s
    q, k, v, al = r(5, 2, 3), r(5, 2, 3), r(5, 2, 4), torch.rand(5, 2, 3, generator=g, dtype=torch.float64)
    o = channel_decay_memory(q, k, v, al)
    want = sum((q[4, 1] * k[s, 1] * al[s + 1:, 1].prod(0)).sum() * v[s, 1] for s in range(5))
    assert torch.allclose(o[4, 1], want)
    # chunks: query 10 with chunks of 4 sees 8, 9, 10; the sink takes its share of the sum and brings no value
    assert chunk_mask(12, 4)[10].tolist() == [False] * 8 + [True] * 3 + [False] and chunk_mask(3, None)[2].all()
    q, k, v, sink = r(12, 2, 3), r(12, 1, 3), r(12, 1, 2), torch.tensor([0.3, 50.0], dtype=torch.float64)
    out = sink_softmax_attention(q, k, v, 0.7, chunk_mask(12, 4), sink)
    e = torch.exp(torch.stack([q[10, 0] @ k[j, 0] for j in range(8, 11)]) * 0.7)
    assert torch.allclose(out[10, 0], (e[:, None] * v[8:11, 0]).sum(0) / (e.sum() + math.exp(0.3)))
    assert out[:, 1].abs().max() < 1e-6                  # a sink far above every score leaves nothing for the values
    # interleaved pairs; a score depends on the distance only; stretched positions
    t = r(1, 1, 6)
    got = rotate_pairs(t, torch.tensor([5]), 4, 100.0, 2.0)[0, 0]
    for i, a in enumerate((2.5, 0.25)):
        assert torch.allclose(got[2 * i], t[0, 0, 2 * i] * math.cos(a) - t[0, 0, 2 * i + 1] * math.sin(a))
        assert torch.allclose(got[2 * i + 1], t[0, 0, 2 * i + 1] * math.cos(a) + t[0, 0, 2 * i] * math.sin(a))
    assert torch.equal(got[4:], t[0, 0, 4:])
    # the router: only the best groups' outputs can be chosen, by score + correction; weights from the scores alone
    h, wr = r(1, 5), r(8, 5)
    corr = torch.tensor([0.0, 0.0, 9.0, 0.0, 0.0, 0.0, -9.0, 0.0], dtype=torch.float64)
    c = {"router": {"experts": 6, "identity": 2, "top": 3, "groups": {"count": 4, "keep": 2}}}
    chosen, weights = route(h, wr, corr, c)
    s = torch.softmax(h @ wr.T, -1)[0]
    assert 2 in chosen[0].tolist() and 6 not in chosen[0].tolist() and abs(weights.sum().item() - 1) < 1e-12
    assert torch.allclose(weights[0], s[chosen[0]] / s[chosen[0]].sum())
    groups_hit = {e // 2 for e in chosen[0].tolist()}
    assert len(groups_hit) <= 2 and 1 in groups_hit
    # an identity expert hands the input back
    w = {"router": torch.zeros(2, 5, dtype=torch.float64), "correction": torch.tensor([0.0, 1.0], dtype=torch.float64), "e0.up": r(3, 5), "e0.down": r(5, 3)}
    assert torch.allclose(moe_ff(h, w, {"router": {"experts": 1, "identity": 1, "top": 1}}), h)
    assert abs(gelu_tanh(torch.tensor(1.0)).item() - 0.841192) < 1e-5 and abs(gelu_erf(torch.tensor(1.0)).item() - 0.841345) < 1e-5


# --------------------------------------------------------------------------- kernels alone
@pytest.mark.gpu
def test_pair_embedding_in_portions_and_slots_used_again():
    require_gpu()
    from hilbert_pruned_8b_b200.cache.manager import CacheManager
    from hilbert_pruned_8b_b200.engine.batch import StepEntry, build_step
    from hilbert_pruned_8b_b200.parts import EMBEDDINGS
    from hilbert_pruned_8b_b200.config.spec import PartSpec
    c = _context(torch.float32)
    g = torch.Generator().manual_seed(2)
    vocab, width, buckets = 50, 24, 11
    emb = EMBEDDINGS.build(PartSpec("hashed_pair_embedding", {"vocab_size": vocab, "hidden_size": width, "tensor_name": "embed", "pair_tensor_name": "bigram",
                                                             "buckets": buckets, "mul_prev": 1000003, "mul_cur": 77}), c)
    table, pairs = torch.randn(vocab, width, generator=g).to(torch.bfloat16), torch.randn(buckets + 1, width, generator=g).to(torch.bfloat16)
    emb.bind({"embed": table.to(DEV), "bigram": pairs.to(DEV)})
    cache = CacheManager({}, {-1: emb.state_need()}, 64 * 8, c.device, torch.float32, max_sequences=3)
    for _ in range(2):                                   # the second round takes the slots the first one left
        toks = [tt.random_tokens(n, vocab, 5 + n) for n in (9, 1, 14)]
        seqs = [cache.open() for _ in toks]
        done, got = [0, 0, 0], [[], [], []]
        for portion in (1, 3, 2, 1, 1, 50):
            live = [i for i in range(3) if done[i] < len(toks[i])]
            if not live:
                break
            new = [min(portion, len(toks[i]) - done[i]) for i in live]
            entries = [StepEntry(seqs[i], toks[i][done[i]: done[i] + n], []) for i, n in zip(live, new)]
            step = build_step(entries, cache, c.workspace, c.device)
            out = torch.empty(sum(new), width, device=DEV)
            emb.forward(step.tokens, out, step=step, state=cache.state_view(-1))
            at = 0
            for i, n in zip(live, new):
                got[i].append(out[at: at + n].cpu().double())
                cache.commit(seqs[i], seqs[i].length + n)
                done[i] += n
                at += n
        for i, t in enumerate(toks):
            rows = bigram_rows(t, buckets, 1000003, 77)
            want = table.double()[torch.tensor(t)] + pairs.double()[torch.tensor(rows)]
            assert (torch.cat(got[i]) - want).abs().max() < 1e-6, f"sequence {i}"
        for s in seqs:
            cache.close(s)
    c.ops.check_errors()


@pytest.mark.gpu
def test_scaled_add_with_the_next_norm_and_the_normed_sum():
    require_gpu()
    c = _context(torch.float32)
    ops, g = c.ops, torch.Generator().manual_seed(4)
    for width in (1, 2, 72, 257, 2500, 9000):
        y, x = (torch.randn(19, width, generator=g) * 3).cuda(), torch.randn(19, width, generator=g).cuda()
        w, w2 = torch.randn(width, generator=g).cuda(), torch.randn(width, generator=g).cuda()
        want = x.double() + 0.37 * y.double()
        x1 = x.clone()
        ops.scaled_add_norm(y, 0.37, x1)
        assert (x1.double() - want).abs().max() < 2e-6
        for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 6e-2)):
            x2, h = x.clone(), torch.empty(19, width, dtype=dtype, device=DEV)
            ops.scaled_add_norm(y, 0.37, x2, then=(w, 1e-5, 0.0), then_out=h)
            assert torch.equal(x2, x1) and (h.double() - rms_norm(want, w.double(), 1e-5)).abs().max() < tol * max(1.0, w.abs().max().item())
        a, b = y, (torch.randn(19, width, generator=g) * 0.01).cuda()
        want = rms_norm(a.double(), w.double(), 1e-6) + rms_norm(b.double(), w2.double(), 1e-6)
        out = torch.full((19, width), 5.0, device=DEV)
        ops.normed_sum(a, w, b, w2, 1e-6, out)
        assert (out.double() - want).abs().max() < 3e-5 * max(1.0, want.abs().max().item())
        ops.normed_sum(a, w, b, w2, 1e-6, out, accumulate=True)
        assert (out.double() - 2 * want).abs().max() < 6e-5 * max(1.0, want.abs().max().item())
    ops.check_errors()


def _route_case(E, identity, top, groups, seed, T=37, W=40):
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(T, W, generator=g)
    wr = (torch.randn(E + identity, W, generator=g) * 3 / W ** 0.5).to(torch.bfloat16).float()
    corr = torch.randn(E + identity, generator=g) * 0.5 / (E + identity)
    c = {"router": {"experts": E, "identity": identity, "top": top}}
    if groups:
        c["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    return h, wr, corr, c


@pytest.mark.gpu
def test_score_router_groups_identity_experts_and_gelu_units():
    require_gpu()
    c = _context(torch.float32)
    ops = c.ops
    for E, identity, top, groups in ((6, 2, 3, (4, 2)), (5, 0, 2, None), (1, 0, 1, None), (3, 1, 4, (2, 2)), (2, 2, 2, (4, 2)), (40, 8, 6, (8, 3)), (7, 1, 1, (2, 1))):
        h, wr, corr, cfg = _route_case(E, identity, top, groups, 10 + E)
        chosen, weights = route(h.double(), wr.double(), corr.double(), cfg)
        experts = torch.empty(h.shape[0], top, dtype=torch.int32, device=DEV)
        wts = torch.empty(h.shape[0], top, device=DEV)
        ops.moe_route_scores(h.cuda(), wr.cuda(), corr.cuda(), top, groups[0] if groups else 1, groups[1] if groups else 1, experts, wts)
        for t in range(h.shape[0]):
            want = dict(zip(chosen[t].tolist(), weights[t].tolist()))
            got = dict(zip(experts[t].tolist(), wts[t].tolist()))
            assert set(want) == set(got), f"token {t}: {sorted(want)} against {sorted(got)}"
            assert all(abs(want[e] - got[e]) < 1e-5 for e in want)
    # negative choice scores: a group that is shut out stays out although its scores are above the chosen ones' choice scores
    h, wr, corr, cfg = _route_case(4, 0, 2, (2, 1), 3)
    corr = torch.tensor([-5.0, -5.0, -9.0, -9.0])
    experts, wts = torch.empty(37, 2, dtype=torch.int32, device=DEV), torch.empty(37, 2, device=DEV)
    ops.moe_route_scores(h.cuda(), wr.cuda(), corr.cuda(), 2, 2, 1, experts, wts)
    assert set(experts.flatten().tolist()) == {0, 1}
    # the experts with the exact gelu, identity experts among the chosen, one to many tokens, both product kernels
    g = torch.Generator().manual_seed(8)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        cd = _context(dtype, cap=512)
        for T, W, F, E, identity, top in ((1, 24, 10, 3, 1, 2), (5, 64, 32, 4, 2, 3), (333, 64, 24, 6, 2, 4), (70, 40, 8, 1, 3, 4)):
            for tc in (True, False):
                cd.ops.use_tensor_cores = tc
                wu, wd = (torch.randn(E, F, W, generator=g) / W ** 0.5).to(torch.bfloat16), (torch.randn(E, W, F, generator=g) / F ** 0.5).to(torch.bfloat16)
                h = torch.randn(T, W, generator=g).to(dtype)
                chosen = torch.stack([torch.randperm(E + identity, generator=g)[:top] for _ in range(T)]).to(torch.int32)
                weights = torch.rand(T, top, generator=g)
                want = torch.zeros(T, W, dtype=torch.float64)
                rnd = to_bf16 if dtype == torch.bfloat16 else (lambda z: z)
                for t in range(T):
                    for e, wgt in zip(chosen[t].tolist(), weights[t].double()):
                        want[t] += wgt * (h[t].double() if e >= E else rnd(gelu_erf(h[t].double() @ wu[e].double().T)) @ wd[e].double().T)
                out = torch.full((T, W), 2.0, device=DEV)
                cd.ops.moe_experts(h.cuda(), chosen.cuda(), weights.cuda(), wu.to(dtype).cuda(), None, wd.to(dtype).cuda(), 0.0, 0.0, out, True,
                                   cd.workspace, 512, tag=".t", identity=True)
                assert (out.cpu().double() - 2.0 - want).abs().max() < tol * max(1.0, want.abs().max().item()), (dtype, T, tc)
        cd.ops.use_tensor_cores = True
        cd.ops.check_errors()
    x = torch.randn(9, 2 * 13 + 3, generator=g).cuda()
    out = torch.empty(9, 13, device=DEV)
    ops.gelu_unit(x, out, "tanh_gated")
    assert (out.cpu().double() - gelu_tanh(x[:, :13].cpu().double()) * x[:, 13:26].cpu().double()).abs().max() < 1e-5
    ops.gelu_unit(x, out, "erf", row_gate=27)
    assert (out.cpu().double() - gelu_erf(x[:, :13].cpu().double()) * torch.sigmoid(x[:, 27:28].cpu().double())).abs().max() < 1e-5
    ops.check_errors()


# --------------------------------------------------------------------------- mixers alone
def _mixer_spec(layer, width, which=None):
    import hilbert_pruned_8b_b200 as hb
    spec = hb.MoponexConfig.from_dict(mp.config(width, 16, [mp.with_mlp(layer, None)])).model_spec().layers[0].parts["mixer"]
    if which is not None:
        return spec.params["branches"][which]["mixer"]
    return spec


def _mixer_weights(spec, seed, width):
    """Local name -> tensor for one mixer, drawn as the tools draw a model's."""
    from hilbert_pruned_8b_b200.parts import MIXERS
    from hilbert_pruned_8b_b200.engine.model import describe_context
    part = MIXERS.build(spec, describe_context())
    cfg = mp.config(width, 16, [])
    g = torch.Generator().manual_seed(seed)
    out = {}
    for p in part.params():
        leaf, shape = p.name.split(".")[-1], tuple(p.shape)
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        t = (n(0.2, 1.0) if leaf in ("norm", "out") and len(shape) == 1 else n(1.0, 2.0) if p.name.endswith("a2.b") else n(0.5) if leaf == "b"
             else n(1.5) if leaf == "sink" else n(0.7, -0.5) if leaf == "A_log" else n(1.0, -1.0) if leaf == "dt_bias" else n(0.5, 1.0) if leaf == "D"
             else n(0.6) if leaf == "conv" else n(1.0 / shape[1] ** 0.5) if len(shape) == 2 else n(1.0))
        out[p.name] = t.to(torch.bfloat16).float()
    return out


def _close(got, want, dtype, what):
    for i, (a, b) in enumerate(zip(got, want)):
        err = (a - b).abs().max(1).values / b.abs().max().clamp(min=1.0)
        assert err.max() < (1e-4 if dtype == torch.float32 else 3e-2), f"{what}: sequence {i} position {int(err.argmax())}: {float(err.max()):.3e}"


SSM = [(4, 8, 16, 2, 3, 2), (1, 8, 1, 1, 1, 1), (4, 4, 4, 4, 5, 4), (2, 64, 128, 1, 4, 2), (6, 40, 48, 3, 3, 1), (3, 20, 100, 1, 2, 3), (8, 16, 256, 2, 4, 1)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_space_heads_in_portions_against_the_recurrence(dtype):
    require_gpu()
    width = 40
    for n, (heads, vdim, state, groups, conv, norm_groups) in enumerate(SSM):
        layer = mp.mamba2(heads, vdim, state, groups, conv, norm_groups)
        spec = _mixer_spec(layer, width)
        w = _mixer_weights(spec, 20 + n, width)
        g = torch.Generator().manual_seed(30 + n)
        hs = [torch.randn(t, width, generator=g).to(torch.bfloat16).float() for t in (70, 3, 131)]
        rnd = to_bf16 if dtype == torch.bfloat16 else (lambda z: z)
        want = [mamba2_mixer(h.double(), {k: v.double() for k, v in w.items()}, layer["mixer"], 1e-5, rnd) for h in hs]
        c = _context(dtype)
        for sizes in ((200,), (1, 2, 3, 1, 64, 5, 200), (33, 1, 1, 1, 1, 1, 200)):
            run = _MixerRun(c, spec, w)
            _close(run.feed(hs, sizes), want, dtype, f"state_space_heads {layer['mixer']} portions {sizes}")
            _close(run.feed(hs, sizes[::-1] + (200,)), want, dtype, "slots used again")     # the slots the first sequences left, not zeroed by the part
        # long portions cut into chunks that run side by side: the same sums
        c.ops.HEAD_SCAN_CHUNK_FROM = 8
        c.ops.sm_count = 10 ** 6
        _close(_MixerRun(c, spec, w).feed(hs, (100, 200)), want, dtype, "chunks side by side")


GLA = [(2, 8, 16, 8.0, 4), (1, 4, 4, 1.0, 1), (3, 12, 8, 2.0, 5), (2, 64, 32, 16.0, 8), (1, 128, 64, 32.0, 8), (4, 40, 24, 64.0, 3), (2, 256, 16, 4.0, 16)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_linear_attention_in_portions_against_the_recurrence(dtype):
    require_gpu()
    width = 48
    for n, right in enumerate(GLA):
        layer = mp.parallel((1, 1, 8, None, None), right)
        spec = _mixer_spec(layer, width, which=1)
        w = _mixer_weights(spec, 40 + n, width)
        g = torch.Generator().manual_seed(50 + n)
        hs = [torch.randn(t, width, generator=g).to(torch.bfloat16).float() for t in (70, 3, 131)]
        rnd = to_bf16 if dtype == torch.bfloat16 else (lambda z: z)
        want = [gated_linear_mixer(h.double(), {k: v.double() for k, v in w.items()}, layer["mixer"]["right"], 1e-5, rnd) for h in hs]
        c = _context(dtype)
        for sizes in ((200,), (1, 2, 3, 1, 64, 5, 200), (33, 1, 1, 1, 1, 1, 200)):
            run = _MixerRun(c, spec, w)
            _close(run.feed(hs, sizes), want, dtype, f"gated_linear_attention {right} portions {sizes}")
            _close(run.feed(hs, (7, 200)), want, dtype, "slots used again")
        c.ops.HEAD_SCAN_CHUNK_FROM = 8
        c.ops.sm_count = 10 ** 6
        _close(_MixerRun(c, spec, w).feed(hs, (100, 200)), want, dtype, "chunks side by side")
    # decays of (nearly) one and (nearly) zero: a bias of +-40 on every channel
    layer = mp.parallel((1, 1, 8, None, None), (2, 8, 8, 1.0, 2))
    spec = _mixer_spec(layer, width, which=1)
    for bias in (40.0, -40.0):
        w = _mixer_weights(spec, 9, width)
        w["a2.b"] = torch.full_like(w["a2.b"], bias)
        hs = [torch.randn(90, width, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).float()]
        rnd = to_bf16 if dtype == torch.bfloat16 else (lambda z: z)
        want = [gated_linear_mixer(hs[0].double(), {k: v.double() for k, v in w.items()}, layer["mixer"]["right"], 1e-5, rnd)]
        _close(_MixerRun(_context(dtype), spec, w).feed(hs, (40, 1, 1, 200)), want, dtype, f"decay bias {bias}")


def _selection(rows, width, at):
    m = torch.zeros(rows, width)
    m[torch.arange(rows), at + torch.arange(rows)] = 1.0
    return m


# (heads, kv heads, dim, chunk, rotated dims): the general kernel, the one-block-per-token kernel in its variants, the
# tensor-core prompt kernel (key heads of 64 and 128 in bfloat16), sixteen heads (weights times values on the tensor cores)
CHUNKS = [(4, 2, 16, 20, 8), (1, 1, 8, 1, 0), (3, 3, 4, 1000, 4), (2, 1, 64, 64, 16), (16, 4, 64, 70, 64), (2, 2, 128, 100, 16), (6, 2, 24, 63, 24),
          (5, 1, 12, 65, 6), (2, 1, 64, None, 64)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_chunked_attention_with_probes_at_the_edges_and_a_sink(dtype):
    require_gpu()
    for n, (H, G, d, chunk, rot) in enumerate(CHUNKS):
        width = H * d + G * d
        layer = mp.parallel((H, G, d, chunk, (rot, 100.0, 2.0) if rot else None), (1, 2, 2, 1.0, 1))
        layer["mixer"]["left"]["scale"] = 3.0 / d ** 0.5 * (4.0 if rot == 0 else 1.0)
        spec = _mixer_spec(layer, width, which=0)
        g = torch.Generator().manual_seed(60 + n)
        # q and k are cut out of the input, so that a probe can be written into it: a query and one key far back in the same
        # direction give a score that stands out (the norm makes both of unit mean square; rotation is off for probes' dims
        # only where rot == 0, elsewhere the probes still stand out at short distances)
        w = {"q": _selection(H * d, width, 0), "k": _selection(G * d, width, H * d), "q.b": torch.zeros(H * d), "k.b": torch.randn(G * d, generator=g) * 0.1,
             "q.norm": torch.ones(d), "k.norm": torch.ones(d), "sink": torch.randn(H, generator=g) * 2, "o": torch.randn(width, H * d, generator=g) / (H * d) ** 0.5}
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
        T = 200
        hs = [torch.randn(T, width, generator=g), torch.randn(77, width, generator=g), torch.randn(1, width, generator=g)]
        size = chunk if chunk is not None else 10 ** 9
        probes = []
        for p in (5, 63, 64, 65, 127, 128, 130, 199):
            start = p - p % size
            for s in (start, start - 1, p - 1, 0):            # just inside the chunk, just outside it, the neighbour, the first token
                if 0 <= s < p:
                    probes.append((p, s))
        for i, (p, s) in enumerate(probes[: 2 * H]):
            head = i % H
            direction = torch.randn(d, generator=g)
            hs[0][p, head * d: (head + 1) * d] = direction * 5
            hs[0][s, H * d + (head // (H // G)) * d: H * d + (head // (H // G) + 1) * d] = direction * 5
        hs = [h.to(torch.bfloat16).float() for h in hs]
        rnd = to_bf16 if dtype == torch.bfloat16 else (lambda z: z)
        want = [chunk_attention_mixer(h.double(), {k: v.double() for k, v in w.items()}, layer["mixer"]["left"], 1e-5, torch.arange(h.shape[0]), rnd)
                for h in hs]
        c = _context(dtype)
        for sizes in ((300,), (60, 3, 1, 1, 1, 1, 1, 1, 1, 58, 1, 1, 1, 1, 1, 1, 1, 300), (2, 126, 1, 1, 300)):
            run = _MixerRun(c, spec, w)
            _close(run.feed(hs, sizes), want, dtype, f"chunk attention {(H, G, d, chunk, rot)} portions {sizes}")
        for flag in ("use_mma_attention", "use_flash_sink_attention"):      # the other kernels for the same steps
            setattr(c.ops, flag, False)
            _close(_MixerRun(c, spec, w).feed(hs, (150, 1, 1, 300)), want, dtype, f"chunk attention {(H, G, d, chunk, rot)} without {flag}")
        run = _MixerRun(c, spec, w)
        run.mixer.use_heads_kernel = False
        _close(run.feed(hs, (150, 1, 1, 300)), want, dtype, f"chunk attention {(H, G, d, chunk, rot)}, the general kernel")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parallel_mixer_with_its_branch_norms(dtype):
    require_gpu()
    width = 64
    layer = mp.parallel((4, 2, 16, 20, (8, 1000.0, 4.0)), (2, 8, 16, 8.0, 4))
    spec = _mixer_spec(layer, width)
    w = _mixer_weights(spec, 77, width)
    g = torch.Generator().manual_seed(78)
    hs = [torch.randn(t, width, generator=g).to(torch.bfloat16).float() for t in (90, 2, 45)]
    rnd = to_bf16 if dtype == torch.bfloat16 else (lambda z: z)
    want = [parallel_mixer(h.double(), {k: v.double() for k, v in w.items()}, layer["mixer"], 1e-5, torch.arange(h.shape[0]), rnd) for h in hs]
    for sizes in ((100,), (3, 2, 1, 1, 30, 100)):
        _close(_MixerRun(_context(dtype), spec, w).feed(hs, sizes), want, dtype, f"parallel mixer portions {sizes}")


# --------------------------------------------------------------------------- the engine
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_token_by_token(models, name, dtype):
    require_gpu()
    folder, cfg, plain = models[name]
    requests = _requests(cfg, [150, 64, 1, 2, 65], 100)
    ref = _reference(plain, requests, dtype)
    eng = _engine(folder, dtype, 64 * 12)
    steps, _ = tt.trace_whole(requests)
    _compare(tt.run_in_process(eng, steps), ref, dtype, f"{name} whole")
    steps, _ = tt.trace_tail(requests, tail=75)
    _compare(tt.run_in_process(eng, steps), ref, dtype, f"{name} last 75 tokens one by one")
    assert all(g.pool.num_free == g.pool.size for g in eng.cache.groups)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompts_in_portions(models, name, dtype):
    require_gpu()
    folder, cfg, plain = models[name]
    requests = _requests(cfg, [170, 71], 200)
    ref = _reference(plain, requests, dtype)
    eng = _engine(folder, dtype, 64 * 12)
    for sizes in ((2, 3, 1, 64, 1, 1, 5, 300), (63, 1, 1, 2, 300), (128, 1, 300)):
        steps = []
        for rid, toks in requests.items():
            at = 0
            for n in sizes:
                part = toks[at: at + n]
                if not part:
                    break
                steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": part, "want": list(range(len(part)))}],
                              "end": [rid] if at + n >= len(toks) else []})
                at += n
        _compare(tt.run_in_process(eng, steps), ref, dtype, f"{name} portions {sizes}")
    # steps cut by the engine itself
    small = _engine(folder, dtype, 64 * 12, max_step_tokens=48)
    steps, _ = tt.trace_whole(requests)
    _compare(tt.run_in_process(small, steps), ref, dtype, f"{name} steps of 48 tokens")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_slots_and_pages_used_again(models, name, dtype):
    require_gpu()
    folder, cfg, plain = models[name]
    lengths = [(140, 100), (30, 3), (67, 64), (90, 1), (129, 128), (12, 12)]
    requests = _requests(cfg, [n for n, _ in lengths], 300)
    ref = _reference(plain, requests, dtype)
    ids = list(requests)
    batches = [{ids[i]: (requests[ids[i]], lengths[i][1]) for i in (0, 1, 2)}, {ids[i]: (requests[ids[i]], lengths[i][1]) for i in (3, 4, 5)},
               {ids[i]: (requests[ids[i]], lengths[i][1]) for i in (1, 4)}]
    steps, peak = tt.trace_batches(batches)
    eng = _engine(folder, dtype, peak + 64, max_sequences=3)
    _compare(tt.run_in_process(eng, steps), ref, dtype, f"{name} batches")
    assert all(g.pool.num_free == g.pool.size for g in eng.cache.groups)
    assert eng.graph_replays > 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_decoding_and_fused_norms_against_separate_ones(models, name):
    require_gpu()
    folder, cfg, plain = models[name]
    requests = _requests(cfg, [420], 400)
    ref = _reference(plain, requests, "float32")
    eng = _engine(folder, "float32", 64 * 8)
    steps, _ = tt.trace_tail(requests, tail=400)
    got = tt.run_in_process(eng, steps)
    _compare(got, ref, "float32", f"{name} 400 decoded tokens")
    assert eng.graph_replays > 300
    plainer = _engine(folder, "float32", 64 * 8)
    for b in plainer.model.blocks:
        b.fuse_norms = False
    steps, _ = tt.trace_whole(requests)
    other = tt.run_in_process(plainer, steps)
    assert max((other[k] - got[k]).abs().max().item() for k in got) < 1e-3 * max(1.0, max(v.abs().max().item() for v in got.values()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_and_the_replay_program(models, dtype, tmp_path):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    folder, cfg, plain = models["mixed"]
    prompts = [tt.random_tokens(n, cfg["vocab"], 500 + n) for n in (40, 3, 21, 1, 66)]
    llm = hb.load(folder, dtype=dtype, max_tokens=64 * 8, max_batch=3)        # two batches: slots are used again
    res = llm.generate(prompts, max_new_tokens=24, stop_token_ids=[])
    for prompt, r in zip(prompts, res):
        assert len(r.tokens) == 24
        if dtype == "float32":
            # every generated token is the plain model's choice given the tokens before it (two nearly tied logits aside)
            lg = plain["exact"].logits(prompt + r.tokens)
            for i, t in enumerate(r.tokens):
                row = lg[len(prompt) + i - 1]
                assert row[t] >= row.max() - 1e-3 * max(1.0, row.abs().max().item()), f"prompt of {len(prompt)} tokens, token {i}"
    assert llm.generator.stats.batches == 2
    assert all(g.pool.num_free == g.pool.size for g in llm.engine.cache.groups)
    requests = _requests(cfg, [70, 9], 600)
    ref = _reference(plain, requests, dtype)
    steps, peak = tt.trace_batches([{rid: (toks, len(toks) - 5) for rid, toks in requests.items()}])
    got = tt.run_program(folder, dtype, steps, peak, str(tmp_path / "out"), cfg["vocab"])
    _compare(got, ref, dtype, "replay program")
