"""Small Moponex configurations and weights for the tests.

The weights are drawn so that every mechanism moves the logits: norm weights far from one, projection biases of the
size of the projections, sinks that take a visible share of the softmax, decays that are neither one nor zero, router
corrections of the size of the scores (some negative), gates that are neither open nor shut.  Stored in bfloat16, so
that a 32-bit engine and the 64-bit plain model read the same numbers.
"""
import json
import os

import torch


def mamba2(heads, vdim, state, groups=1, conv=4, norm_groups=1):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def parallel(left, right):
    heads, kv_heads, dim, size, rot = left
    h2, d2, dv2, tau, rank = right
    a = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": 1.3 * dim ** -0.5}
    if size is not None:
        a["mask"] = {"size": size}
    if rot is not None:
        dims, base, factor = rot
        a["rot"] = {"base": base, "dims": dims}
        if factor is not None:
            a["rot"]["scaling"] = {"factor": factor}
    return {"type": "parallel", "mixer": {"left": a, "right": {"heads": h2, "dim": d2, "vdim": dv2, "tau": tau, "decay_rank": rank}}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0, groups=None, shared=None):
    router = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": router, "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


def config(width, vocab, layers, eps=1e-5, mult=0.7, logit_scale=0.8, bigram=(61, 7, 13)):
    c = {"architecture": "Moponex", "layers": layers, "logit_scale": logit_scale, "norm": {"eps": eps}, "residual_mult": mult,
         "vocab": vocab, "width": width}
    if bigram is not None:
        c["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return c


# both kinds of layer, every kind of feed-forward and none; chunks that prompts pass several times; partly rotated heads
# with stretched positions; grouped state-space parameters and a grouped norm; identity experts, groups and a shared expert
MIXED = config(64, 200, [
    with_mlp(mamba2(4, 8, 16, groups=2, conv=3, norm_groups=2), dense(80)),
    with_mlp(parallel((4, 2, 16, 20, (8, 1000.0, 4.0)), (2, 8, 16, 8.0, 4)), moe(6, 3, 24, identity=2, groups=(4, 2), shared=32)),
    with_mlp(mamba2(3, 12, 10, conv=4), None),
    with_mlp(parallel((6, 1, 8, 33, (8, 300.0, None)), (3, 12, 8, 2.0, 5)), moe(5, 2, 16)),
    with_mlp(mamba2(2, 16, 24, groups=2, conv=2), moe(4, 1, 8, identity=1, shared=8))])
# sizes that are equal or 1 where the others differ: one head, as many groups as heads, a convolution of one tap, a norm
# group per head, a chunk of one token, a chunk longer than any prompt, no mask at all, heads that are not rotated or wholly,
# tau of one, a rank of one, one expert, every expert chosen, as many kept groups as groups, factors of one, no pair table
EDGES = config(48, 130, [
    with_mlp(mamba2(1, 8, 1, conv=1), dense(8)),
    with_mlp(parallel((1, 1, 8, 1, None), (1, 4, 4, 1.0, 1)), moe(1, 1, 8)),
    with_mlp(mamba2(4, 4, 4, groups=4, conv=5, norm_groups=4), moe(3, 4, 8, identity=1, groups=(2, 2))),
    with_mlp(parallel((2, 2, 8, 1000, (8, 50.0, 1.0)), (3, 8, 4, 64.0, 3)), None),
    with_mlp(parallel((3, 3, 4, None, (0, 10.0, None)), (2, 2, 2, 3.0, 2)), moe(2, 2, 4, identity=2, groups=(4, 2), shared=4))],
    eps=1e-6, mult=1.0, logit_scale=1.0, bigram=None)
# widths the tensor-core products take; key heads of 64 and 128 (the tensor-core prompt kernel); sixteen heads; chunks of
# exactly one page and chunks that straddle pages; states of 64 and 128; experts whose sizes the tensor-core tiles take
WIDE = config(128, 300, [
    with_mlp(mamba2(4, 32, 64, groups=2), moe(8, 2, 64, identity=0, groups=(2, 1), shared=64)),
    with_mlp(parallel((2, 1, 64, 64, (16, 10000.0, 4.0)), (2, 64, 32, 12.0, 8)), dense(192)),
    with_mlp(mamba2(2, 64, 128, norm_groups=2), None),
    with_mlp(parallel((16, 4, 64, 70, (64, 500.0, None)), (4, 32, 32, 4.0, 16)), moe(6, 2, 32, identity=2, groups=(4, 3))),
    with_mlp(parallel((2, 2, 128, 100, (16, 100.0, 8.0)), (1, 128, 64, 32.0, 8)), dense(64))], bigram=(997, 1000003, 31))

CONFIGS = {"mixed": MIXED, "edges": EDGES, "wide": WIDE}


def draw_tensors(cfg, seed):
    """name -> bfloat16 tensor for every tensor the configuration's model reads."""
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.engine.model import weight_table
    table = weight_table(hb.MoponexConfig.from_dict(cfg).model_spec(), "")
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in table.items():
        if spec.optional:
            continue
        shape = tuple(spec.shape)
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        leaf = name.split(".")[-1]
        if leaf in ("norm", "norm1", "norm2", "out") and len(shape) == 1:
            t = n(0.2, 1.0)
        elif name.endswith("a2.b"):
            t = n(1.0, 2.0)
        elif leaf == "b":
            t = n(0.5)
        elif leaf == "sink":
            t = n(1.5)
        elif leaf == "correction":
            t = n(0.5 / shape[0])
        elif leaf == "A_log":
            t = n(0.7, -0.5)
        elif leaf == "dt_bias":
            t = n(1.0, -1.0)
        elif leaf == "D":
            t = n(0.5, 1.0)
        elif leaf == "conv":
            t = n(0.6)
        elif leaf == "router":
            t = n(3.0 / shape[1] ** 0.5)
        elif name in ("embed", "bigram"):
            t = n(1.0 if name == "embed" else 0.7)
        elif leaf == "g":
            t = n(2.0 / shape[1] ** 0.5)
        elif len(shape) == 2:
            t = n(1.0 / shape[1] ** 0.5)
        else:
            t = n(1.0)
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, state_rank=True):
    """Writes config.json and model.safetensors; ``state_rank`` False leaves ``decay_rank`` out of config.json, so that a
    reader must take it from the tensor's shape."""
    import copy
    from hilbert_pruned_8b_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    tensors = draw_tensors(cfg, seed)
    stored = copy.deepcopy(cfg)
    if not state_rank:
        for layer in stored["layers"]:
            if layer["type"] == "parallel":
                layer["mixer"]["right"].pop("decay_rank", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(stored, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return tensors
