"""Small Tonovik configurations and weights for the tests.

The weights are drawn so that every mechanism moves the logits: norm weights and biases far from one and
zero, projection biases of the size of the projections, gates that are neither open nor shut.  Stored in
bfloat16, so that a 32-bit engine and the 64-bit plain model read the same numbers.
"""
import json
import os

import torch


def latent(heads, dim, rot_dim, vdim, rank, base=10000.0, scaling=None, scale=None, dims=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                                                  "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": rot}}


def parallel(left, right, left_scale=1.25, right_scale=0.8):
    heads, kv_heads, dim, vdim, size, rot = left
    h2, d2, dv2, decay, rot2 = right
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 1.5 * dim ** -0.5, "mask": {"size": size},
                 "rot": {"base": 10000.0, "dims": rot}},
        "right": {"heads": h2, "dim": d2, "vdim": dv2, "decay": list(decay), "rot": {"base": 300.0, "dims": rot2}},
        "left_scale": left_scale, "right_scale": right_scale}}


def with_mlp(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


def config(width, vocab, layers, eps=1e-5, scale=2.0):
    return {"architecture": "Tonovik", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


# both kinds of layer, with and without a feed-forward; windows that prompts pass; partly rotated heads; YaRN; odd sizes
MIXED = config(64, 200, [
    with_mlp(latent(4, 16, 8, 8, 24, scaling=(4.0, 64, 8.0, 1.0)), 80),
    with_mlp(parallel((4, 2, 16, 8, 20, 8), (2, 8, 16, (0.7, 0.98), 4)), None),
    with_mlp(latent(3, 12, 4, 20, 40, base=500.0), None),
    with_mlp(parallel((6, 1, 8, 12, 33, 8), (3, 12, 8, (0.5, 0.9, 0.999), 12)), 72)])
# sizes that are equal or 1 where the others differ: one head, as many kv heads as heads, a window of one token, a window longer
# than any prompt, heads that are not rotated at all or wholly, decays of one and of zero, an embedding scale of one, a rank
# smaller than a head, rotated parts of two dimensions, branch weights of one and zero
EDGES = config(48, 130, [
    with_mlp(parallel((1, 1, 8, 12, 1, 0), (1, 4, 4, (1.0,), 0), 1.0, 1.0), 24),
    with_mlp(latent(1, 8, 2, 8, 5, scaling=(1.5, 16, 2.0, 1.0)), None),
    with_mlp(parallel((2, 2, 8, 4, 1000, 8), (3, 8, 4, (0.0, 0.5, 1.0), 8), 0.5, 1.5), None),
    with_mlp(latent(2, 4, 6, 4, 16, dims=4), 16),
    with_mlp(parallel((3, 3, 4, 4, 2, 2), (2, 2, 2, (0.25, 0.75), 2), 1.0, 0.0), 8)], eps=1e-6, scale=1.0)
# widths the tensor-core products take; head sizes of 64 and 128 (the tensor-core prompt kernels, also for the latent's one
# key head); sixteen heads; windows that straddle page borders; a window of exactly one page
WIDE = config(128, 300, [
    with_mlp(latent(4, 32, 64, 32, 64, scaling=(2.0, 128, 16.0, 1.0)), 192),
    with_mlp(parallel((2, 1, 64, 128, 70, 32), (2, 32, 64, (0.9, 0.999), 16)), 64),
    with_mlp(latent(16, 16, 32, 16, 128), None),
    with_mlp(parallel((4, 2, 128, 64, 64, 128), (4, 16, 16, (0.5, 0.8, 0.95, 0.99), 16)), 160),
    with_mlp(latent(2, 64, 16, 64, 96, scaling=(8.0, 32, 4.0, 2.0)), 64)])

CONFIGS = {"mixed": MIXED, "edges": EDGES, "wide": WIDE}


def draw_tensors(cfg, seed):
    """name -> bfloat16 tensor for every tensor the configuration's model reads."""
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.engine.model import weight_table
    table = weight_table(hb.TonovikConfig.from_dict(cfg).model_spec(), "")
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in table.items():
        shape = tuple(spec.shape)
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        leaf = name.split(".")[-1]
        if name.endswith(("norm1.b", "norm2.b", "final.norm.b")):
            t = n(0.3)
        elif leaf in ("norm", "norm1", "norm2"):
            t = n(0.2, 1.0)
        elif leaf == "b":
            t = n(0.5)
        elif name == "embed":
            t = n(1.0)
        elif leaf == "g":
            t = n(2.0 / shape[1] ** 0.5)
        elif len(shape) == 2:
            t = n(1.0 / shape[1] ** 0.5)
        else:
            t = n(1.0)
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed):
    from hilbert_pruned_8b_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    tensors = draw_tensors(cfg, seed)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return tensors
