"""Typed configuration of the Moponex decoder: a pre-norm stack (RMS norms) whose sublayers' results enter the residual
stream times one fixed factor, with two kinds of mixer (a state-space mixer with one scalar decay per head and token; a
softmax attention over chunks of positions with a sink, beside a gated linear attention with a decay per key channel, both
normed and averaged), a dense gated feed-forward, a mixture of experts with grouped, corrected routing, identity experts
and a gated shared expert, or none; a hashed embedding of token pairs beside the token embedding; the head is the embedding
table, its logits times a constant.

config.json keys (every size and every constant that may differ between models comes from here): ``architecture``
("Moponex"), ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (default 1), ``logit_scale`` (default 1),
``embedding.bigram {buckets, mul_prev, mul_cur}`` (optional) and ``layers``: a list of ``{"type", "mixer", "mlp"}`` with ``type``

* "mamba2": ``mixer`` = ``heads, vdim, state, groups, conv, norm_groups``;
* "parallel": ``mixer`` = ``left {heads, kv_heads, dim, vdim, scale, mask {size} | null, rot {base, dims, scaling {factor}} | null}``,
  ``right {heads, dim, vdim, tau}`` (the rank of the decay's two-step projection is the row count of the tensor
  ``l<i>.mix.right.a1``, which ``with_tensor_shapes`` reads; a config.json may state it as ``decay_rank``);

and ``mlp`` null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "router {experts, top, identity, groups {count, keep}}",
"expert {ff}", "shared {ff} | null"}``.  Tensor names: ``embed``, ``bigram``, ``l<i>.norm1|norm2``, ``l<i>.mix.*`` (``left.*`` /
``right.*`` and ``left.out`` / ``right.out`` below it for the parallel mixer), ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

import copy
import dataclasses
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, PlanEntry
from .vuladra import _float, _int, _number


def _optional_float(d: Any, key: str, where: str, default: float) -> float:
    return default if not isinstance(d, dict) or d.get(key) is None else _float(d, key, where)


def _mlp(mlp: Any, where: str) -> Optional[Dict[str, Any]]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config: {where}kind must be dense or moe (or mlp null)")
    if mlp["kind"] == "dense":
        return {"kind": "dense", "ff": _int(mlp, "ff", where)}
    router, expert, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
    rw = where + "router."
    r = {"experts": _int(router, "experts", rw), "top": _int(router, "top", rw),
         "identity": _int(router, "identity", rw, least=0) if isinstance(router, dict) and router.get("identity") is not None else 0}
    groups = router.get("groups") if isinstance(router, dict) else None
    if groups is not None:
        r["groups"] = {"count": _int(groups, "count", rw + "groups."), "keep": _int(groups, "keep", rw + "groups.")}
    outputs = r["experts"] + r["identity"]
    count, keep = (r["groups"]["count"], r["groups"]["keep"]) if groups is not None else (1, 1)
    if outputs % count or keep > count:
        raise ConfigError(f"config: {rw}groups do not divide the {outputs} router outputs, or keep more groups than there are")
    if r["top"] > outputs // count * keep:
        raise ConfigError(f"config: {rw}top is larger than the number of router outputs that can be chosen")
    out = {"kind": "moe", "router": r, "expert": {"ff": _int(expert, "ff", where + "expert.")}, "shared": None}
    if shared is not None:
        out["shared"] = {"ff": _int(shared, "ff", where + "shared.")}
    return out


@dataclass(frozen=True)
class MoponexConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    bigram: Optional[Dict[str, int]] = None
    layers: List[Dict[str, Any]] = field(default_factory=list)       # the validated entries of config.json
    eos_token_ids: List[int] = field(default_factory=list)
    max_position_embeddings: Optional[int] = None

    architecture = "Moponex"
    model_type = "moponex"

    # llama-style names that the generic entry points and the benchmark read
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, root: Dict[str, Any]) -> "MoponexConfig":
        if not isinstance(root, dict):
            raise ConfigError("config: config.json is not an object")
        vocab, width = _int(root, "vocab", ""), _int(root, "width", "")
        eps = _float(root.get("norm"), "eps", "norm.")
        bigram = None
        emb = root.get("embedding")
        if isinstance(emb, dict) and emb.get("bigram") is not None:
            b = emb["bigram"]
            bigram = {"buckets": _int(b, "buckets", "embedding.bigram."), "mul_cur": _int(b, "mul_cur", "embedding.bigram.", least=0),
                      "mul_prev": _int(b, "mul_prev", "embedding.bigram.", least=0)}
        raw = root.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config: layers must be a list with at least one entry")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or entry.get("type") not in ("mamba2", "parallel"):
                raise ConfigError(f"config: {where}type must be mamba2 or parallel")
            m = entry.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config: missing {where}mixer")
            mw = where + "mixer."
            if entry["type"] == "mamba2":
                mixer = {k: _int(m, k, mw) for k in ("heads", "vdim", "state", "conv")}
                mixer["groups"] = _int(m, "groups", mw) if m.get("groups") is not None else 1
                mixer["norm_groups"] = _int(m, "norm_groups", mw) if m.get("norm_groups") is not None else 1
                if mixer["heads"] % mixer["groups"]:
                    raise ConfigError(f"config: {mw}heads is no multiple of groups")
                if (mixer["heads"] * mixer["vdim"]) % mixer["norm_groups"]:
                    raise ConfigError(f"config: {mw}norm_groups does not divide heads * vdim")
            else:
                a, b = m.get("left"), m.get("right")
                lw, rw = mw + "left.", mw + "right."
                left = {k: _int(a, k, lw) for k in ("heads", "kv_heads", "dim", "vdim")}
                left["scale"] = _float(a, "scale", lw)
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"config: {lw}heads is no multiple of kv_heads")
                if left["vdim"] != left["dim"]:
                    raise ConfigError(f"config: {lw}vdim differs from dim, but the values are the keys")
                mask = a.get("mask")
                left["mask"] = {"size": _int(mask, "size", lw + "mask.")} if mask is not None else None
                rot = a.get("rot")
                left["rot"] = None
                if rot is not None:
                    dims = _int(rot, "dims", lw + "rot.", least=0)
                    if dims % 2 or dims > left["dim"]:
                        raise ConfigError(f"config: {lw}rot.dims must be even and at most dim")
                    scaling = rot.get("scaling")
                    left["rot"] = {"base": _float(rot, "base", lw + "rot."), "dims": dims,
                                   "scaling": {"factor": _float(scaling, "factor", lw + "rot.scaling.")} if scaling is not None else None}
                right = {k: _int(b, k, rw) for k in ("heads", "dim", "vdim")}
                right["tau"] = _float(b, "tau", rw)
                if not right["tau"] > 0.0:
                    raise ConfigError(f"config: {rw}tau must be positive")
                if b.get("decay_rank") is not None:
                    right["decay_rank"] = _int(b, "decay_rank", rw)
                mixer = {"left": left, "right": right}
            layers.append({"type": entry["type"], "mixer": mixer, "mlp": _mlp(entry.get("mlp"), where + "mlp.")})
        eos = root.get("eos_token_id")
        eos_ids = [int(eos)] if _number(eos) else [int(e) for e in eos if _number(e)] if isinstance(eos, list) else []
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config: eos_token_id {e} is outside the vocabulary")
        max_pos = root.get("max_position_embeddings")
        return cls(vocab=vocab, width=width, eps=eps, residual_mult=_optional_float(root, "residual_mult", "", 1.0),
                   logit_scale=_optional_float(root, "logit_scale", "", 1.0), bigram=bigram, layers=layers, eos_token_ids=eos_ids,
                   max_position_embeddings=int(max_pos) if _number(max_pos) and max_pos >= 1 else None)

    def with_tensor_shapes(self, shapes: Dict[str, Any]) -> "MoponexConfig":
        """The configuration with the sizes that only a tensor's shape gives (``shapes``: tensor name -> shape): the rank of
        every gated linear attention's decay projection."""
        layers = copy.deepcopy(self.layers)
        for i, l in enumerate(layers):
            if l["type"] != "parallel":
                continue
            name = f"l{i}.mix.right.a1"
            shape = shapes.get(name)
            if shape is not None and len(shape) == 2:
                stated = l["mixer"]["right"].get("decay_rank")
                if stated is not None and stated != int(shape[0]):
                    raise ConfigError(f"config: layers[{i}].mixer.right.decay_rank is {stated}, but {name} has {int(shape[0])} rows")
                l["mixer"]["right"]["decay_rank"] = int(shape[0])
        return dataclasses.replace(self, layers=layers)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "layers": copy.deepcopy(self.layers), "logit_scale": self.logit_scale,
                             "norm": {"eps": self.eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.bigram is not None:
            d["embedding"] = {"bigram": dict(self.bigram)}
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d

    # ------------------------------------------------------------------ model description
    def model_spec(self) -> ModelSpec:
        W = self.width
        norm = PartSpec("rmsnorm", {"size": W, "eps": self.eps, "tensor_name": ""})
        layers: List[LayerSpec] = []
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            if l["type"] == "mamba2":
                mixer = PartSpec("state_space_heads", {
                    "hidden_size": W, "num_heads": m["heads"], "head_dim": m["vdim"], "state": m["state"], "groups": m["groups"],
                    "conv": m["conv"], "norm_groups": m["norm_groups"], "eps": self.eps})
            else:
                a, b = m["left"], m["right"]
                rot = a["rot"]
                position = None
                if rot is not None and rot["dims"] > 0:
                    position = PartSpec("rotary", {"head_dim": a["dim"], "rotary_dim": rot["dims"], "theta": rot["base"],
                                                   "linear": rot["scaling"]["factor"] if rot["scaling"] else 1.0})
                left = PartSpec("sink_attention", {
                    "hidden_size": W, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"], "v_head_dim": a["vdim"],
                    "chunk": a["mask"]["size"] if a["mask"] else 0, "scale": a["scale"], "bias": True, "out_bias": False,
                    "qk_norm_weight": True, "eps": self.eps, "sink": True, "v_from_k": True, "rotary_pairs": "interleaved",
                    "position": position})
                if b.get("decay_rank") is None:
                    raise ConfigError(f"config: layers[{i}].mixer.right: the decay projection's rank is neither stated (decay_rank) "
                                      f"nor known from the shape of l{i}.mix.right.a1")
                right = PartSpec("gated_linear_attention", {"hidden_size": W, "num_heads": b["heads"], "head_dim": b["dim"],
                                                            "v_head_dim": b["vdim"], "tau": b["tau"], "eps": self.eps,
                                                            "decay_rank": b["decay_rank"]})
                mixer = PartSpec("parallel", {"hidden_size": W, "branches": (
                    {"prefix": "left.", "mixer": left, "scale": 0.5}, {"prefix": "right.", "mixer": right, "scale": 0.5}),
                    "branch_norm": {"eps": self.eps, "names": ("left.out", "right.out")}})
            parts = {"mixer_norm": norm, "mixer": mixer}
            prefixes = {"mixer_norm": "norm1", "mixer": "mix."}
            f = l["mlp"]
            if f is not None:
                if f["kind"] == "dense":
                    ff = PartSpec("gated_gelu", {"hidden_size": W, "intermediate_size": f["ff"], "tensor_names": ("gate", "up", "down")})
                else:
                    r, shared = f["router"], f["shared"]
                    groups = r.get("groups") or {"count": 1, "keep": 1}
                    ff = PartSpec("moe", {"hidden_size": W, "num_experts": r["experts"], "top": r["top"], "expert_size": f["expert"]["ff"],
                                          "router": "scores", "unit": "gelu", "identity": r["identity"], "groups": groups["count"],
                                          "keep": groups["keep"], "shared_size": shared["ff"] if shared else 0, "shared_gate": bool(shared)})
                parts.update({"feed_forward_norm": norm, "feed_forward": ff})
                prefixes.update({"feed_forward_norm": "norm2", "feed_forward": "mlp."})
            layers.append(LayerSpec(prefix=f"l{i}.", block="prenorm_scaled", parts=parts, part_prefixes=prefixes,
                                    block_params={"residual_scale": self.residual_mult}))
        if self.bigram is not None:
            embedding = PartSpec("hashed_pair_embedding", {"vocab_size": self.vocab, "hidden_size": W, "tensor_name": "embed",
                                                           "pair_tensor_name": "bigram", **self.bigram})
        else:
            embedding = PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": W, "tensor_name": "embed"})
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=W, vocab_size=self.vocab, layers=layers,
            plan=[PlanEntry(i) for i in range(len(layers))], embedding=embedding, final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": True, "scale": self.logit_scale}),
            weight_prefixes=[""], embedding_prefix="", final_norm_prefix="final.norm", head_prefix="lm_head.",
            stop_token_ids=list(self.eos_token_ids), max_position=self.max_position_embeddings)
        spec.validate()
        return spec
