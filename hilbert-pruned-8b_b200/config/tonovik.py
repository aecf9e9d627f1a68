"""Typed configuration of the Tonovik decoder: a stack whose sublayers read the residual stream itself and
whose layer norms (weight and bias) sit on the sublayers' outputs, ``x += norm(sublayer(x))``, with two kinds
of mixer: two mixers side by side (a softmax attention over a sliding window with biases, a weighted norm of
queries and keys per head, rotary positions and a gate per head; and a matrix memory with a fixed decay per
head, rotary positions, a norm per head and a silu gate), added with two weights; and an attention over one
small cached latent per token with YaRN-scaled rotary positions on a separate part of queries and keys.  The
feed-forward is SwiGLU or absent.  The head has a matrix of its own.

config.json keys (every size and every constant that may differ between models comes from here):
``architecture`` ("Tonovik"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and ``layers``: a list of
``{"type", "mixer", "mlp"}`` with ``type``

* "parallel": ``mixer`` = ``left {heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims}}``,
  ``right {heads, dim, vdim, decay [per head], rot {base, dims}}``, ``left_scale``, ``right_scale``;
* "latent_attention": ``mixer`` = ``heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims, scaling {factor,
  original, fast, slow} | absent}``;

and ``mlp`` null or ``{"kind": "dense", "ff"}``.  Tensor names: ``embed``, ``l<i>.norm1|norm2`` (bias: ``.b`` added),
``l<i>.mix.*`` (``left.*`` / ``right.*`` below it for the parallel mixer), ``l<i>.mlp.gate|up|down``, ``final.norm``,
``head``.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, PlanEntry


def _number(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _int(d: Any, key: str, where: str, least: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if not _number(v) or v != math.floor(v) or v < least or v > 1e9:
        raise ConfigError(f"config: missing or bad {where}{key}")
    return int(v)


def _float(d: Any, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if not _number(v) or not math.isfinite(v):
        raise ConfigError(f"config: missing or bad {where}{key}")
    return float(v)


def _rot(m: Any, where: str, most: int, scaling: bool) -> Dict[str, Any]:
    r = m.get("rot") if isinstance(m, dict) else None
    out: Dict[str, Any] = {"base": _float(r, "base", where + "rot."), "dims": _int(r, "dims", where + "rot.", least=0)}
    if out["dims"] % 2 or out["dims"] > most:
        raise ConfigError(f"config: {where}rot.dims must be even and at most {most}")
    if out["base"] <= 0.0:
        raise ConfigError(f"config: {where}rot.base must be positive")
    s = r.get("scaling")
    if s is not None:
        if not scaling:
            raise ConfigError(f"config: {where}rot.scaling is not part of this mixer")
        sw = where + "rot.scaling."
        out["scaling"] = {"factor": _float(s, "factor", sw), "original": _float(s, "original", sw), "fast": _float(s, "fast", sw),
                          "slow": _float(s, "slow", sw)}
        if min(out["scaling"].values()) <= 0.0:
            raise ConfigError(f"config: the numbers of {where}rot.scaling must be positive")
    return out


@dataclass(frozen=True)
class TonovikConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: List[Dict[str, Any]] = field(default_factory=list)       # the validated entries of config.json
    eos_token_ids: List[int] = field(default_factory=list)
    max_position_embeddings: Optional[int] = None

    architecture = "Tonovik"
    model_type = "tonovik"

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
    def from_dict(cls, root: Dict[str, Any]) -> "TonovikConfig":
        if not isinstance(root, dict):
            raise ConfigError("config: config.json is not an object")
        vocab, width = _int(root, "vocab", ""), _int(root, "width", "")
        eps = _float(root.get("norm"), "eps", "norm.")
        emb = root.get("embedding")
        scale = _float(emb, "scale", "embedding.") if emb is not None else 1.0
        raw = root.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config: layers must be a list with at least one entry")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or entry.get("type") not in ("parallel", "latent_attention"):
                raise ConfigError(f"config: {where}type must be parallel or latent_attention")
            m = entry.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config: missing {where}mixer")
            mw = where + "mixer."
            if entry["type"] == "parallel":
                a, b = m.get("left"), m.get("right")
                lw, rw = mw + "left.", mw + "right."
                left = {"heads": _int(a, "heads", lw), "kv_heads": _int(a, "kv_heads", lw), "dim": _int(a, "dim", lw),
                        "vdim": _int(a, "vdim", lw), "scale": _float(a, "scale", lw)}
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"config: {lw}heads is no multiple of kv_heads")
                left["mask"] = {"size": _int(a.get("mask"), "size", lw + "mask.")}
                left["rot"] = _rot(a, lw, left["dim"], scaling=False)
                right = {"heads": _int(b, "heads", rw), "dim": _int(b, "dim", rw), "vdim": _int(b, "vdim", rw)}
                decay = b.get("decay")
                if not isinstance(decay, list) or len(decay) != right["heads"] or not all(_number(x) and 0.0 <= x <= 1.0 for x in decay):
                    raise ConfigError(f"config: {rw}decay must give a number in [0, 1] per head")
                right["decay"] = [float(x) for x in decay]
                right["rot"] = _rot(b, rw, right["dim"], scaling=False)
                mixer = {"left": left, "right": right, "left_scale": _float(m, "left_scale", mw), "right_scale": _float(m, "right_scale", mw)}
            else:
                mixer = {"heads": _int(m, "heads", mw), "dim": _int(m, "dim", mw), "rot_dim": _int(m, "rot_dim", mw, least=0),
                         "vdim": _int(m, "vdim", mw), "kv_rank": _int(m, "kv_rank", mw), "scale": _float(m, "scale", mw)}
                mixer["rot"] = _rot(m, mw, mixer["rot_dim"], scaling=True)
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config: {where}mlp.kind must be dense (or mlp null)")
                mlp = {"kind": "dense", "ff": _int(mlp, "ff", where + "mlp.")}
            layers.append({"type": entry["type"], "mixer": mixer, "mlp": mlp})
        eos = root.get("eos_token_id")
        eos_ids = [int(eos)] if _number(eos) else [int(e) for e in eos if _number(e)] if isinstance(eos, list) else []
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config: eos_token_id {e} is outside the vocabulary")
        max_pos = root.get("max_position_embeddings")
        return cls(vocab=vocab, width=width, eps=eps, embedding_scale=scale, layers=layers, eos_token_ids=eos_ids,
                   max_position_embeddings=int(max_pos) if _number(max_pos) and max_pos >= 1 else None)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                             "layers": copy.deepcopy(self.layers), "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d

    # ------------------------------------------------------------------ model description
    @staticmethod
    def _rotary(head_dim: int, rot: Dict[str, Any]) -> Optional[PartSpec]:
        if not rot["dims"]:
            return None
        params = {"head_dim": head_dim, "rotary_dim": rot["dims"], "theta": rot["base"], "frequencies_in_64_bit": True}
        if rot.get("scaling") is not None:
            params["yarn"] = dict(rot["scaling"])
        return PartSpec("rotary", params)

    def model_spec(self) -> ModelSpec:
        W = self.width
        norm = PartSpec("layernorm", {"size": W, "eps": self.eps, "tensor_name": ""})
        layers: List[LayerSpec] = []
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            if l["type"] == "parallel":
                a, b = m["left"], m["right"]
                left = PartSpec("sink_attention", {
                    "hidden_size": W, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"], "v_head_dim": a["vdim"],
                    "window": a["mask"]["size"], "keep_first": 0, "scale": a["scale"], "bias": True, "out_bias": False,
                    "qk_norm_weight": True, "eps": self.eps, "head_gate": True, "talk": False, "v_mix": None,
                    "position": self._rotary(a["dim"], a["rot"])})
                right = PartSpec("decay_memory", {
                    "hidden_size": W, "num_heads": b["heads"], "head_dim": b["dim"], "v_head_dim": b["vdim"], "decay": tuple(b["decay"]),
                    "eps": self.eps, "activation": "none", "position": self._rotary(b["dim"], b["rot"]), "k_scale": float(b["dim"]) ** -0.5,
                    "norm": "heads", "norm_weight": False, "gate": "silu"})
                mixer = PartSpec("parallel", {"hidden_size": W, "branches": (
                    {"prefix": "left.", "mixer": left, "scale": m["left_scale"]},
                    {"prefix": "right.", "mixer": right, "scale": m["right_scale"]})})
            else:
                mixer = PartSpec("latent_attention", {
                    "hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "rotary_head_dim": m["rot_dim"], "v_head_dim": m["vdim"],
                    "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": self.eps, "head_gate": True,
                    "position": self._rotary(m["rot_dim"], m["rot"]) if m["rot_dim"] else None})
            parts = {"mixer": mixer, "mixer_post_norm": norm}
            prefixes = {"mixer": "mix.", "mixer_post_norm": "norm1"}
            if l["mlp"] is not None:
                parts.update({"feed_forward": PartSpec("swiglu", {"hidden_size": W, "intermediate_size": l["mlp"]["ff"],
                                                                  "tensor_names": ("gate", "up", "down")}),
                              "feed_forward_post_norm": norm})
                prefixes.update({"feed_forward": "mlp.", "feed_forward_post_norm": "norm2"})
            layers.append(LayerSpec(prefix=f"l{i}.", block="postnorm", parts=parts, part_prefixes=prefixes))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=W, vocab_size=self.vocab, layers=layers,
            plan=[PlanEntry(i) for i in range(len(layers))],
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": W, "tensor_name": "embed", "scale": self.embedding_scale}),
            final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": False, "tensor_name": "head"}),
            weight_prefixes=[""], embedding_prefix="", final_norm_prefix="final.norm", head_prefix="",
            stop_token_ids=list(self.eos_token_ids), max_position=self.max_position_embeddings)
        spec.validate()
        return spec
