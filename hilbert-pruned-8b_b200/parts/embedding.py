"""Token embedding and output head.

``x[t] = E[token[t]]`` widened to 32-bit, no scaling (cleanroom-transformer/src/cpu_backend.c:236)
unless the spec gives a ``scale``;
``logit[v] = dot(h, W[v])`` with ``W = E`` when the embeddings are tied, else ``lm_head.weight``,
which carries no decoder prefix (model.c:399-406).

``hashed_pair_embedding`` adds an embedding of the pair (previous token, token) to the token's own: row ``(previous *
mul_prev + token * mul_cur) mod buckets`` of a second table, whose last row (number ``buckets``) serves a sequence's first
token.  The previous token is per-sequence state (one int32), so that a sequence may be fed in any portions.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import EMBEDDINGS, HEADS, ParamSpec, Part, StateNeed


@EMBEDDINGS.register("embedding")
class TokenEmbedding(Part):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.scale = float(spec.get("scale", 1.0))            # multiplies every embedding (a tied head reads the table itself)
        self.tensor_name = spec.get("tensor_name", "weight")
        self.weight = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec(self.tensor_name, (self.vocab, self.hidden))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor_name].contiguous()

    def share(self, stored) -> None:
        """Reads the table from ``stored`` from now on (the same values in the layout a tied head
        keeps them in), so that one copy serves both; the row-major copy is let go."""
        self.weight = stored

    def forward(self, tokens, out) -> None:
        self.ctx.ops.embed(tokens, self.weight, out, self.scale)


@EMBEDDINGS.register("hashed_pair_embedding")
class HashedPairEmbedding(TokenEmbedding):
    # the model hands the step and the embedding's per-sequence state to forward()
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.buckets = int(spec.params["buckets"])
        self.mul_prev = int(spec.params["mul_prev"])
        self.mul_cur = int(spec.params["mul_cur"])
        if self.buckets < 1 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("hashed_pair_embedding: buckets must be positive and the multipliers not negative")
        self.pair_tensor_name = spec.get("pair_tensor_name", "pairs")
        self.pairs = None

    def params(self) -> List[ParamSpec]:
        return super().params() + [ParamSpec(self.pair_tensor_name, (self.buckets + 1, self.hidden))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        super().bind(tensors)
        self.pairs = tensors[self.pair_tensor_name].contiguous()

    def state_need(self) -> StateNeed:
        return StateNeed((1,), torch.int32)

    def forward(self, tokens, out, step=None, state=None) -> None:
        if step is None or state is None:
            raise ValueError("hashed_pair_embedding: the step and the sequences' state are needed (the previous token is state)")
        self.ctx.ops.embed_pair(step, self.weight, self.pairs, state, out, self.buckets, self.mul_prev, self.mul_cur, self.scale)


@HEADS.register("lm_head")
class LMHead(Part):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied = bool(spec.get("tied", False))
        self.tensor_name = spec.get("tensor_name", "weight")      # behind the head's prefix
        self.scale = float(spec.get("scale", 1.0))                # multiplies the logits
        self.weight = None

    def params(self) -> List[ParamSpec]:
        # a tied checkpoint may still carry a copy of the head; it is then not read
        return [ParamSpec(self.tensor_name, (self.vocab, self.hidden), absolute=True, optional=self.tied)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = self.ctx.ops.pack_weight(tensors[self.tensor_name].contiguous())

    def tie(self, embedding_weight: torch.Tensor):
        """The head reads the embedding table; returns the form it keeps it in (tiles, where the
        tensor-core product can read them), which the embedding can gather from as well."""
        self.weight = self.ctx.ops.pack_weight(embedding_weight)
        return self.weight

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, hn, logits) -> None:
        """``logits[n, vocab]`` (32-bit) from normalised rows ``hn[n, hidden]``."""
        self.ctx.ops.linear(hn, self.weight, logits)
        if self.scale != 1.0:
            self.ctx.ops.scaled_sum(logits, self.scale, logits, 0.0, logits)
