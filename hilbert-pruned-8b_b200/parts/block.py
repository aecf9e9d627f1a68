"""The arrangement of the parts of a layer.

A block is built from a ``LayerSpec``: it declares the roles it fills (``ROLES``: role name
-> the registry the part in that role comes from), builds them, and runs them in its order.
What the model needs of a block: ``named_parts()`` for the weight table, ``cache_need()``
and ``state_need()`` for the cache, and ``forward``.

``prenorm``: ``x += mixer(norm_a(x)); x += feed_forward(norm_b(x))`` with the residual
stream ``x`` in 32-bit (cleanroom-transformer/src/cpu_backend.c:237-252, cuda_backend.cu:628).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, TOKEN_FILTERS, CacheNeed, Registry, StateNeed


class Block:
    """Base of the arrangements: builds the parts that ``ROLES`` names from the layer's spec."""

    ROLES: Dict[str, Registry] = {}
    OPTIONAL: Tuple[str, ...] = ()      # roles a layer may leave empty

    def __init__(self, layer_spec, ctx):
        self.spec = layer_spec
        self.ctx = ctx
        extra = sorted(set(layer_spec.parts) - set(self.ROLES))
        if extra:
            raise ValueError(f"block {layer_spec.block!r} has no role for the parts {extra} of layer "
                             f"{layer_spec.prefix!r} (its roles: {', '.join(self.ROLES)})")
        self.parts = {role: registry.build(layer_spec.part(role), ctx) for role, registry in self.ROLES.items()
                      if role not in self.OPTIONAL or role in layer_spec.parts}
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in self.parts.values())

    def named_parts(self) -> List[Tuple[str, object]]:
        """(name prefix below the layer's prefix, part) for every part that may own weights."""
        return [(self.spec.part_prefix(role), part) for role, part in self.parts.items()]

    # the cache belongs to the part that mixes tokens, if the block has one
    def cache_need(self) -> Optional[CacheNeed]:
        mixer = self.parts.get("mixer")
        return mixer.cache_need() if mixer is not None else None

    def state_need(self) -> Optional[StateNeed]:
        mixer = self.parts.get("mixer")
        return mixer.state_need() if mixer is not None else None

    # A block with ``folds_norms = True`` takes two more keyword arguments and returns a value, by
    # which norms at the seam between two blocks are folded into the products around them (see
    # ``parts.base.Mixer``): ``prepared`` is what the block in front returned (None: nothing
    # prepared, the block runs its first norm), ``prepare_next`` what the next block's
    # ``fold_request`` said (None: nobody asks).  Other blocks are called without them.
    folds_norms = False

    def fold_request(self, step):
        """What the block in front has to prepare so that this block need not run its first
        norm (``Norm.fold_request`` of that norm, on the buffer this block reads), or None."""
        return None

    def forward(self, x, step, cache, state, append: bool):
        raise NotImplementedError


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    ROLES = {"mixer_norm": NORMS, "mixer": MIXERS, "feed_forward_norm": NORMS, "feed_forward": FEED_FORWARDS}

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        self.mixer_norm, self.mixer = self.parts["mixer_norm"], self.parts["mixer"]
        self.feed_forward_norm, self.feed_forward = self.parts["feed_forward_norm"], self.parts["feed_forward"]

    folds_norms = True

    def _normed(self, step, size: int):
        """The buffer the norms write and the mixer and the feed-forward read."""
        return self.ctx.workspace.buffer("block.h", (self.ctx.max_step_tokens, size), self.ctx.dtype)[:step.num_tokens]

    def _may_fold(self, step, size: int) -> bool:
        ops = self.ctx.ops
        return ops is not None and hasattr(ops, "can_fold_norm") and ops.can_fold_norm(step.num_tokens, size, self.ctx.dtype)

    def fold_request(self, step):
        # the mixer must be able to apply the prepared norm's factor; the norm says how wide the residual stream is
        size = getattr(self.mixer_norm, "size", None)
        if not getattr(self.mixer, "folds_norms", False) or size is None or not self._may_fold(step, size):
            return None
        return self.mixer_norm.fold_request(self._normed(step, size))

    def forward(self, x, step, cache, state, append: bool, prepared=None, prepare_next=None):
        h = self._normed(step, x.shape[1])
        fold = self._may_fold(step, x.shape[1])
        mixer_folds, ff_folds = getattr(self.mixer, "folds_norms", False), getattr(self.feed_forward, "folds_norms", False)
        # x += mixer(norm(x)); the mixer's last product prepares the next norm if the feed-forward can use it
        if prepared is None:
            self.mixer_norm.forward(x, h)
        if mixer_folds:
            request = self.feed_forward_norm.fold_request(h) if fold and ff_folds else None
            prepared = self.mixer.forward(h, x, step, cache, state, append, prepared=prepared, prepare=request)
        else:
            self.mixer.forward(h, x, step, cache, state, append)
            prepared = None
        # x += feed_forward(norm(x)); its last product prepares the next block's first norm if that block asked
        if prepared is None:
            self.feed_forward_norm.forward(x, h)
        if ff_folds:
            return self.feed_forward.forward(h, x, step, prepared=prepared, prepare=prepare_next if fold else None)
        self.feed_forward.forward(h, x, step)
        return None


@BLOCKS.register("prenorm_filtered")
class FilteredPreNormBlock(Block):
    """``x += mixer(filter(norm_a(x)))``, then, if the layer has a feed-forward,
    ``x += feed_forward(norm_b(x))``.  The filter (a short convolution over time) and the mixer may
    both keep per-sequence state: the block asks the cache for one area per sequence and gives each
    its share, the filter's first.  A filter that can apply the norm in front of it itself
    (``TokenFilter.fuses_norm``) gets the residual stream and the norm: one pass instead of two."""

    ROLES = {"mixer_norm": NORMS, "mixer_filter": TOKEN_FILTERS, "mixer": MIXERS, "feed_forward_norm": NORMS,
             "feed_forward": FEED_FORWARDS}
    OPTIONAL = ("mixer_filter", "feed_forward_norm", "feed_forward")

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        p = self.parts
        self.mixer_norm, self.mixer, self.filter = p["mixer_norm"], p["mixer"], p.get("mixer_filter")
        self.feed_forward_norm, self.feed_forward = p.get("feed_forward_norm"), p.get("feed_forward")
        if (self.feed_forward is None) != (self.feed_forward_norm is None):
            raise ValueError(f"layer {layer_spec.prefix!r}: a feed-forward and its norm come together")
        needs = [part.state_need() if part is not None else None for part in (self.filter, self.mixer)]
        for need in needs:
            if need is not None and (need.dtype != torch.float32 or len(need.shape) != 1):
                raise ValueError(f"layer {layer_spec.prefix!r}: per-sequence state is a flat run of 32-bit values here")
        self._state_sizes = [0 if need is None else int(need.shape[0]) for need in needs]
        self.fuse_norm_and_filter = True        # tests switch it off to compare the two ways

    def state_need(self) -> Optional[StateNeed]:
        total = sum(self._state_sizes)
        return StateNeed((total,), torch.float32) if total else None

    def _shares(self, state):
        """The filter's and the mixer's views of the block's state area ``[slots, total]``."""
        n_f, n_m = self._state_sizes
        return (state[:, :n_f] if n_f else None), (state[:, n_f:n_f + n_m] if n_m else None)

    def forward(self, x, step, cache, state, append: bool):
        ws, cap, T = self.ctx.workspace, self.ctx.max_step_tokens, step.num_tokens
        f_state, m_state = self._shares(state) if state is not None else (None, None)
        h = ws.buffer("block.h", (cap, x.shape[1]), self.ctx.dtype)[:T]
        if self.filter is None:
            self.mixer_norm.forward(x, h)
        elif self.fuse_norm_and_filter and self.filter.fuses_norm(self.mixer_norm):
            self.filter.forward(x, h, step, f_state, norm=self.mixer_norm)
        else:
            normed = ws.buffer("block.normed", (cap, x.shape[1]), torch.float32)[:T]      # the filter reads 32-bit values
            self.mixer_norm.forward(x, normed)
            self.filter.forward(normed, h, step, f_state)
        self.mixer.forward(h, x, step, cache, m_state, append)
        if self.feed_forward is not None:
            self.feed_forward_norm.forward(x, h)
            self.feed_forward.forward(h, x, step)
        return None


class NormAhead(tuple):
    """What a block's first norm needs so that the block in front can make its output while it adds its last sublayer's
    result to the stream: ``(weight, offset, eps, out)``, the form of ``Norm.fold_request``.  A type of its own, so that a
    block only honours requests of blocks that will understand what it answers with (``NORMED``)."""


NORMED = "normed"       # what such a block returns when it has written the next block's first norm output


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """Norms before AND after each sublayer: ``x += post_a(mixer(norm_a(x)))``, then, if the layer has a
    feed-forward, ``x += post_b(feed_forward(norm_b(x)))``.  A sublayer writes its result to a 32-bit buffer
    of the residual stream's shape (parts with ``can_overwrite`` write it, for others the buffer is zeroed and
    they add); the norm on the output adds it to the stream (``Norm.add_normed``) and, where it can, makes
    the next sublayer's input in the same pass: the feed-forward's inside the layer, and across the seam the
    next layer's first norm when that layer is of this kind too (``fold_request`` / ``prepare_next``)."""

    ROLES = {"mixer_norm": NORMS, "mixer": MIXERS, "mixer_post_norm": NORMS, "feed_forward_norm": NORMS,
             "feed_forward": FEED_FORWARDS, "feed_forward_post_norm": NORMS}
    OPTIONAL = ("feed_forward_norm", "feed_forward", "feed_forward_post_norm")
    folds_norms = True

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        p = self.parts
        self.mixer_norm, self.mixer, self.mixer_post = p["mixer_norm"], p["mixer"], p["mixer_post_norm"]
        self.ff_norm, self.ff, self.ff_post = p.get("feed_forward_norm"), p.get("feed_forward"), p.get("feed_forward_post_norm")
        if len({self.ff_norm is None, self.ff is None, self.ff_post is None}) != 1:
            raise ValueError(f"layer {layer_spec.prefix!r}: a feed-forward and its two norms come together")
        self.fuse_norms = True              # tests switch it off to run every norm as a kernel of its own

    @staticmethod
    def _run(part, y, args):
        if getattr(part, "can_overwrite", False):
            part.forward(*args, accumulate=False)
        else:
            y.zero_()
            part.forward(*args)

    def _h(self, step, size: int):
        return self.ctx.workspace.buffer("block.h", (self.ctx.max_step_tokens, size), self.ctx.dtype)[:step.num_tokens]

    def fold_request(self, step):
        size = getattr(self.mixer_norm, "size", None)
        if not self.fuse_norms or size is None:
            return None
        request = self.mixer_norm.fold_request(self._h(step, size))
        return NormAhead(request) if request is not None else None

    def forward(self, x, step, cache, state, append: bool, prepared=None, prepare_next=None):
        ws, cap, T = self.ctx.workspace, self.ctx.max_step_tokens, step.num_tokens
        h = self._h(step, x.shape[1])
        y = ws.buffer("block.branch", (cap, x.shape[1]), torch.float32)[:T]
        ahead = prepare_next if (self.fuse_norms and isinstance(prepare_next, NormAhead)) else None
        if prepared is not NORMED:
            self.mixer_norm.forward(x, h)
        self._run(self.mixer, y, (h, y, step, cache, state, append))
        if self.ff is None:
            return NORMED if self.mixer_post.add_normed(y, x, then=ahead) else None
        if not (self.fuse_norms and self.mixer_post.add_normed(y, x, then=self.ff_norm, then_out=h)):
            if not self.fuse_norms:
                self.mixer_post.add_normed(y, x)
            self.ff_norm.forward(x, h)
        self._run(self.ff, y, (h, y, step))
        return NORMED if self.ff_post.add_normed(y, x, then=ahead) else None


class StreamCopyAhead(tuple):
    """What a block whose sublayers read the residual stream itself asks of the block in front: ``(out,)``, the buffer
    that should hold the stream's rows in the products' dtype when the block in front is done."""


COPIED = "copied"       # what a block returns when it has left that copy


@BLOCKS.register("postnorm")
class PostNormBlock(Block):
    """Norms on the sublayers' OUTPUTS only: ``x += post_a(mixer(x))``, then, if the layer has a feed-forward,
    ``x += post_b(feed_forward(x))``.  The sublayers read the 32-bit stream ``x`` itself: in 32-bit mode directly, in
    bfloat16 mode through a rounded copy, which the norm in front leaves while it adds to the stream (``add_normed(...,
    copy=)``; only a stack's first block converts with a kernel of its own).  A sublayer writes its result to a 32-bit
    buffer (parts with ``can_overwrite`` write it, for others it is zeroed and they add).  A mixer that is a weighted sum
    of two branches (``forward_branches``) hands its two results to the norm, which sums them on the fly
    (``add_normed_sum``)."""

    ROLES = {"mixer": MIXERS, "mixer_post_norm": NORMS, "feed_forward": FEED_FORWARDS, "feed_forward_post_norm": NORMS}
    OPTIONAL = ("feed_forward", "feed_forward_post_norm")
    folds_norms = True

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        p = self.parts
        self.mixer, self.mixer_post = p["mixer"], p["mixer_post_norm"]
        self.ff, self.ff_post = p.get("feed_forward"), p.get("feed_forward_post_norm")
        if (self.ff is None) != (self.ff_post is None):
            raise ValueError(f"layer {layer_spec.prefix!r}: a feed-forward and the norm on its output come together")
        self.fuse_sum = True                # tests switch it off to run the weighted sum as a kernel of its own

    def _copy_buffer(self, step, size: int):
        return self.ctx.workspace.buffer("block.h", (self.ctx.max_step_tokens, size), self.ctx.dtype)[:step.num_tokens]

    def fold_request(self, step):
        size = getattr(self.mixer_post, "size", None)
        if self.ctx.dtype == torch.float32 or size is None:
            return None
        return StreamCopyAhead((self._copy_buffer(step, size),))

    def forward(self, x, step, cache, state, append: bool, prepared=None, prepare_next=None):
        ws, cap, T = self.ctx.workspace, self.ctx.max_step_tokens, step.num_tokens
        exact = self.ctx.dtype == torch.float32
        h = x if exact else self._copy_buffer(step, x.shape[1])
        if not exact and prepared is not COPIED:
            self.ctx.ops.convert(x, h)
        y = ws.buffer("block.branch", (cap, x.shape[1]), torch.float32)[:T]
        ahead = prepare_next[0] if isinstance(prepare_next, StreamCopyAhead) else None
        mixer_copy = None if exact else (h if self.ff is not None else ahead)
        if self.fuse_sum and hasattr(self.mixer, "forward_branches") and hasattr(self.mixer_post, "add_normed_sum"):
            (a, sa), (b, sb) = self.mixer.forward_branches(h, step, cache, state, append)
            self.mixer_post.add_normed_sum(a, sa, b, sb, x, copy=mixer_copy)
        else:
            SandwichBlock._run(self.mixer, y, (h, y, step, cache, state, append))
            self.mixer_post.add_normed(y, x, copy=mixer_copy)
        if self.ff is None:
            return COPIED if mixer_copy is not None else None
        SandwichBlock._run(self.ff, y, (h, y, step))
        self.ff_post.add_normed(y, x, copy=ahead)
        return COPIED if ahead is not None else None


@BLOCKS.register("prenorm_scaled")
class ScaledPreNormBlock(Block):
    """``x += m * mixer(norm_a(x))``, then, if the layer has a feed-forward, ``x += m * feed_forward(norm_b(x))``, with one
    fixed factor ``m`` (the layer's ``block_params["residual_scale"]``) on every sublayer's result.  A sublayer writes its
    result to a 32-bit buffer of the residual stream's shape (parts with ``can_overwrite`` write it, for others the buffer is
    zeroed and they add); one kernel adds ``m`` times that buffer to the stream and, in the same pass, makes the next
    norm's output from the values it still holds: the feed-forward's inside the layer, and across the seam the next layer's
    first norm when that layer asks for it (``fold_request`` / ``prepare_next``, the protocol of the sandwich block)."""

    ROLES = {"mixer_norm": NORMS, "mixer": MIXERS, "feed_forward_norm": NORMS, "feed_forward": FEED_FORWARDS}
    OPTIONAL = ("feed_forward_norm", "feed_forward")
    folds_norms = True

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        p = self.parts
        self.mixer_norm, self.mixer = p["mixer_norm"], p["mixer"]
        self.ff_norm, self.ff = p.get("feed_forward_norm"), p.get("feed_forward")
        if (self.ff is None) != (self.ff_norm is None):
            raise ValueError(f"layer {layer_spec.prefix!r}: a feed-forward and its norm come together")
        self.scale = float(layer_spec.block_params.get("residual_scale", 1.0))
        self.fuse_norms = True              # tests switch it off to run every norm as a kernel of its own

    def _h(self, step, size: int):
        return self.ctx.workspace.buffer("block.h", (self.ctx.max_step_tokens, size), self.ctx.dtype)[:step.num_tokens]

    def fold_request(self, step):
        size = getattr(self.mixer_norm, "size", None)
        if not self.fuse_norms or size is None:
            return None
        request = self.mixer_norm.fold_request(self._h(step, size))
        return NormAhead(request) if request is not None else None

    def _add(self, y, x, then) -> bool:
        """``x += scale * y``; ``then`` (weight, offset, eps, out) of the norm that reads ``x`` next, or None."""
        ops = self.ctx.ops
        if then is not None and tuple(then[3].shape) == tuple(x.shape):
            ops.scaled_add_norm(y, self.scale, x, then=(then[0], then[2], then[1]), then_out=then[3])
            return True
        ops.scaled_add_norm(y, self.scale, x)
        return False

    def forward(self, x, step, cache, state, append: bool, prepared=None, prepare_next=None):
        ws, cap, T = self.ctx.workspace, self.ctx.max_step_tokens, step.num_tokens
        h = self._h(step, x.shape[1])
        y = ws.buffer("block.branch", (cap, x.shape[1]), torch.float32)[:T]
        ahead = prepare_next if (self.fuse_norms and isinstance(prepare_next, NormAhead)) else None
        if prepared is not NORMED:
            self.mixer_norm.forward(x, h)
        SandwichBlock._run(self.mixer, y, (h, y, step, cache, state, append))
        if self.ff is None:
            return NORMED if self._add(y, x, ahead) else None
        request = self.ff_norm.fold_request(h) if self.fuse_norms else None
        if not self._add(y, x, request):
            self.ff_norm.forward(x, h)
        SandwichBlock._run(self.ff, y, (h, y, step))
        return NORMED if self._add(y, x, ahead) else None
