"""Several mixers side by side: all read the same input, the result is the weighted sum of
theirs, ``sum_i scale_i mixer_i(h)``.

``branches``: a list of ``{"prefix", "mixer" (a PartSpec), "scale"}``; a branch's tensors are named
``<prefix><its own names>`` below this part's prefix.  Every branch may keep keys and values
(the cache then holds a group per need, and each branch gets its own view) and fixed-size state
(one flat run of 32-bit values per sequence, shared out in the branches' order).  Each branch
writes its result to a 32-bit buffer of its own; one small kernel forms the weighted sum.

``branch_norm`` (a dict with ``eps`` and ``names``, one tensor name per branch): each branch's result is first divided by its
root mean square over the model width and multiplied by a weight of its own (plain, not one-plus), so the mixer's result is
``sum_i scale_i * rmsnorm_i(mixer_i(h))``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import MIXERS, Mixer, ParamSpec, StateNeed


@MIXERS.register("parallel")
class ParallelMixers(Mixer):
    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden = int(spec.params["hidden_size"])
        branches = spec.params["branches"]
        if len(branches) != 2:
            raise ValueError("parallel: two branches are built")
        self.prefixes = [str(b["prefix"]) for b in branches]
        self.scales = [float(b.get("scale", 1.0)) for b in branches]
        self.mixers = [MIXERS.build(b["mixer"], ctx) for b in branches]
        self.graph_safe = all(getattr(m, "graph_safe", True) for m in self.mixers)
        needs = [m.cache_need() for m in self.mixers]
        self._cache_counts = [0 if n is None else (len(n) if isinstance(n, (tuple, list)) else 1) for n in needs]
        self._cache_tuple = [isinstance(n, (tuple, list)) for n in needs]
        self._needs = [x for n in needs if n is not None for x in (n if isinstance(n, (tuple, list)) else (n,))]
        states = [m.state_need() for m in self.mixers]
        for s in states:
            if s is not None and (s.dtype != torch.float32 or len(s.shape) != 1):
                raise ValueError("parallel: per-sequence state is a flat run of 32-bit values here")
        self._state_sizes = [0 if s is None else int(s.shape[0]) for s in states]
        norm = spec.params.get("branch_norm")
        self.norm_eps = float(norm["eps"]) if norm else None
        self.norm_names = [str(n) for n in norm["names"]] if norm else []
        if norm and len(self.norm_names) != len(branches):
            raise ValueError("parallel: one norm weight per branch")
        self.norm_weights = None

    def params(self) -> List[ParamSpec]:
        out = []
        for prefix, m in zip(self.prefixes, self.mixers):
            for p in m.params():
                out.append(ParamSpec(prefix + p.name, p.shape, p.kind, p.init, p.absolute, p.optional))
        out += [ParamSpec(n, (self.hidden,), kind="vector", init="ones") for n in self.norm_names]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, m in zip(self.prefixes, self.mixers):
            m.bind({p.name: tensors[prefix + p.name] for p in m.params() if prefix + p.name in tensors})
        if self.norm_names:
            # the branch's share of the sum is part of its norm weight
            self.norm_weights = [tensors[n].reshape(-1).to(torch.float32).mul(s).contiguous() for n, s in zip(self.norm_names, self.scales)]

    def weight_bytes(self) -> int:
        return sum(m.weight_bytes() for m in self.mixers)

    def cache_need(self):
        if not self._needs:
            return None
        return self._needs[0] if len(self._needs) == 1 else tuple(self._needs)

    def state_need(self) -> Optional[StateNeed]:
        total = sum(self._state_sizes)
        return StateNeed((total,), torch.float32) if total else None

    def forward_branches(self, h, step, cache, state, append: bool):
        """Runs the branches and returns ``[(result, scale), (result, scale)]`` (32-bit buffers of the residual stream's
        shape) for a caller that forms the weighted sum itself, in a kernel that reads it anyway."""
        if self.norm_weights is not None:
            raise ValueError("parallel: branches with norms of their own are summed by the mixer itself")
        return list(zip(self._run_branches(h, step, cache, state, append), self.scales))

    def forward(self, h, residual, step, cache, state, append: bool, accumulate: bool = True):
        ops = self.ctx.ops
        outs = self._run_branches(h, step, cache, state, append)
        if self.norm_weights is not None:
            ops.normed_sum(outs[0], self.norm_weights[0], outs[1], self.norm_weights[1], self.norm_eps, residual, accumulate=accumulate)
        elif accumulate:
            # residual += s0 a + s1 b: the sum first, in the first branch's buffer, then added
            ops.scaled_sum(outs[0], self.scales[0], outs[1], self.scales[1], outs[0])
            ops.scaled_sum(residual, 1.0, outs[0], 1.0, residual)
        else:
            ops.scaled_sum(outs[0], self.scales[0], outs[1], self.scales[1], residual)

    def _run_branches(self, h, step, cache, state, append: bool):
        ws, T, cap = self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        views = [] if cache is None else (list(cache) if isinstance(cache, (tuple, list)) else [cache])
        outs, at_c, at_s = [], 0, 0
        for i, m in enumerate(self.mixers):
            n = self._cache_counts[i]
            mine = None if n == 0 else (tuple(views[at_c: at_c + n]) if self._cache_tuple[i] else views[at_c])
            at_c += n
            size = self._state_sizes[i]
            st = state[:, at_s: at_s + size] if size else None
            at_s += size
            out = ws.buffer(f"parallel.branch{i}", (cap, self.hidden), torch.float32)[:T]
            if getattr(m, "can_overwrite", False):
                m.forward(h, out, step, mine, st, append, accumulate=False)
            else:
                out.zero_()
                m.forward(h, out, step, mine, st, append)
            outs.append(out)
        return outs
