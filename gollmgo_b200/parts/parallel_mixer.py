"""Mixers side by side: every branch reads the same input, each branch's output is RMS-normed
over the model width with a weight of its own, and the result is ``coef`` times their sum
(half the sum of two branches by default).

A branch is any registered mixer; its tensors live under the branch's prefix, the weight of its
output norm under ``norm_name``.  What the branches need of the cache is handed on as one
tuple, in the order of the branches (a branch that needs several things contributes a tuple of
its own), and every branch gets its part of the cache entry's view.

With ``branch_norm=False`` the branches are not normed: the result is the sum of the branches'
outputs, each times its own factor (``scales``), and the mixer owns no tensors of its own.

params: hidden_size, eps, branches = tuple of (PartSpec, tensor prefix, norm_name), coef
(default 1 / number of branches), branch_norm (default True), scales (one factor per branch; with
branch_norm=False only).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import WeightSpec
from .registry import build_mixer, register_mixer


class ParallelMixer:
    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.eps = float(spec["eps"])
        branches = tuple(spec["branches"])
        if not (1 <= len(branches) <= 4):
            raise ValueError(f"{len(branches)} branches are outside 1..4")
        self.coef = float(spec.get("coef") or 1.0 / len(branches))
        self.branch_norm = bool(spec.get("branch_norm", True))
        self.scales = tuple(float(x) for x in (spec.get("scales") or (1.0,) * len(branches)))
        if len(self.scales) != len(branches):
            raise ValueError(f"{len(self.scales)} factors for {len(branches)} branches")
        self.prefixes = [b[1] for b in branches]
        self.norm_names = [b[2] for b in branches]
        self.mixers = []
        for i, (part, _, _) in enumerate(branches):
            params = dict(part.params)
            params["out_buffer"] = f"branch{i}_out"              # the branches' results are alive together
            self.mixers.append(build_mixer(type(part)(part.kind, params), ctx))
        self.norm_w = [None] * len(branches)
        ctx.workspace.reserve("mixer_out", ctx.max_tokens * self.hidden, ctx.act_dtype)

    def cache_need(self):
        return tuple(m.cache_need() for m in self.mixers)

    def query_tiles(self):
        need = []
        for m in self.mixers:
            for n in getattr(m, "query_tiles", lambda: ())():
                if n not in need:
                    need.append(n)
        return need

    def step_tags(self, facts):
        tags = []
        for m in self.mixers:
            f = getattr(m, "step_tags", None)
            if f is not None:
                tags.extend(f(facts))
        return tuple(tags)

    def weights(self):
        w = {}
        for m, p, n in zip(self.mixers, self.prefixes, self.norm_names):
            w.update({p + local: s for local, s in m.weights().items()})
            if self.branch_norm:
                w[n] = WeightSpec((self.hidden,))
        return w

    def load(self, get):
        for i, (m, p, n) in enumerate(zip(self.mixers, self.prefixes, self.norm_names)):
            m.load(lambda local, p=p: get(p + local))
            if self.branch_norm:
                self.norm_w[i] = get(n).to(torch.float32).contiguous()

    def forward(self, x, batch, cache, writes_cache=True):
        ys = [m.forward(x, batch, c, writes_cache) for m, c in zip(self.mixers, cache)]
        out = self.ctx.workspace.get("mixer_out", x.shape[0], self.hidden)
        if self.branch_norm:
            ops.rms_mix(ys, self.norm_w, self.coef, self.eps, out)
        else:
            ops.weighted_sum(ys, self.scales, out)
        return out


register_mixer("parallel", ParallelMixer)
