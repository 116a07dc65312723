"""Token shift: a mixer that reads, instead of its input h_t, a per-channel blend of it with the
previous token's,

    h'_t = h_t + (h_{t-1} - h_t) * mu,        h_{-1} = 0,

and hands that to the mixer it wraps.  The previous token's row (as it came in, before the blend)
is part of a request's state: a float32 row per request in its state slot, beside whatever the
wrapped mixer keeps.  Only the mixer reads the blend; whatever else reads h (a feed-forward in
a parallel block) reads it as it is.

params: hidden_size, inner (the wrapped mixer's PartSpec), inner_prefix (prefix of its tensors under
this mixer's prefix), name (local name of mu, [hidden_size]).
"""
from __future__ import annotations

import torch

from ..cache import FixedStateNeed
from ..csrc import ops
from ..weights import WeightSpec
from .registry import build_mixer, register_mixer


class TokenShift:
    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.inner = build_mixer(spec["inner"], ctx)
        self.inner_prefix = spec.get("inner_prefix") or ""
        self.name = spec.get("name") or "shift"
        self.mu = None
        ctx.workspace.reserve("shifted", ctx.max_tokens * self.hidden, ctx.act_dtype)

    def cache_need(self):
        return (FixedStateNeed((self.hidden,), "float32"), self.inner.cache_need())

    def query_tiles(self):
        return getattr(self.inner, "query_tiles", lambda: ())()

    def step_tags(self, facts):
        f = getattr(self.inner, "step_tags", None)
        return tuple(f(facts)) if f is not None else ()

    @property
    def deferred_bias(self):
        return getattr(self.inner, "deferred_bias", None)

    def weights(self):
        w = {self.name: WeightSpec((self.hidden,), init="normal")}
        w.update({self.inner_prefix + local: s for local, s in self.inner.weights().items()})
        return w

    def load(self, get):
        self.mu = get(self.name).to(torch.float32).contiguous()
        self.inner.load(lambda local: get(self.inner_prefix + local))

    def forward(self, x, batch, cache, writes_cache=True):
        prev, inner_cache = cache
        out = self.ctx.workspace.get("shifted", x.shape[0], self.hidden)
        ops.token_shift(x, self.mu, prev, batch.cu_q_lens, batch.context_lens, batch.state_slots, batch.num_seqs, out)
        return self.inner.forward(out, batch, inner_cache, writes_cache)


register_mixer("token_shift", TokenShift)
