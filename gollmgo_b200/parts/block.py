"""Arrangements of a layer's parts.  "pre_norm" is the reference's run_layer
(kernels/gollmgo_model.cu:551-792): x += mixer(norm(x)); x += ffn(norm(x)), the
residual stream x in float32.

Each residual add is fused into the norm that follows it, so a block takes the
residual and a pending delta (what the previous block still owes the residual)
and returns its own pending delta.

"post_norm": x += s1 * norm(mixer(x)); x += s2 * norm(ffn(x)): the norm on the
sublayer's output, an optional per-channel scale, the sublayers reading x itself.

"sandwich": x += norm_b(gate(h) * mixer(h)), h = norm_a(x), and the same for the
feed-forward: a norm before and after every sublayer, and between them an optional
learned gate sigmoid(W h + b) per channel on the sublayer's result.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import WeightSpec
from .linear import NextNorm, NormedRows, linear
from .registry import register_block


class PreNormBlock:
    """forward(resid, delta, ...) -> the delta this block still owes the residual.

    In steps of a few tokens the two residual adds and norms move into the products around
    them where the parts offer it (the optional protocol of parts/linear.py: a part's
    ``takes_normed_rows(T)`` / ``fuses_next_norm(T)`` and a norm's ``rms_weight_eps()``):
    the mixer's last product adds to the residual and prepares the second norm's input for
    the feed-forward's first product, and the feed-forward's last product does the same for
    the first norm of the block that runs next, if that block ``takes_normed_rows`` too.  The
    delta handed on is then a NormedRows: the add is done and the norm's input is ready."""

    chains_norms = True          # forward takes next_block= and may return or receive NormedRows

    def __init__(self, layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.ctx = ctx
        self.hidden = mixer_norm.size
        ctx.workspace.reserve("normed", ctx.max_tokens * self.hidden, ctx.act_dtype)
        ctx.workspace.reserve("norm_partials", -(-self.hidden // 16) * 16, torch.float32)

    @staticmethod
    def _can(part, what, T):
        f = getattr(part, what, None)
        return bool(f and f(T))

    def takes_normed_rows(self, T):
        """Whether the block before may hand this one its first norm's input as NormedRows."""
        return hasattr(self.mixer_norm, "rms_weight_eps") and self._can(self.mixer, "takes_normed_rows", T)

    def _next_norm(self, norm, resid, T):
        w, eps = norm.rms_weight_eps()
        ws = self.ctx.workspace
        return NextNorm(resid, w, eps, ws.get("normed", T, self.hidden),
                        ws.get("norm_partials", -(-self.hidden // 16), 16))

    def forward(self, resid, delta, batch, cache, writes_cache=True, next_block=None):
        T = resid.shape[0]
        if isinstance(delta, NormedRows):
            h = delta                                   # the block before did the add and prepared the norm
        else:
            h = self.ctx.workspace.get("normed", T, self.hidden)
            self.mixer_norm.add_norm(resid, delta, h)
        if (hasattr(self.ffn_norm, "rms_weight_eps") and self._can(self.mixer, "fuses_next_norm", T)
                and self._can(self.feed_forward, "takes_normed_rows", T)):
            h = self.mixer.forward(h, batch, cache, writes_cache, then=self._next_norm(self.ffn_norm, resid, T))
        else:
            a = self.mixer.forward(h, batch, cache, writes_cache)
            h = self.ctx.workspace.get("normed", T, self.hidden)
            self.ffn_norm.add_norm(resid, a, h)
        nxt = next_block
        if (nxt is not None and getattr(nxt, "chains_norms", False) and nxt.takes_normed_rows(T)
                and nxt.hidden == self.hidden and self._can(self.feed_forward, "fuses_next_norm", T)):
            return self.feed_forward.forward(h, batch, then=self._next_norm(nxt.mixer_norm, resid, T))
        return self.feed_forward.forward(h, batch)


class ResidualRows:
    """What a block hands on when it has already added everything to the residual stream:
    ``rows`` is the stream rounded to the activation type (the stream itself in the float32
    mode), ready for a sublayer that reads the stream."""

    def __init__(self, rows):
        self.rows = rows


class PostNormBlock:
    """x += s1 * norm1(mixer(x)); x += s2 * norm2(ff(x)): the sublayers read the residual stream
    itself and the norms sit on what they return.  s1, s2 are per-channel scales ("layer scale":
    tensors ``scale_names`` under the layer's block prefix) or absent.  A layer without a
    feed-forward stops after the first line.  params: layer_scale (bool), scale_names (two names).

    Norm, scale, the add to the float32 stream and the stream's rounding for the next sublayer are
    one kernel (csrc/layernorm.cu); any norm that offers ``norm_scale_add`` can be used."""

    def __init__(self, layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.ctx = ctx
        self.hidden = mixer_norm.size
        p = layer_spec.block
        self.layer_scale = bool(p.get("layer_scale", False))
        self.scale_names = tuple(p.get("scale_names", ("ls1", "ls2")))
        self.scale1 = self.scale2 = None
        for n in (mixer_norm, ffn_norm):
            if n is not None and not hasattr(n, "norm_scale_add"):
                raise TypeError(f"norm {type(n).__name__} cannot sit on a sublayer's output (no norm_scale_add)")
        if feed_forward is not None and ffn_norm is None:
            raise ValueError("a post-norm block with a feed-forward needs its norm")
        if ctx.act_dtype != torch.float32:
            ctx.workspace.reserve("stream_rows", ctx.max_tokens * self.hidden, ctx.act_dtype)

    def weights(self):
        if not self.layer_scale:
            return {}
        names = self.scale_names if self.feed_forward is not None else self.scale_names[:1]
        return {n: WeightSpec((self.hidden,)) for n in names}

    def load(self, get):
        if self.layer_scale:
            self.scale1 = get(self.scale_names[0]).to(torch.float32).contiguous()
            if self.feed_forward is not None:
                self.scale2 = get(self.scale_names[1]).to(torch.float32).contiguous()

    def forward(self, resid, delta, batch, cache, writes_cache=True):
        T = resid.shape[0]
        f32 = self.ctx.act_dtype == torch.float32
        if isinstance(delta, ResidualRows):
            h = delta.rows
        else:
            if delta is not None:
                raise ValueError("a post-norm block cannot take a pending delta from the block before it")
            h = resid
            if not f32:
                h = self.ctx.workspace.get("stream_rows", T, self.hidden)
                ops.cast_rows(resid, h)
        nxt = resid if f32 else h                    # where the stream's rounded copy goes: over the rows just read
        y = self.mixer.forward(h, batch, cache, writes_cache)
        self.mixer_norm.norm_scale_add(resid, y, self.scale1, None if f32 else nxt)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(nxt, batch)
            self.ffn_norm.norm_scale_add(resid, y, self.scale2, None if f32 else nxt)
        return ResidualRows(nxt)


class ParallelBlock:
    """x += mult * (mixer(h) + ff(h)) with h = norm(x): one norm, and both sublayers read its
    output.  A layer without a feed-forward adds the mixer alone.  params: residual_mult (default 1).
    The sum of the sublayers and the add to the stream are float32 (one kernel); a mixer that leaves
    the bias of its output projection in ``deferred_bias`` has it added by the same kernel."""

    def __init__(self, layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx):
        self.mixer, self.feed_forward, self.mixer_norm, self.ctx = mixer, feed_forward, mixer_norm, ctx
        if ffn_norm is not None:
            raise ValueError("a parallel block has one norm; the feed-forward reads the mixer's")
        self.hidden = mixer_norm.size
        self.mult = float(layer_spec.block.get("residual_mult", 1.0))
        ctx.workspace.reserve("normed", ctx.max_tokens * self.hidden, ctx.act_dtype)

    def forward(self, resid, delta, batch, cache, writes_cache=True):
        T = resid.shape[0]
        if isinstance(delta, ResidualRows):
            delta = None                                  # the block before has added everything itself
        elif delta is not None and not torch.is_tensor(delta):
            raise ValueError("a parallel block cannot take the norm's input from the block before it")
        h = self.ctx.workspace.get("normed", T, self.hidden)
        self.mixer_norm.add_norm(resid, delta, h)
        a = self.mixer.forward(h, batch, cache, writes_cache)
        f = self.feed_forward.forward(h, batch) if self.feed_forward is not None else None
        ops.scaled_add(resid, a, f, self.mult, getattr(self.mixer, "deferred_bias", None))
        return None


class SandwichBlock:
    """x += norm1b(g1 * mixer(h)) with h = norm1(x) and g1 = sigmoid(W1 h + b1); then the same with norm2, the
    feed-forward, W2, b2 and norm2b.  norm1 and norm2 are the layer's two norms; the norms on the results (RMS norms
    with a weight) and the gates are the block's own tensors, under the layer's block prefix.  A layer without a
    feed-forward stops after the first line.  params: eps, gated (bool: the gates exist), post_names (names of the
    two result norms), gate_names (names of the two gate weights; a bias is that name + ".b").

    The gate's product reads the same rows as the sublayer.  Gate, norm and the add to the float32 stream are one
    kernel (csrc/layernorm.cu), which also adds a bias that the sublayer's last product left in ``deferred_bias``."""

    def __init__(self, layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.ctx = ctx
        self.hidden = mixer_norm.size
        p = layer_spec.block
        self.eps = float(p["eps"])
        self.gated = bool(p.get("gated", True))
        self.post_names = tuple(p.get("post_names", ("norm1b", "norm2b")))
        self.gate_names = tuple(p.get("gate_names", ("rg1", "rg2")))
        if feed_forward is not None and ffn_norm is None:
            raise ValueError("a sandwich block with a feed-forward needs the norm before it")
        ctx.workspace.reserve("normed", ctx.max_tokens * self.hidden, ctx.act_dtype)
        if self.gated:
            ctx.workspace.reserve("resid_gate", ctx.max_tokens * self.hidden, ctx.act_dtype)
        self.post_w = [None, None]
        self.gate_w = [None, None]
        self.gate_b = [None, None]

    def _count(self):
        return 2 if self.feed_forward is not None else 1

    def weights(self):
        w = {}
        for i in range(self._count()):
            w[self.post_names[i]] = WeightSpec((self.hidden,))
            if self.gated:
                w[self.gate_names[i]] = WeightSpec((self.hidden, self.hidden))
                w[self.gate_names[i] + ".b"] = WeightSpec((self.hidden,), init="normal")
        return w

    def load(self, get):
        for i in range(self._count()):
            self.post_w[i] = get(self.post_names[i]).to(torch.float32).contiguous()
            if self.gated:
                self.gate_w[i] = get(self.gate_names[i]).contiguous()
                self.gate_b[i] = get(self.gate_names[i] + ".b").to(torch.float32).contiguous()

    def _join(self, i, resid, h, y, part):
        g = None
        if self.gated:
            g = linear(h, self.gate_w[i], self.ctx.workspace.get("resid_gate", h.shape[0], self.hidden))
        ops.gate_norm_add(resid, y, getattr(part, "deferred_bias", None), g, self.gate_b[i], self.post_w[i], self.eps)

    def forward(self, resid, delta, batch, cache, writes_cache=True):
        T = resid.shape[0]
        if isinstance(delta, ResidualRows):
            delta = None
        elif delta is not None and not torch.is_tensor(delta):
            raise ValueError("a sandwich block cannot take the norm's input from the block before it")
        h = self.ctx.workspace.get("normed", T, self.hidden)
        self.mixer_norm.add_norm(resid, delta, h)
        self._join(0, resid, h, self.mixer.forward(h, batch, cache, writes_cache), self.mixer)
        if self.feed_forward is not None:
            self.ffn_norm.add_norm(resid, None, h)
            self._join(1, resid, h, self.feed_forward.forward(h, batch), self.feed_forward)
        return None


register_block("pre_norm", PreNormBlock)
register_block("sandwich", SandwichBlock)
register_block("parallel", ParallelBlock)
register_block("post_norm", PostNormBlock)
