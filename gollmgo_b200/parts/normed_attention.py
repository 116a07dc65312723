"""Attention with normed heads: grouped-query softmax attention over the paged cache in which

* every query and key head is divided by its root mean square and multiplied by a weight vector of the
  head's size (one for all query heads, one for all key heads) before the rotation,
* every value head is divided by its root mean square (no weight), and cached so,
* a query sees the keys of its own chunk only (``chunk``: the sequence is cut into runs of that many
  positions, counted from position 0) or of a sliding window (``window``) or all earlier keys,
* the softmax denominator has one more term exp(sink_h) per head, with no key and no value,
* the values may be blended with those the first such layer of the model made for the same token:
  v <- (1 - lam) v + lam v_first (``v_mix``: "first" stores its values for the step, "blend" reads them;
  the blended values are what is cached),
* head h's result is multiplied by sigmoid(Wg x)_h before the output projection.

One product makes [q | k | v | gates]; one kernel norms, rotates, blends and writes the cache
(csrc/head_norm.cu); the general attention kernels (csrc/attention.cu, float32 arithmetic) take the chunk
and the sink as arguments.  Norms, the blend, scores and weights are float32.

params: hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim, position (PartSpec), scale, eps,
qk_norm (bool), v_norm (bool), chunk, window, sink (bool), v_mix (None | "first" | "blend"), head_gate (bool),
names (dict: q, k, v, o, q_norm, k_norm, sink, vmix, gate), out_buffer.
"""
from __future__ import annotations

import torch

from ..cache import PagedKVNeed
from ..csrc import ops
from ..weights import WeightSpec
from .attention import ATTN_POLICY, TILES_GENERAL, TILES_MMA_X, Attention, context_tiles, decode_splits
from .linear import linear
from .registry import register_mixer

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink",
          "vmix": "vmix", "gate": "g"}


class NormedAttention(Attention):
    extras = True                # the kernels with all options (csrc/attention.cu: gg_attn_prefill_x, gg_attn_decode_x)

    def __init__(self, spec, ctx):
        params = dict(spec.params)
        names = dict(_NAMES, **(params.pop("names", None) or {}))
        params["names"] = (names["q"], names["k"], names["v"], names["o"])
        self.chunk = int(spec.get("chunk") or 0)          # (before the base class sizes its scratch by _splits)
        super().__init__(type(spec)(spec.kind, params), ctx)
        self.tensor_names = names
        self.eps = float(spec["eps"])
        self.qk_norm = bool(spec.get("qk_norm", True))
        self.v_norm = bool(spec.get("v_norm", True))
        self.chunk = int(spec.get("chunk") or 0)
        if self.chunk and self.window:
            raise ValueError("an attention layer is chunked or windowed, not both")
        self.has_sink = bool(spec.get("sink", True))
        self.v_mix = spec.get("v_mix") or None
        if self.v_mix not in (None, "first", "blend"):
            raise ValueError(f"v_mix {self.v_mix!r} is not known (known: first, blend)")
        self.head_gate = bool(spec.get("head_gate", True))
        a8 = lambda n: -(-n // 8) * 8
        self.gate_col = a8((self.nh + self.nkv) * self.d + self.nv * self.dv)
        self.qkv_width = self.gate_col + (a8(self.nh) if self.head_gate else 0)
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("qkv", T * self.qkv_width, ctx.act_dtype)
        if self.v_mix:
            ws.reserve("v_first", T * self.nv * self.dv, torch.float32)
        # bfloat16 with keys and values of 64 or 128: the mma.sync kernels, where they take this layer's options
        self._mma_x = (ctx.act_dtype == torch.bfloat16 and ctx.device.type == "cuda" and self.d in (64, 128)
                       and self.dv in (64, 128) and ATTN_POLICY != "general"
                       and (not (self.chunk or self.has_sink) or ops.attn_mma_x_chunk_sink()))
        self.q_w = self.k_w = self.sink = None
        self.lam = 0.0

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window, v_heads=self.nv, v_head_dim=self.dv)

    def query_tiles(self):
        return [TILES_GENERAL, TILES_MMA_X] if self._mma_x else [TILES_GENERAL]

    def _splits(self, n_dec, max_context):
        return decode_splits(n_dec, self._ctas_per_split, self.num_sms, self._cluster_cap,
                             context_tiles(max_context, self.chunk or self.window), self._tile_bytes)

    def weights(self):
        n = self.tensor_names
        w = {n["q"]: WeightSpec((self.nh * self.d, self.hidden)), n["k"]: WeightSpec((self.nkv * self.d, self.hidden)),
             n["v"]: WeightSpec((self.nv * self.dv, self.hidden)), n["o"]: WeightSpec((self.hidden, self.nh * self.dv))}
        if self.qk_norm:
            w[n["q_norm"]] = WeightSpec((self.d,))
            w[n["k_norm"]] = WeightSpec((self.d,))
        if self.has_sink:
            w[n["sink"]] = WeightSpec((self.nh,), init="normal")
        if self.v_mix:
            w[n["vmix"]] = WeightSpec((), init="fraction")      # the first layer holds one too and does not use it
        if self.head_gate:
            w[n["gate"]] = WeightSpec((self.nh, self.hidden))
        return w

    def load(self, get):
        n = self.tensor_names
        parts = [get(n["q"]), get(n["k"]), get(n["v"])]
        gate = get(n["gate"]) if self.head_gate else None
        dt = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        w = torch.zeros(self.qkv_width, self.hidden, dtype=dt, device=parts[0].device)
        rows = torch.cat([p.to(dt) for p in parts], dim=0)
        w[:rows.shape[0]] = rows
        if gate is not None:
            w[self.gate_col:self.gate_col + self.nh] = gate.to(dt)
        self.w_qkv = w.contiguous()
        self.w_o = get(n["o"]).contiguous()
        if self.qk_norm:
            self.q_w = get(n["q_norm"]).float().contiguous()
            self.k_w = get(n["k_norm"]).float().contiguous()
        if self.has_sink:
            self.sink = get(n["sink"]).float().contiguous()
        if self.v_mix:
            lam = get(n["vmix"])
            self.lam = float(lam.float().reshape(-1)[0].item()) if self.v_mix == "blend" else 0.0

    def takes_normed_rows(self, num_tokens):
        return False

    def fuses_next_norm(self, num_tokens):
        return False

    def forward(self, x, batch, cache, writes_cache=True, then=None):
        T, ws = x.shape[0], self.ctx.workspace
        kc, vc, group = cache
        proj = linear(x, self.w_qkv, ws.get("qkv", T, self.qkv_width))
        if hasattr(self.position, "apply"):
            raise TypeError("a position encoding that rewrites q and k itself cannot be used with normed heads")
        v_first = ws.get("v_first", T, self.nv * self.dv) if self.v_mix else None
        ops.qkv_norm_rope_write(proj, batch.positions, batch.slot_mapping[group], self.position.rope_table(),
                                float(getattr(self.position, "magnitude", 1.0)), self.q_w, self.k_w, self.eps, self.v_norm,
                                v_first, {None: 0, "first": 1, "blend": 2}[self.v_mix], self.lam, kc, vc, self.nh,
                                self.nkv, self.d, self.nv, self.dv, self.ctx.page_size, self.position.interleaved,
                                writes_cache)
        out = ws.get("attn_out", T, self.nh * self.dv)
        window, bt = int(self.window or 0), batch.block_tables[group]
        more = dict(chunk=self.chunk, sink=self.sink)
        if batch.num_portions:
            if TILES_GENERAL not in batch.tiles:
                raise RuntimeError("the step's batch was built without the index lists this mixer declares in "
                                   "query_tiles(): give them to the BatchBuilder (query_tiles=...)")
            t16, t64 = batch.tiles[TILES_GENERAL], batch.tiles.get(TILES_MMA_X) if self._mma_x else None
            ops.attn_prefill_x(proj, self.qkv_width, kc, vc, bt, batch.bt_stride, batch.cu_q_lens, batch.context_lens,
                               t16.seq, t16.q0, t16.count, out, self.nh, self.nkv, self.d, self.dv, 1,
                               self.ctx.page_size, window, self.scale, 0.0,
                               t64.seq if t64 else None, t64.q0 if t64 else None, t64.count if t64 else 0,
                               allow_mma=t64 is not None, **more)
        if batch.num_decode:
            n = batch.num_decode
            facts = getattr(batch, "facts", None)
            longest = facts.max_context if facts is not None else max(s + q for s, q in zip(batch.q_starts, batch.q_lens))
            splits = self._splits(n, longest)
            ops.attn_decode_x(proj, self.qkv_width, kc, vc, bt, batch.bt_stride, batch.cu_q_lens, batch.context_lens,
                              batch.dec_seqs, n, splits, ws.get("attn_part_o", 1, n * self.nh * splits * self.dv),
                              ws.get("attn_part_ml", 1, n * self.nh * splits * 2), out, self.nh, self.nkv, self.d,
                              self.dv, 1, self.ctx.page_size, window, self.scale, 0.0, allow_mma=self._mma_x, **more)
        if self.head_gate:
            ops.head_gate(out, proj, self.gate_col, self.nh)
        return linear(out, self.w_o, ws.get(self.out_buffer, T, self.hidden), then)


register_mixer("normed_attention", NormedAttention)
