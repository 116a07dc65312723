"""Sigmoid attention over the paged cache: every visible key weighs sigmoid(score) on its own and
nothing is normalised over the keys,

    o_i = sum_j sigmoid(scale * q_i . k_j + rel[bucket(i - j), h] + pb_h) * k_j,

with the keys serving as values (there is no value projection, and the cache holds one tensor per
layer), grouped query heads, biases on q and k, a learned bias by distance, a sliding window that
keeps the first tokens of the sequence visible, and an output gate sigmoid(Wg x) on the concatenated
heads before the output projection.  No rotation: positions enter through the distance alone.

Distance buckets, for a table of R rows and ``bias_max`` = D: bucket(n) = n for n < R / 2, else
min(R - 1, R / 2 + floor(ln(n / (R / 2)) / ln(D / (R / 2)) * (R - R / 2))): one row per distance
nearby, rows at logarithmic steps further away, the last row from D on.  R is read from the
checkpoint's tensor.  The table of buckets (D + 1 entries) is made once on the host in float64.

One product makes [q | k | gate]; the general attention kernels (csrc/attention.cu) do the rest
in float32 arithmetic.

params: hidden_size, num_heads, num_kv_heads, head_dim, window (None: all keys), keep_first, scale,
bias_max, bias_rows (the table's rows where random weights are made: a checkpoint's shape decides),
names (q, k, gate, o, rel, pb), out_buffer.
"""
from __future__ import annotations

import math

import torch

from ..cache import PagedKVNeed
from ..csrc import ops
from ..weights import WeightSpec
from .attention import ATTN_POLICY, TILES_GENERAL, TILES_MMA_X, Attention
from .linear import linear
from .registry import register_mixer


def distance_buckets(rows: int, far: int) -> torch.Tensor:
    """bucket(n) for n = 0 .. far (int32); every distance beyond ``far`` has the bucket of ``far``."""
    half = rows // 2
    if far <= half or half < 1:
        raise ValueError(f"a distance table of {rows} rows needs bias_max above {half}, got {far}")
    out = []
    for n in range(far + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return torch.tensor(out, dtype=torch.int32)


class SigmoidAttention(Attention):
    bias = True                  # q and k have biases: the general path

    def __init__(self, spec, ctx):
        params = dict(spec.params)
        params.setdefault("position", type(spec)("none"))
        names = dict({"q": "q", "k": "k", "gate": "g", "o": "o", "rel": "rel", "pb": "pb"}, **(params.pop("names", None) or {}))
        params["names"] = (names["q"], names["k"], names["k"], names["o"])
        params["v_head_dim"] = params["head_dim"]
        super().__init__(type(spec)(spec.kind, params), ctx)
        self.tensor_names = names
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        self.bias_max = int(spec["bias_max"])
        self.bias_rows = int(spec.get("bias_rows") or 32)
        # bfloat16 with heads of 64 or 128 and a distance table that fits in shared memory: mma.sync kernels
        self._mma_x = (ctx.act_dtype == torch.bfloat16 and self.d in (64, 128) and ATTN_POLICY != "general"
                       and self.bias_max < ops.ATTN_MMA_X_MAX_DIST
                       and ctx.page_size & (ctx.page_size - 1) == 0)
        # the projection's columns: queries, keys (which are the values), then the output gate
        self.gate_col = (self.nh + self.nkv) * self.d
        self.qkv_width = -(-(self.gate_col + self.nh * self.d) // 8) * 8
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("qkv", T * self.qkv_width, ctx.act_dtype)
        ws.reserve("attn_sum", T * self.nh * self.d, torch.float32)
        self.rel = self.pb = self.buckets = None

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window, shared_kv=True, keep_first=self.keep_first)

    def query_tiles(self):
        return [TILES_GENERAL, TILES_MMA_X] if self._mma_x else [TILES_GENERAL]

    def weights(self):
        n = self.tensor_names
        return {n["q"]: WeightSpec((self.nh * self.d, self.hidden)), n["q"] + ".b": WeightSpec((self.nh * self.d,), init="normal"),
                n["k"]: WeightSpec((self.nkv * self.d, self.hidden)), n["k"] + ".b": WeightSpec((self.nkv * self.d,), init="normal"),
                n["gate"]: WeightSpec((self.nh * self.d, self.hidden)),
                n["o"]: WeightSpec((self.hidden, self.nh * self.d)),
                n["rel"]: WeightSpec((self.bias_rows, self.nh), init="normal", free_dims=(0,)),
                n["pb"]: WeightSpec((self.nh,), init="normal")}

    def load(self, get):
        n = self.tensor_names
        q, k, g = get(n["q"]), get(n["k"]), get(n["gate"])
        dt = torch.float32 if torch.float32 in (q.dtype, k.dtype, g.dtype) else q.dtype
        w = torch.zeros(self.qkv_width, self.hidden, dtype=dt, device=q.device)
        w[:self.gate_col] = torch.cat([q.to(dt), k.to(dt)], dim=0)
        w[self.gate_col:self.gate_col + self.nh * self.d] = g.to(dt)
        self.w_qkv = w.contiguous()
        self.w_o = get(n["o"]).contiguous()
        self.qkv_bias = torch.cat([get(n["q"] + ".b").float(), get(n["k"] + ".b").float()]).contiguous()
        self.rel = get(n["rel"]).float().contiguous()
        self.pb = get(n["pb"]).float().contiguous()
        self.buckets = distance_buckets(self.rel.shape[0], self.bias_max).to(self.rel.device)

    def takes_normed_rows(self, num_tokens):
        return False

    def fuses_next_norm(self, num_tokens):
        return False

    def forward(self, x, batch, cache, writes_cache=True, then=None):
        T, ws = x.shape[0], self.ctx.workspace
        kc, vc, group = cache                       # one tensor: the keys are the values
        proj = linear(x, self.w_qkv, ws.get("qkv", T, self.qkv_width))
        ops.rope_kv_write_x(proj, batch.positions, batch.slot_mapping[group], None, 1.0, self.qkv_bias, kc, vc,
                            self.nh, self.nkv, self.d, 0, self.d, self.ctx.page_size, False, writes_cache)
        out = ws.get("attn_sum", T, self.nh * self.d)
        window, bt = int(self.window or 0), batch.block_tables[group]
        extras = dict(keep_first=self.keep_first, sigmoid_weights=True, head_bias=self.pb, dist_bias=self.rel,
                      dist_bucket=self.buckets)
        if batch.num_portions:
            if TILES_GENERAL not in batch.tiles:
                raise RuntimeError("the step's batch was built without the index lists this mixer declares in "
                                   "query_tiles(): give them to the BatchBuilder (query_tiles=...)")
            t16, t64 = batch.tiles[TILES_GENERAL], batch.tiles.get(TILES_MMA_X) if self._mma_x else None
            ops.attn_prefill_x(proj, self.qkv_width, kc, vc, bt, batch.bt_stride, batch.cu_q_lens, batch.context_lens,
                               t16.seq, t16.q0, t16.count, out, self.nh, self.nkv, self.d, self.d, 1,
                               self.ctx.page_size, window, self.scale, 0.0,
                               t64.seq if t64 else None, t64.q0 if t64 else None, t64.count if t64 else 0,
                               allow_mma=t64 is not None, **extras)
        if batch.num_decode:
            n = batch.num_decode
            facts = getattr(batch, "facts", None)
            longest = facts.max_context if facts is not None else max(s + q for s, q in zip(batch.q_starts, batch.q_lens))
            splits = self._splits(n, longest)
            ops.attn_decode_x(proj, self.qkv_width, kc, vc, bt, batch.bt_stride, batch.cu_q_lens, batch.context_lens,
                              batch.dec_seqs, n, splits, ws.get("attn_part_o", 1, n * self.nh * splits * self.d),
                              ws.get("attn_part_ml", 1, n * self.nh * splits * 2), out, self.nh, self.nkv, self.d,
                              self.d, 1, self.ctx.page_size, window, self.scale, 0.0, allow_mma=self._mma_x, **extras)
        gated = ws.get("attn_out", T, self.nh * self.d)
        ops.sigmoid_gate(out, proj[:, self.gate_col:self.gate_col + self.nh * self.d], gated)
        return linear(gated, self.w_o, ws.get(self.out_buffer, T, self.hidden), then)


register_mixer("sigmoid_attention", SigmoidAttention)
