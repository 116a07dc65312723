"""Latent attention: every head's keys and values are expanded from one low-rank row per token
(the latent), which is all the cache keeps.  Without position encoding, or (``rot_dim`` > 0) with a
rotated part: every query head has ``rot_dim`` more values [head_dim unrotated | rot_dim rotated], the
down-projection has ``rot_dim`` more rows that are, rotated and not normed, one key part shared by all
heads, and the score is the sum of both dot products.  The cache row is then [latent | rotated key part]
and the query in the latent's space [Wuk_h^T q_h | rotated query part]: one dot product gives the score,
and the values are still the row's first ``rank`` columns.  ``window``: a query sees itself and the
window - 1 tokens before it (the cache group gives older pages back).  ``gate``: "head" (one sigmoid gate
per head), "element" (one per output channel of the concatenated heads) or False.

    q = Wq x  (heads x dim);   c = rmsnorm(Wdkv x) * w  (rank);   k_h = Wuk_h c;   v_h = Wuv_h c
    out = Wo concat_h( sigmoid(Wg x)_h * softmax_j(scale q_h . k_hj) v_hj ),  j <= i

The cache is a paged group with one "kv head" of size rank whose keys and values are the same
rows (``PagedKVNeed(shared_kv=True)``), so the engine's paged attention kernels run it as they
run a multi-query layer, in the latent's space: q_h . k_hj = (Wuk_h^T q_h) . c_j, and the sum of
p_j v_hj is Wuv_h (sum p_j c_j).  The two per-head products around the attention are one grouped
product each (csrc/grouped_gemm.cu; the second one applies the head's gate), the latent's norm
and its write to the cache one kernel (csrc/latent.cu).  q, the latent and the gates come from
one product with the three weights stacked.

params: hidden_size, num_heads, head_dim (of q and k, the unrotated part), v_head_dim, kv_rank, scale, eps (of the
latent's norm), gate (True = "head" | "element" | False), rot_dim, position (PartSpec of the rotated part; its
``interleaved`` and ``magnitude`` are honoured), window, expand (bool: the rotated form as multi-head attention over
cached per-head keys and values, which a row beyond 256 values takes by itself), names: dict of the tensors' local names.
"""
from __future__ import annotations

import os

import torch

from ..cache import PagedKVNeed
from ..csrc import ops
from ..weights import WeightSpec
from .attention import ATTN_POLICY, TILES_GENERAL, TILES_MMA, TILES_TC, context_tiles, decode_splits, TILE_KEYS, MAX_TILES
from .linear import GEMM_POLICY, linear
from .registry import build_position, register_mixer

DEFAULT_NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "gate": "g", "o": "o"}
RANK_ALIGN = 16          # the latent's rows are padded to a multiple of this in the cache (zeros)
# Steps of at least this many tokens (bfloat16, a latent that needs no padding) run the two per-head
# products as batched products of the vendor library, as the other products of prompt steps are:
# the grouped kernel's tiles of 32 rows are made for steps that stream the weights.  Measured on
# a prompt step of 2048 tokens (16 heads, 64 -> 128 and 128 -> 128): 20 us a product with the
# grouped kernel.
BMM_MIN_TOKENS = int(os.environ.get("GOLLMGO_B200_LATENT_BMM_TOKENS", "256"))


class LatentAttention:
    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.dim = int(spec["head_dim"])
        self.vdim = int(spec["v_head_dim"])
        self.rank = int(spec["kv_rank"])
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        gate = spec.get("gate", True)
        self.gate_kind = "head" if gate is True else (gate or None)
        if self.gate_kind not in (None, "head", "element"):
            raise ValueError(f"gate {gate!r} is not known (known: head, element)")
        self.gated = self.gate_kind == "head"
        self.names = {**DEFAULT_NAMES, **(spec.get("names") or {})}
        self.rot = int(spec.get("rot_dim") or 0)
        self.window = spec.get("window") or None
        self.position = build_position(spec["position"], ctx) if self.rot else None
        if self.rot and (self.position.rope_table() is None or 2 * self.position.rope_table().numel() != self.rot):
            raise ValueError(f"the rotated part of {self.rot} values needs a rotation of exactly that width")
        self.qh = self.dim + self.rot                     # a query head: [dim unrotated | rot rotated]
        self.rank_p = -(-self.rank // RANK_ALIGN) * RANK_ALIGN
        # A latent wider than the attention kernels' head size (256) cannot be read as a head: such a layer
        # caches the expanded keys and values instead (heads x max(dim, vdim) values each, zero-padded to one
        # size) and runs as ordinary multi-head attention.  More cache, the same result.
        self.expanded = self.rank_p > 256
        # the cache row and the query in the latent's space: the latent (padded), then the rotated part; in bfloat16 the
        # row is widened to 64 or 128 values where that is all it takes to run on the tensor-core kernels
        self.row = self.rank_p + -(-self.rot // 8) * 8
        if self.rot and ctx.act_dtype == torch.bfloat16 and self.row <= 128 and ATTN_POLICY != "general":
            self.row = 64 if self.row <= 64 else 128
        # The rotated form with a row beyond 256 values (or ``expand``): every head's keys [rotated part | expanded
        # part] and values are cached, and the layer runs as multi-head attention on the general kernels.
        self.wide = bool(self.rot) and (bool(spec.get("expand")) or self.expanded or self.row > 256)
        self.dk = -(-self.qh // 8) * 8
        if self.wide:
            self.expanded = False
            if self.dk > 256 or self.vdim > 256:
                raise ValueError(f"heads of {self.qh} key values or {self.vdim} values are beyond what the attention kernels take (256)")
            self.row = self.rank_p
        self.dmax = -(-max(self.dim, self.vdim) // 8) * 8
        if self.expanded and self.dmax > 256:
            raise ValueError(f"a latent of {self.rank} values with heads of {self.dim} / {self.vdim} values is beyond "
                             f"what the attention kernels take (256 for the latent or for the heads)")
        # columns of the stacked first product: q | latent | gates, each start a multiple of 8
        a8 = lambda n: -(-n // 8) * 8
        self.col_c = a8(self.nh * self.qh)
        self.col_g = self.col_c + a8(self.rank + self.rot)
        self.gate_cols = {None: 0, "head": self.nh, "element": self.nh * self.vdim}[self.gate_kind]
        self.width1 = self.col_g + a8(self.gate_cols)
        self.num_sms = torch.cuda.get_device_properties(ctx.device).multi_processor_count \
            if ctx.device.type == "cuda" else 148
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("lat_proj", T * self.width1, ctx.act_dtype)
        ws.reserve("lat_q", T * self.nh * self.row, ctx.act_dtype)
        ws.reserve("lat_o", T * self.nh * self.row, ctx.act_dtype)
        ws.reserve("attn_out", T * self.nh * self.vdim, ctx.act_dtype)
        ws.reserve("mixer_out", T * self.hidden, ctx.act_dtype)
        # the attention as the kernels see it: kv heads, query heads per kv head, head size
        self._nkv, self._group, self._d = (self.nh, 1, self.dmax) if self.expanded else (1, self.nh, self.row)
        if self.wide:
            self._nkv, self._group, self._d = self.nh, 1, max(self.dk, self.vdim)
        self._ctas_per_split = self._nkv * -(-self._group // 16)
        self._cluster_cap = None
        if ctx.device.type == "cuda":
            self._cluster_cap = [0] + [ops.attn_decode_cluster_capacity(ctx.act_dtype, self._d, s, self._group)
                                       for s in range(1, ops.ATTN_MAX_CLUSTER + 1)]
        esize = torch.empty((), dtype=ctx.act_dtype).element_size()
        self._tile_bytes = TILE_KEYS * self._d * esize * (2 if self.expanded or self.wide else 1)
        rows = max(n * self._splits(n, TILE_KEYS << b) for n in range(1, ctx.max_seqs + 1)
                   for b in range(MAX_TILES.bit_length()))
        ws.reserve("attn_part_o", rows * self.nh * self._d, torch.float32)
        ws.reserve("attn_part_ml", rows * self.nh * 2, torch.float32)
        if self.wide:
            self.wide_width = -(-(self.nh * (2 * self.dk + self.vdim)) // 8) * 8
            ws.reserve("lat_c", T * self.rank_p, ctx.act_dtype)
            ws.reserve("lat_qkv", T * self.wide_width, ctx.act_dtype)
            self._iota = torch.arange(T, dtype=torch.int32, device=ctx.device)
        if self.expanded:
            ws.reserve("lat_c", T * self.rank_p, ctx.act_dtype)
            ws.reserve("lat_qkv", T * 3 * self.nh * self.dmax, ctx.act_dtype)
            ws.reserve("lat_o", T * self.nh * self.dmax, ctx.act_dtype)
            self._iota = torch.arange(T, dtype=torch.int32, device=ctx.device)
        self.w_in = self.w_norm = self.w_uk_t = self.w_uv = self.w_o = None

    def cache_need(self):
        if self.wide:
            return PagedKVNeed(self.nh, self.dk, self.window, v_heads=self.nh, v_head_dim=self.vdim)
        if self.expanded:
            return PagedKVNeed(self.nh, self.dmax, self.window)
        return PagedKVNeed(1, self.row, self.window, shared_kv=True)

    def _fast(self):
        return not self.wide and self.ctx.act_dtype == torch.bfloat16 and self._d in (64, 128) and ATTN_POLICY != "general"

    def query_tiles(self):
        need = [TILES_GENERAL]
        if self._fast():
            need.append(TILES_MMA)
            if ATTN_POLICY == "auto" and (self._group % 2 == 0 or self._group == 1):
                need.append(TILES_TC)
        return need

    def _splits(self, n_dec, max_context):
        return decode_splits(n_dec, self._ctas_per_split, self.num_sms, self._cluster_cap,
                             context_tiles(max_context, self.window), self._tile_bytes)

    def step_tags(self, facts):
        n = facts.num_seqs if facts.decode_only else 0
        return (f"latent_slices={self._splits(n, facts.max_context)}",) if n else ()

    def weights(self):
        n, H = self.names, self.hidden
        m = {n["q"]: WeightSpec((self.nh * self.qh, H)),
             n["dkv"]: WeightSpec((self.rank + self.rot, H)),
             n["dkv_norm"]: WeightSpec((self.rank,)),
             n["uk"]: WeightSpec((self.nh * self.dim, self.rank)),
             n["uv"]: WeightSpec((self.nh * self.vdim, self.rank)),
             n["o"]: WeightSpec((H, self.nh * self.vdim))}
        if self.gate_cols:
            m[n["gate"]] = WeightSpec((self.gate_cols, H))
        return m

    def load(self, get):
        n = self.names
        q, dkv = get(n["q"]), get(n["dkv"])
        w = torch.zeros(self.width1, self.hidden, dtype=q.dtype, device=q.device)
        if self.wide:          # every query head as [rotated part | unrotated part]: the rotation kernel turns a head's first values
            q3 = q.view(self.nh, self.qh, self.hidden)
            q = torch.cat([q3[:, self.dim:], q3[:, :self.dim]], dim=1).reshape(self.nh * self.qh, self.hidden)
        w[:self.nh * self.qh] = q
        w[self.col_c:self.col_c + self.rank + self.rot] = dkv
        if self.gate_cols:
            w[self.col_g:self.col_g + self.gate_cols] = get(n["gate"])
        self.w_in = w.contiguous()
        self.w_norm = get(n["dkv_norm"]).to(torch.float32).contiguous()
        # [heads, rank, dim]: the transpose of each head's key expansion, so that the query goes
        # to the latent's space with the same grouped product that brings the result back
        self.w_uk_t = get(n["uk"]).view(self.nh, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = get(n["uv"]).view(self.nh, self.vdim, self.rank).contiguous()
        self.w_uk = get(n["uk"]).view(self.nh, self.dim, self.rank).contiguous() if self.expanded or self.wide else None
        self.w_o = get(n["o"]).contiguous()

    def _attend(self, q, q_stride, kc, vc, group, batch, o):
        """The engine's paged attention over this step's queries q (head h of token t at q[t, h * d ...])."""
        ws, nh, nkv, d, ps = self.ctx.workspace, self.nh, self._nkv, self._d, self.ctx.page_size
        bt = batch.block_tables[group]
        if batch.num_portions:
            if TILES_GENERAL not in batch.tiles:
                raise RuntimeError("the step's batch was built without the index lists this mixer declares in "
                                   "query_tiles(): give them to the BatchBuilder (query_tiles=...)")
            t16, t64, t128 = batch.tiles[TILES_GENERAL], batch.tiles.get(TILES_MMA), batch.tiles.get(TILES_TC)
            if not self._fast():
                t64 = t128 = None
            ops.attn_prefill(q, q_stride, kc, vc, bt, batch.bt_stride, batch.cu_q_lens, batch.context_lens,
                             t16.seq, t16.q0, t16.count, o, nh, nkv, d, ps, int(self.window or 0), self.scale,
                             t64.seq if t64 else None, t64.q0 if t64 else None, t64.count if t64 else 0,
                             allow_mma=t64 is not None,
                             tile128_seq=t128.seq if t128 else None, tile128_q0=t128.q0 if t128 else None,
                             num_tiles128=t128.count if t128 else 0, allow_tc=t128 is not None)
        if batch.num_decode:
            n = batch.num_decode
            facts = getattr(batch, "facts", None)
            longest = facts.max_context if facts is not None else max(s + l for s, l in zip(batch.q_starts, batch.q_lens))
            splits = self._splits(n, longest)
            ops.attn_decode(q, q_stride, kc, vc, bt, batch.bt_stride, batch.cu_q_lens, batch.context_lens,
                            batch.dec_seqs, n, splits, ws.get("attn_part_o", 1, n * nh * splits * d),
                            ws.get("attn_part_ml", 1, n * nh * splits * 2), o, nh, nkv, d, ps, int(self.window or 0), self.scale,
                            allow_mma=self._fast())

    def _forward_expanded(self, x, batch, cache, writes_cache):
        """Keys and values expanded from the latent before they are cached (a latent too wide to be a head)."""
        T, ws = x.shape[0], self.ctx.workspace
        kc, vc, group = cache
        nh, R, Rp, dm = self.nh, self.rank, self.rank_p, self.dmax
        proj = ws.get("lat_proj", T, self.width1)
        linear(x, self.w_in, proj)
        c = ws.get("lat_c", T, Rp)
        ops.latent_norm_write(proj, self.col_c, R, self.w_norm, self.eps, self._iota[:T], c)      # row t of c: the latent of token t
        qkv = ws.get("lat_qkv", T, 3 * nh * dm)
        qkv.zero_()                                           # the padding of every head stays zero
        qkv.view(T, 3, nh, dm)[:, 0, :, :self.dim].copy_(proj[:, :nh * self.dim].view(T, nh, self.dim))      # (no rotated part here)
        ops.grouped_gemm(c, self.w_uk, qkv[:, nh * dm:], self.dim, R, nh, a_group_cols=0, o_group_cols=dm, n_padded=dm, rows=T)
        ops.grouped_gemm(c, self.w_uv, qkv[:, 2 * nh * dm:], self.vdim, R, nh, a_group_cols=0, o_group_cols=dm, n_padded=dm, rows=T)
        ops.rope_kv_write(qkv, batch.positions, batch.slot_mapping[group], None, kc, vc, nh, nh, dm, self.ctx.page_size,
                          False, writes_cache)
        o = ws.get("lat_o", T, nh * dm)
        self._attend(qkv, 3 * nh * dm, kc, vc, group, batch, o)
        a = ws.get("attn_out", T, nh * self.vdim)
        a3 = a.view(T, nh, self.vdim)
        a3.copy_(o.view(T, nh, dm)[:, :, :self.vdim])
        if self.gated:
            ops.head_gate(a, proj, self.col_g, nh)
        elif self.gate_cols:
            ops.gate_mul(a, proj[:, self.col_g:self.col_g + self.gate_cols])
        return linear(a, self.w_o, ws.get("mixer_out", T, self.hidden))

    def _forward_wide(self, x, batch, cache, writes_cache):
        """The rotated form as multi-head attention: per head the keys [rot(shared key part) | Wuk_h c] and the values
        Wuv_h c are cached; the queries are [rot(rotated part) | unrotated part]."""
        T, ws = x.shape[0], self.ctx.workspace
        kc, vc, group = cache
        nh, R, Rp, dk, rot, vd = self.nh, self.rank, self.rank_p, self.dk, self.rot, self.vdim
        proj = linear(x, self.w_in, ws.get("lat_proj", T, self.width1))
        c = ws.get("lat_c", T, Rp)
        ops.latent_norm_write(proj, self.col_c, R, self.w_norm, self.eps, self._iota[:T], c)      # row t of c: the latent of token t
        qkv = ws.get("lat_qkv", T, self.wide_width)
        if dk != self.qh or self.wide_width != nh * (2 * dk + vd):
            qkv.zero_()                                       # the padding of every head stays zero
        qkv[:, :nh * dk].view(T, nh, dk)[:, :, :self.qh].copy_(proj[:, :nh * self.qh].view(T, nh, self.qh))
        k3 = qkv[:, nh * dk:2 * nh * dk].view(T, nh, dk)
        k3[:, :, :rot].copy_(proj[:, self.col_c + R:self.col_c + R + rot].unsqueeze(1).expand(T, nh, rot))
        ops.grouped_gemm(c, self.w_uk, qkv[:, nh * dk + rot:], self.dim, R, nh, a_group_cols=0, o_group_cols=dk,
                         n_padded=self.dim, rows=T)
        ops.grouped_gemm(c, self.w_uv, qkv[:, 2 * nh * dk:], vd, R, nh, a_group_cols=0, o_group_cols=vd, n_padded=vd, rows=T)
        ops.rope_kv_write_x(qkv, batch.positions, batch.slot_mapping[group], self.position.rope_table(),
                            float(getattr(self.position, "magnitude", 1.0)), None, kc, vc, nh, nh, dk, nh, vd,
                            self.ctx.page_size, self.position.interleaved, writes_cache)
        a = ws.get("attn_out", T, nh * vd)
        window, bt = int(self.window or 0), batch.block_tables[group]
        if batch.num_portions:
            t16 = batch.tiles[TILES_GENERAL]
            ops.attn_prefill_x(qkv, self.wide_width, kc, vc, bt, batch.bt_stride, batch.cu_q_lens, batch.context_lens,
                               t16.seq, t16.q0, t16.count, a, nh, nh, dk, vd, 1, self.ctx.page_size, window, self.scale, 0.0,
                               allow_mma=False)
        if batch.num_decode:
            n = batch.num_decode
            facts = getattr(batch, "facts", None)
            longest = facts.max_context if facts is not None else max(s + l for s, l in zip(batch.q_starts, batch.q_lens))
            splits = self._splits(n, longest)
            ops.attn_decode_x(qkv, self.wide_width, kc, vc, bt, batch.bt_stride, batch.cu_q_lens, batch.context_lens,
                              batch.dec_seqs, n, splits, ws.get("attn_part_o", 1, n * nh * splits * vd),
                              ws.get("attn_part_ml", 1, n * nh * splits * 2), a, nh, nh, dk, vd, 1, self.ctx.page_size, window,
                              self.scale, 0.0, allow_mma=False)
        if self.gated:
            ops.head_gate(a, proj, self.col_g, nh)
        elif self.gate_cols:
            ops.gate_mul(a, proj[:, self.col_g:self.col_g + self.gate_cols])
        return linear(a, self.w_o, ws.get("mixer_out", T, self.hidden))

    def forward(self, x, batch, cache, writes_cache=True):
        if self.wide:
            return self._forward_wide(x, batch, cache, writes_cache)
        if self.expanded:
            return self._forward_expanded(x, batch, cache, writes_cache)
        T, ws = x.shape[0], self.ctx.workspace
        kc, vc, group = cache
        nh, R, Rp, row = self.nh, self.rank, self.rank_p, self.row
        proj = linear(x, self.w_in, ws.get("lat_proj", T, self.width1))
        if writes_cache:
            ops.latent_norm_write(proj, self.col_c, R, self.w_norm, self.eps, batch.slot_mapping[group], kc)
        q = ws.get("lat_q", T, nh * row)
        lib = (T >= BMM_MIN_TOKENS and Rp == R and self.ctx.act_dtype == torch.bfloat16 and GEMM_POLICY != "tc")
        q_heads = proj[:, :nh * self.qh].view(T, nh, self.qh)[:, :, :self.dim].transpose(0, 1)      # [heads, T, dim]
        if lib and row == R:
            # [heads, T, dim] @ [heads, dim, rank] -> [heads, T, rank], all three as views of the step's buffers
            torch.bmm(q_heads, self.w_uk_t.transpose(1, 2), out=q.view(T, nh, Rp).transpose(0, 1))
        elif lib:
            qv = q.view(T, nh, row)
            qv[:, :, R:].zero_()                                   # the padding of every head's row stays zero
            qv[:, :, :R].copy_(torch.bmm(q_heads, self.w_uk_t.transpose(1, 2)).transpose(0, 1))
        else:
            ops.grouped_gemm(proj, self.w_uk_t, q, R, self.dim, nh, a_group_cols=self.qh, o_group_cols=row,
                             n_padded=row, rows=T)
        if self.rot:
            # the rotated parts: the shared key part into the cache row, every head's query part into its row of q
            ops.latent_rope(proj, self.col_c + R, self.qh, self.dim, nh, batch.positions, self.position.rope_table(),
                            float(getattr(self.position, "magnitude", 1.0)), self.position.interleaved,
                            batch.slot_mapping[group], kc, q, row, Rp, writes_cache)
        o = ws.get("lat_o", T, nh * row)
        self._attend(q, nh * row, kc, vc, group, batch, o)
        a = ws.get("attn_out", T, nh * self.vdim)
        if lib:
            torch.bmm(o.view(T, nh, row)[:, :, :R].transpose(0, 1), self.w_uv.transpose(1, 2),
                      out=a.view(T, nh, self.vdim).transpose(0, 1))
            if self.gated:
                ops.head_gate(a, proj, self.col_g, nh)
        else:
            ops.grouped_gemm(o, self.w_uv, a, self.vdim, R, nh, a_group_cols=row, o_group_cols=self.vdim, rows=T,
                             gate=proj if self.gated else None, gate_col0=self.col_g)
        if self.gate_kind == "element":
            ops.gate_mul(a, proj[:, self.col_g:self.col_g + self.gate_cols])
        return linear(a, self.w_o, ws.get("mixer_out", T, self.hidden))


register_mixer("latent_attention", LatentAttention)
