"""A mixture of experts as a feed-forward: a router picks ``top`` of ``experts`` small SiLU-gated
feed-forwards per token, their results are summed with the router's weights, and an optional
shared expert (any registered feed-forward) runs for every token and is added.

Router: logits = x Wr^T + b in float32; the ``top`` largest are chosen and weighted by the
softmax over the chosen logits alone.  Everything happens on the device (csrc/moe.cu): the
(token, choice) pairs are sorted by expert there, two grouped products (csrc/grouped_gemm.cu) run
every expert over its own rows (first product with the gate's activation in its epilogue; long
steps in bfloat16 take the tcgen05 product of csrc/gemm_tc.cu over rows gathered into whole tiles
per expert), and a last kernel sums each token's results in float32.  No count ever reaches the host, so a step of
decoded tokens is captured like any other.

Variants, all parameters: ``router_weigh="softmax_all"``: the scores are the softmax over all
experts and the weights the chosen scores divided by their sum (+ 1e-20); ``groups`` = (count, keep):
the experts form ``count`` equal groups of neighbours, a group's score is its best expert's, and
only experts of the ``keep`` best groups can be chosen; ``activation="clamped_swish"`` (``limit``,
``alpha`` = 1.702, ``shift`` = 1): an expert computes g * sigmoid(alpha g) * (u + shift) with
g = min(gate, limit), u = clamp(up, -limit, limit) instead of silu(gate) * up.

params: hidden_size, intermediate_size, experts, top, router_bias (bool), router_weigh, groups,
activation, limit, alpha, shift, shared (a feed-forward PartSpec or None), names: dict with "router",
"router_bias", "expert" (a format string with {e}), "gate", "up", "down", "shared" (prefix of the
shared expert's tensors).
"""
from __future__ import annotations

import torch

import os

from ..csrc import ops
from ..weights import WeightSpec
from .linear import GEMM_POLICY, linear
from .registry import build_feed_forward, register_feed_forward

# Steps with at least this many (token, choice) pairs run the experts' products on tcgen05
# (csrc/gemm_tc.cu, grouped): every expert's rows gathered into a block that starts at a multiple
# of the product's tile height.  Below, a tile of 128 rows would be mostly padding.
TC_MIN_PAIRS = int(os.environ.get("GOLLMGO_B200_MOE_TC_PAIRS", "1024"))
TC_TILE = 128
# From this many tokens the router's logits are a product of the vendor library (bfloat16 rows, float32
# accumulation and result) followed by the choice alone; below, one kernel does both from shared memory.
ROUTE_LIB_TOKENS = int(os.environ.get("GOLLMGO_B200_MOE_ROUTE_LIB_TOKENS", "512"))

DEFAULT_NAMES = {"router": "router", "router_bias": "router.b", "expert": "e{e}.", "gate": "gate",
                 "up": "up", "down": "down", "shared": "shared."}


class MixtureOfExperts:
    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        if not (0 < self.top <= self.experts):
            raise ValueError(f"{self.top} choices of {self.experts} experts")
        if self.experts > ops.MOE_MAX_EXPERTS or self.top > ops.MOE_MAX_TOP:
            raise ValueError(f"the routing kernels take at most {ops.MOE_MAX_EXPERTS} experts and "
                             f"{ops.MOE_MAX_TOP} choices a token")
        self.router_bias = bool(spec.get("router_bias", True))
        self.weigh = spec.get("router_weigh") or "softmax_chosen"
        if self.weigh not in ops.MOE_WEIGH:
            raise ValueError(f"router weights {self.weigh!r} are not known (known: {sorted(ops.MOE_WEIGH)})")
        self.group_count, self.group_keep = (int(g) for g in (spec.get("groups") or (1, 1)))
        if self.experts % self.group_count or not (1 <= self.group_keep <= self.group_count) \
                or self.top > self.group_keep * (self.experts // self.group_count):
            raise ValueError(f"{self.experts} experts in {self.group_count} groups of which {self.group_keep} are kept "
                             f"do not give {self.top} choices")
        self.activation = spec.get("activation") or "silu"
        if self.activation not in ("silu", "clamped_swish"):
            raise ValueError(f"activation {self.activation!r} is not supported (known: silu, clamped_swish)")
        if self.activation == "clamped_swish":
            self.limit = float(spec["limit"])
            self.alpha = float(spec.get("alpha", 1.702))
            self.shift = float(spec.get("shift", 1.0))
        self.names = {**DEFAULT_NAMES, **(spec.get("names") or {})}
        shared = spec.get("shared")
        self.shared = build_feed_forward(shared, ctx) if shared is not None else None
        ws, T = ctx.workspace, ctx.max_tokens
        n = T * self.top
        self.tc_ok = (ctx.act_dtype == torch.bfloat16 and GEMM_POLICY != "lib" and self.hidden % 8 == 0
                      and self.inter % 8 == 0 and ctx.device.type == "cuda")
        slots = self._slots(n) if self.tc_ok and n >= TC_MIN_PAIRS else n
        ws.reserve("moe_logits", T * self.experts, torch.float32)
        ws.reserve("moe_idx", n, torch.int32)
        ws.reserve("moe_wgt", n, torch.float32)
        ws.reserve("moe_order", slots, torch.int32)
        ws.reserve("moe_place", n, torch.int32)
        ws.reserve("moe_offsets", self.experts + 1, torch.int32)
        ws.reserve("moe_tiles", slots // TC_TILE + 1, torch.int32)
        ws.reserve("moe_in", slots * self.hidden, ctx.act_dtype)
        ws.reserve("moe_act", slots * self.inter, ctx.act_dtype)
        if self.activation != "silu":
            ws.reserve("moe_gate_up", slots * 2 * self.inter, ctx.act_dtype)
        ws.reserve("moe_rows", slots * self.hidden, ctx.act_dtype)
        ws.reserve("moe_out", T * self.hidden, ctx.act_dtype)
        self.w_router = self.b_router = self.w_gate_up = self.w_down = None

    def _slots(self, n):
        """Places of the padded row block: every expert's rows rounded up to whole tiles."""
        return (-(-n // TC_TILE) + self.experts) * TC_TILE

    def _expert(self, e, which):
        return self.names["expert"].format(e=e) + self.names[which]

    def weights(self):
        m = {self.names["router"]: WeightSpec((self.experts, self.hidden))}
        if self.router_bias:
            m[self.names["router_bias"]] = WeightSpec((self.experts,))
        for e in range(self.experts):
            m[self._expert(e, "gate")] = WeightSpec((self.inter, self.hidden))
            m[self._expert(e, "up")] = WeightSpec((self.inter, self.hidden))
            m[self._expert(e, "down")] = WeightSpec((self.hidden, self.inter))
        if self.shared is not None:
            m.update({self.names["shared"] + k: v for k, v in self.shared.weights().items()})
        return m

    def load(self, get):
        self.w_router = get(self.names["router"]).contiguous()
        self.b_router = get(self.names["router_bias"]).to(torch.float32).contiguous() if self.router_bias else None
        # [experts, 2 * inter, hidden]: an expert's gate rows, then its up rows
        self.w_gate_up = torch.stack([torch.cat([get(self._expert(e, "gate")), get(self._expert(e, "up"))], dim=0)
                                      for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([get(self._expert(e, "down")) for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.load(lambda local: get(self.names["shared"] + local))

    def route(self, x):
        """(choices [T, top] int32, weights [T, top] float32) of the rows x."""
        T, ws = x.shape[0], self.ctx.workspace
        idx, wgt = ws.get("moe_idx", T, self.top), ws.get("moe_wgt", T, self.top)
        if T >= ROUTE_LIB_TOKENS and x.dtype == torch.bfloat16:
            # a long step: the logits are a product like any other (bfloat16 rows, float32 sums and result)
            z = ws.get("moe_logits", T, self.experts)
            linear(x, self.w_router, z)
            ops.moe_topk(z, self.b_router, self.top, idx, wgt, self.weigh, self.group_count, self.group_keep)
        else:
            ops.moe_route(x, self.w_router, self.b_router, self.top, idx, wgt, self.weigh, self.group_count,
                          self.group_keep)
        return idx, wgt

    def _activate(self, gate_up, a):
        ops.clamped_gate(gate_up, a, self.limit, self.alpha, self.shift)

    def forward(self, x, batch):
        T, ws = x.shape[0], self.ctx.workspace
        n, E = T * self.top, self.experts
        idx, wgt = self.route(x)
        place = ws.get("moe_place", 1, n)
        offsets = ws.get("moe_offsets", 1, E + 1)
        if self.tc_ok and n >= TC_MIN_PAIRS and x.is_contiguous():
            # a long step: rows gathered by expert into whole tiles, both products on tcgen05
            slots = self._slots(n)
            order, tiles = ws.get("moe_order", 1, slots), ws.get("moe_tiles", 1, slots // TC_TILE)
            ops.moe_align(idx, n, E, offsets, order, place, pad=TC_TILE, tile_group=tiles)
            xin = ws.get("moe_in", slots, self.hidden)
            ops.moe_gather(x, order, self.top, xin)
            a = ws.get("moe_act", slots, self.inter)
            if self.activation == "silu":
                ops.gemm_tc_grouped(xin, self.w_gate_up, a, tiles, E, gated=True)
            else:
                gu = ws.get("moe_gate_up", slots, 2 * self.inter)
                ops.gemm_tc_grouped(xin, self.w_gate_up, gu, tiles, E)
                self._activate(gu, a)
            y = ws.get("moe_rows", slots, self.hidden)
            ops.gemm_tc_grouped(a, self.w_down, y, tiles, E)
        else:
            order = ws.get("moe_order", 1, n)
            ops.moe_align(idx, n, E, offsets, order, place)
            a = ws.get("moe_act", n, self.inter)
            if self.activation == "silu":
                ops.grouped_gemm(x, self.w_gate_up, a, self.inter, self.hidden, E, offsets=offsets, row_index=order,
                                 row_div=self.top, rows=n, gated=True)
            else:
                gu = ws.get("moe_gate_up", n, 2 * self.inter)
                ops.grouped_gemm(x, self.w_gate_up, gu, 2 * self.inter, self.hidden, E, offsets=offsets, row_index=order,
                                 row_div=self.top, rows=n)
                self._activate(gu, a)
            y = ws.get("moe_rows", n, self.hidden)
            ops.grouped_gemm(a, self.w_down, y, self.hidden, self.inter, E, offsets=offsets, rows=n)
        shared = self.shared.forward(x, batch) if self.shared is not None else None
        out = ws.get("moe_out", T, self.hidden)
        ops.moe_combine(y, place, wgt, shared, out, self.top)
        return out


register_feed_forward("moe", MixtureOfExperts)
