"""A state-space mixer of the Mamba-2 kind.  One product makes [z | x | B | C | dt] from the input
(``heads`` heads of ``v_head_dim`` values in z and x, ``groups`` groups of ``state`` values in B and C,
one dt per head); x, B and C pass a short causal convolution per channel (with bias) and SiLU;
dt <- softplus(dt + dt_bias).  Per head h (reading group h // (heads / groups)) a state matrix
S [state, v_head_dim] evolves as

    S <- exp(-exp(A_log_h) dt) S + dt B x^T,        y = S^T C + D_h x,

y is multiplied by silu(z), RMS-normed in ``norm_groups`` equal parts of the row, multiplied by a
weight, and projected back.

State per request, in its state slot: S in float32 [heads, v_head_dim, state] and the last
taps - 1 inputs of the convolution in float32 [taps - 1, channels].  Nothing is paged.  The
recurrence is the linear-recurrence kernel of the delta rule without the delta (csrc/delta_rule.cu,
csrc/ssm.cu); everything between the two products is float32.

params: hidden_size, num_heads, v_head_dim, state, groups, conv (taps), norm_groups, eps, out_buffer,
names (optional dict: in, conv, conv_bias, dt_bias, A_log, D, norm, o).
"""
from __future__ import annotations

import torch

from ..cache import FixedStateNeed
from ..csrc import ops
from ..weights import WeightSpec
from .linear import linear
from .registry import register_mixer

_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
          "norm": "norm", "o": "o"}


class StateSpaceMixer:
    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.p = int(spec["v_head_dim"])
        self.n = int(spec["state"])
        self.groups = int(spec.get("groups") or 1)
        self.taps = int(spec["conv"])
        self.parts = int(spec.get("norm_groups") or 1)
        self.eps = float(spec["eps"])
        self.names = dict(_NAMES, **(spec.get("names") or {}))
        self.out_buffer = spec.get("out_buffer") or "mixer_out"
        if self.nh % self.groups:
            raise ValueError(f"{self.nh} heads are not a multiple of {self.groups} groups")
        if self.n > 256:
            raise ValueError(f"state size {self.n} is beyond what the recurrence kernel takes (256)")
        if not (1 <= self.taps <= 17):
            raise ValueError(f"{self.taps} taps are outside 1..17")
        self.inner = self.nh * self.p
        if self.inner % self.parts:
            raise ValueError(f"{self.inner} values do not split into {self.parts} equal parts")
        self.channels = self.inner + 2 * self.groups * self.n                 # x, B, C: what the convolution sees
        self.proj_width = self.inner + self.channels + self.nh               # z, x, B, C, dt
        self.proj_padded = -(-self.proj_width // 8) * 8
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("ssm_proj", T * self.proj_padded, ctx.act_dtype)
        ws.reserve("ssm_cbx", T * self.channels, torch.float32)
        ws.reserve("ssm_dt", T * self.nh, torch.float32)
        ws.reserve("ssm_decay", T * self.nh, torch.float32)
        ws.reserve("ssm_y", T * self.inner, torch.float32)
        ws.reserve("ssm_out", T * self.inner, ctx.act_dtype)
        ws.reserve(self.out_buffer, T * self.hidden, ctx.act_dtype)
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.a_log = self.dt_bias = self.d_skip = self.norm_w = None

    def cache_need(self):
        need = [FixedStateNeed((self.nh, self.p, self.n), "float32")]
        if self.taps > 1:
            need.append(FixedStateNeed((self.taps - 1, self.channels), "float32"))
        return tuple(need)

    def weights(self):
        n = self.names
        return {n["in"]: WeightSpec((self.proj_width, self.hidden)),
                n["conv"]: WeightSpec((self.channels, self.taps), init="taps"),
                n["conv_bias"]: WeightSpec((self.channels,), init="normal"),
                n["dt_bias"]: WeightSpec((self.nh,), init="normal"),
                n["A_log"]: WeightSpec((self.nh,), init="normal"),
                n["D"]: WeightSpec((self.nh,), init="normal"),
                n["norm"]: WeightSpec((self.inner,)),
                n["o"]: WeightSpec((self.hidden, self.inner))}

    def load(self, get):
        n = self.names
        w = get(n["in"])
        if self.proj_padded != self.proj_width:           # rows of zeros: the product's rows start on 16-byte borders
            w = torch.cat([w, torch.zeros(self.proj_padded - self.proj_width, self.hidden, dtype=w.dtype, device=w.device)])
        self.w_in = w.contiguous()
        self.w_o = get(n["o"]).contiguous()
        self.conv_w = get(n["conv"]).float().contiguous()
        self.conv_b = get(n["conv_bias"]).float().contiguous()
        self.a_log = get(n["A_log"]).float().contiguous()
        self.dt_bias = get(n["dt_bias"]).float().contiguous()
        self.d_skip = get(n["D"]).float().contiguous()
        self.norm_w = get(n["norm"]).float().contiguous()

    def forward(self, x, batch, cache, writes_cache=True, then=None):
        T, ws = x.shape[0], self.ctx.workspace
        state = cache[0]
        conv_state = cache[1] if self.taps > 1 else None
        proj = linear(x, self.w_in, ws.get("ssm_proj", T, self.proj_padded))
        cbx = ws.get("ssm_cbx", T, self.channels)
        dt, decay = ws.get("ssm_dt", T, self.nh), ws.get("ssm_decay", T, self.nh)
        B = batch.num_seqs
        ops.ssm_prep(proj, self.conv_w, self.conv_b, conv_state, self.a_log, self.dt_bias, batch.cu_q_lens,
                     batch.context_lens, batch.state_slots, B, self.nh, self.p, self.groups, self.n, cbx, dt, decay)
        y = ws.get("ssm_y", T, self.inner)
        # rows [C | B | x] are the recurrence's q, k, v; the step size takes beta's place
        ops.delta_recur(cbx, dt, decay, state, batch.cu_q_lens, batch.context_lens, batch.state_slots, B,
                        self.groups, self.nh, self.n, self.p, y, plain=True)
        out = ws.get("ssm_out", T, self.inner)
        ops.ssm_out(y, cbx, 2 * self.groups * self.n, proj[:, :self.inner], self.d_skip, self.norm_w, self.eps,
                    self.nh, self.p, self.parts, out)
        return linear(out, self.w_o, ws.get(self.out_buffer, T, self.hidden), then)


register_mixer("mamba2", StateSpaceMixer)
