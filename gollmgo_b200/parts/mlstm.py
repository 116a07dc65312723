"""The matrix memory with exponential gates (mLSTM): a recurrent mixer whose state per head is a matrix
S [d, dv], a vector n [d] and a running maximum m,

    m_t = max(f_t + m_{t-1}, i_t)                                  (m before the first token: 0)
    S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T,    n_t the same with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + floor),

with q = Wq x * d^-1/2, k = Wk x, v = Wv x per head, the log input gate i = cap tanh((Wi x + bi) / cap) and the
log forget gate f = logsigmoid(cap tanh((Wf x + bf) / cap)) per head.  Each head's o is divided by its root
mean square, the heads together are multiplied by a weight and by sigmoid(Wg x), and projected.

The recurrence is the engine's plain linear recurrence (csrc/delta_rule.cu, the form of a state-space layer)
with one more value column that is always 1, so that n is a column of S; the gates, the maxima and the
normaliser are csrc/mlstm.cu.  State per request, in its state slot: S with n in float32
[heads, dvp, d] (dvp = dv + 1 rounded up to 4) and m [heads].  Nothing is paged.  The gates' product is
summed and left in float32, and so is everything between the projections and the gated rows.

params: hidden_size, num_heads, head_dim, v_head_dim, gate_cap (0: none), eps, floor (default 1e-6), out_buffer,
names (optional dict: q, k, v, i, f, gate, o, norm; the gates' biases are the i, f names + ".b").
"""
from __future__ import annotations

import torch

from ..cache import FixedStateNeed
from ..csrc import ops
from ..weights import WeightSpec
from .linear import linear
from .registry import register_mixer

_NAMES = {"q": "q", "k": "k", "v": "v", "i": "i", "f": "f", "gate": "g", "o": "o", "norm": "norm"}


class MatrixMemory:
    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec["v_head_dim"])
        self.cap = float(spec.get("gate_cap") or 0.0)
        self.eps = float(spec["eps"])
        self.floor = float(spec.get("floor", 1e-6))
        self.names = dict(_NAMES, **(spec.get("names") or {}))
        self.out_buffer = spec.get("out_buffer") or "mixer_out"
        if self.d > 256:
            raise ValueError(f"key size {self.d} is beyond what the recurrence kernel takes (256)")
        self.dvp = -(-(self.dv + 1) // 4) * 4
        pad8 = lambda n: -(-n // 8) * 8
        self.qkv_cols = self.nh * (2 * self.d + self.dv)
        self.gate_col = pad8(self.qkv_cols)
        self.proj_width = pad8(self.gate_col + self.nh * self.dv)
        self.rows_width = self.nh * (2 * self.d + self.dvp)
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("mlstm_proj", T * self.proj_width, ctx.act_dtype)
        ws.reserve("mlstm_if", T * 2 * self.nh, torch.float32)
        ws.reserve("mlstm_rows", T * self.rows_width, torch.float32)
        ws.reserve("mlstm_beta", T * self.nh, torch.float32)
        ws.reserve("mlstm_decay", T * self.nh, torch.float32)
        ws.reserve("mlstm_m", T * self.nh, torch.float32)
        ws.reserve("mlstm_o", T * self.nh * self.dvp, torch.float32)
        ws.reserve("mlstm_y", T * self.nh * self.dv, ctx.act_dtype)
        ws.reserve(self.out_buffer, T * self.hidden, ctx.act_dtype)
        self.w_proj = self.w_if = self.b_i = self.b_f = self.norm_w = self.w_o = None

    def cache_need(self):
        return (FixedStateNeed((self.nh, self.dvp, self.d), "float32"), FixedStateNeed((self.nh,), "float32"))

    def weights(self):
        n, H, qk, vv = self.names, self.hidden, self.nh * self.d, self.nh * self.dv
        return {n["q"]: WeightSpec((qk, H)), n["k"]: WeightSpec((qk, H)), n["v"]: WeightSpec((vv, H)),
                n["gate"]: WeightSpec((vv, H)), n["o"]: WeightSpec((H, vv)), n["norm"]: WeightSpec((vv,)),
                n["i"]: WeightSpec((self.nh, H)), n["i"] + ".b": WeightSpec((self.nh,), init="normal"),
                n["f"]: WeightSpec((self.nh, H)), n["f"] + ".b": WeightSpec((self.nh,), init="normal")}

    def load(self, get):
        n = self.names
        parts = [get(n[x]) for x in ("q", "k", "v")]
        gate = get(n["gate"])
        dt = torch.float32 if any(p.dtype == torch.float32 for p in parts + [gate]) else parts[0].dtype
        w = torch.zeros(self.proj_width, self.hidden, dtype=dt, device=gate.device)
        w[:self.qkv_cols] = torch.cat([p.to(dt) for p in parts], dim=0)
        w[self.gate_col:self.gate_col + self.nh * self.dv] = gate.to(dt)
        self.w_proj = w.contiguous()
        self.w_if = torch.cat([get(n["i"]), get(n["f"])], dim=0).contiguous()
        self.b_i = get(n["i"] + ".b").float().contiguous()
        self.b_f = get(n["f"] + ".b").float().contiguous()
        self.norm_w = get(n["norm"]).float().contiguous()
        self.w_o = get(n["o"]).contiguous()

    def forward(self, x, batch, cache, writes_cache=True, then=None):
        T, ws, H = x.shape[0], self.ctx.workspace, self.nh
        state, m_state = cache
        proj = linear(x, self.w_proj, ws.get("mlstm_proj", T, self.proj_width))
        # the gates' inputs: a product of the activation type's values summed in float32 and left in float32
        zif = linear(x, self.w_if, ws.get("mlstm_if", T, 2 * H))
        beta, decay, m_row = ws.get("mlstm_beta", T, H), ws.get("mlstm_decay", T, H), ws.get("mlstm_m", T, H)
        B = batch.num_seqs
        ops.mlstm_gates(zif[:, :H], zif[:, H:], self.b_i, self.b_f, self.cap, m_state, batch.cu_q_lens, batch.context_lens,
                        batch.state_slots, B, H, beta, decay, m_row)
        rows = ws.get("mlstm_rows", T, self.rows_width)
        ops.mlstm_rows(proj, H, self.d, self.dv, self.dvp, self.d ** -0.5, rows)
        o = ws.get("mlstm_o", T, H * self.dvp)
        ops.delta_recur(rows, beta, decay, state, batch.cu_q_lens, batch.context_lens, batch.state_slots, B,
                        H, H, self.d, self.dvp, o, plain=True)
        y = ws.get("mlstm_y", T, H * self.dv)
        ops.mlstm_out(o, m_row, proj[:, self.gate_col:self.gate_col + H * self.dv], self.norm_w, self.eps, self.floor,
                      H, self.dv, self.dvp, y)
        return linear(y, self.w_o, ws.get(self.out_buffer, T, self.hidden), then)


register_mixer("mlstm", MatrixMemory)
