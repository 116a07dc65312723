"""The gated delta rule: a recurrent mixer whose state per head is a matrix S [d, dv],

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q,

with q and k (``num_kv_heads`` heads of size ``head_dim``, shared by ``num_heads / num_kv_heads``
value heads each) and v (``num_heads`` heads of size ``v_head_dim``) passed through a short causal
convolution and SiLU, q and k made unit vectors (q times head_dim^-1/2), beta = sigmoid(Wb x),
g = exp(-exp(A_log) * softplus(Wa x + dt_bias)) per head.  The result is divided by its root mean
square per head, multiplied by a weight shared by the heads and by silu(Wg x), and projected.

State per request, in its state slot: S in float32 [heads, dv, d] and the last taps - 1 inputs
of the convolution in float32 [taps - 1, channels].  Nothing is paged.  Everything between the
projections and the output projection is float32 (csrc/delta_rule.cu).

Variants, all parameters: ``decay="channel"``: g is a factor per head and key channel (a row of S,
``dt_bias`` then [heads * head_dim]) instead of one per head; ``a_rank`` / ``gate_rank``: the
decay's input and the output gate come through two products of that inner width (tensors a1, a2 and
g1, g2) instead of one; ``gate_act="sigmoid"``: the output gate is a sigmoid instead of SiLU.

params: hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim, conv (taps), eps, out_buffer,
decay ("head" | "channel"), a_rank, gate_rank (None: one product; else the inner width that random
weights are made with: a checkpoint's tensors decide), gate_act ("silu" | "sigmoid"),
names (optional dict: q, k, v, beta, a, gate, o, A_log, dt_bias, norm, a1, a2, g1, g2; the
convolutions' tensors are the q, k, v names + ".conv").
"""
from __future__ import annotations

import torch

from ..cache import FixedStateNeed
from ..csrc import ops
from ..weights import WeightSpec
from .linear import linear
from .registry import register_mixer

_NAMES = {"q": "q", "k": "k", "v": "v", "beta": "b", "a": "a", "gate": "g", "o": "o", "A_log": "A_log",
          "dt_bias": "dt_bias", "norm": "norm", "a1": "a1", "a2": "a2", "g1": "g1", "g2": "g2"}


class GatedDeltaRule:
    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec["v_head_dim"])
        self.taps = int(spec["conv"])
        self.eps = float(spec["eps"])
        self.names = dict(_NAMES, **(spec.get("names") or {}))
        self.out_buffer = spec.get("out_buffer") or "mixer_out"
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads are not a multiple of {self.nkv} q/k heads")
        if self.d > 256:
            raise ValueError(f"key size {self.d} is beyond what the recurrence kernel takes (256)")
        if not (1 <= self.taps <= 17):
            raise ValueError(f"{self.taps} taps are outside 1..17")
        decay = spec.get("decay") or "head"
        if decay not in ("head", "channel"):
            raise ValueError(f"decay {decay!r} is not known (known: head, channel)")
        self.dw = self.d if decay == "channel" else 1                        # decays per head and token
        self.a_rank = int(spec.get("a_rank") or 0)
        self.gate_rank = int(spec.get("gate_rank") or 0)
        self.gate_act = spec.get("gate_act") or "silu"
        if self.gate_act not in ("silu", "sigmoid"):
            raise ValueError(f"gate activation {self.gate_act!r} is not known (known: silu, sigmoid)")
        self.channels = 2 * self.nkv * self.d + self.nh * self.dv            # q, k, v: what the convolution sees
        self._layout()
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("delta_ba", T * self.nh * (1 + self.dw), torch.float32)
        ws.reserve("delta_qkv", T * self.channels, torch.float32)
        ws.reserve("delta_beta", T * self.nh, torch.float32)
        ws.reserve("delta_decay", T * self.nh * self.dw, torch.float32)
        if self.gate_rank:
            ws.reserve("delta_gate", T * self.nh * self.dv, ctx.act_dtype)
        ws.reserve("delta_o", T * self.nh * self.dv, torch.float32)
        ws.reserve("delta_y", T * self.nh * self.dv, ctx.act_dtype)
        ws.reserve(self.out_buffer, T * self.hidden, ctx.act_dtype)
        self.w_proj = self.w_ba = self.w_o = self.w_a2 = self.w_g2 = None
        self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def _layout(self):
        """Columns of the stacked first product: q, k, v, then the gate (or its inner values), then the
        decay's inner values; every part starts at a multiple of 8 columns."""
        pad8 = lambda n: -(-n // 8) * 8
        self.gate_col = pad8(self.channels)
        self.gate_cols = self.gate_rank or self.nh * self.dv
        self.a_col = pad8(self.gate_col + self.gate_cols)
        self.proj_width = pad8(self.a_col + self.a_rank) if self.a_rank else pad8(self.gate_col + self.gate_cols)
        self.ctx.workspace.reserve("delta_proj", self.ctx.max_tokens * self.proj_width, self.ctx.act_dtype)

    def cache_need(self):
        need = [FixedStateNeed((self.nh, self.dv, self.d), "float32")]
        if self.taps > 1:
            need.append(FixedStateNeed((self.taps - 1, self.channels), "float32"))
        return tuple(need)

    def weights(self):
        n = self.names
        qk, vv = self.nkv * self.d, self.nh * self.dv
        w = {n["q"]: WeightSpec((qk, self.hidden)), n["k"]: WeightSpec((qk, self.hidden)),
             n["v"]: WeightSpec((vv, self.hidden)),
             n["beta"]: WeightSpec((self.nh, self.hidden)),
             n["A_log"]: WeightSpec((self.nh,), init="normal"),
             n["dt_bias"]: WeightSpec((self.nh * self.dw,), init="normal"),
             n["norm"]: WeightSpec((self.dv,)), n["o"]: WeightSpec((self.hidden, vv))}
        if self.gate_rank:
            # the inner widths are the checkpoint's: what the parameters say is what random weights are made with
            w[n["g1"]] = WeightSpec((self.gate_rank, self.hidden), free_dims=(0,))
            w[n["g2"]] = WeightSpec((vv, self.gate_rank), free_dims=(1,))
        else:
            w[n["gate"]] = WeightSpec((vv, self.hidden))
        if self.a_rank:
            w[n["a1"]] = WeightSpec((self.a_rank, self.hidden), free_dims=(0,))
            w[n["a2"]] = WeightSpec((self.nh * self.dw, self.a_rank), free_dims=(1,))
        else:
            w[n["a"]] = WeightSpec((self.nh * self.dw, self.hidden))
        w.update({n["q"] + ".conv": WeightSpec((qk, self.taps), init="taps"),
                  n["k"] + ".conv": WeightSpec((qk, self.taps), init="taps"),
                  n["v"] + ".conv": WeightSpec((vv, self.taps), init="taps")})
        return w

    def load(self, get):
        n = self.names
        parts = [get(n[x]) for x in ("q", "k", "v")] + [get(n["g1"] if self.gate_rank else n["gate"])]
        if self.a_rank:
            parts.append(get(n["a1"]))
        ranks = (parts[3].shape[0] if self.gate_rank else 0, parts[4].shape[0] if self.a_rank else 0)
        if self.gate_rank and get(n["g2"]).shape[1] != ranks[0] or self.a_rank and get(n["a2"]).shape[1] != ranks[1]:
            raise ValueError("the two products of a low-rank input disagree in their inner width")
        if ranks != (self.gate_rank, self.a_rank):
            self.gate_rank, self.a_rank = ranks
            self._layout()
        dt = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        w_proj = torch.zeros(self.proj_width, self.hidden, dtype=dt, device=parts[0].device)
        w_proj[:self.channels] = torch.cat([p.to(dt) for p in parts[:3]], dim=0)
        w_proj[self.gate_col:self.gate_col + self.gate_cols] = parts[3].to(dt)
        if self.a_rank:
            w_proj[self.a_col:self.a_col + self.a_rank] = parts[4].to(dt)
            # the decay's second product reads the padded inner values: columns of zeros for the padding
            a2 = get(n["a2"])
            self.w_a2 = torch.zeros(a2.shape[0], self.proj_width - self.a_col, dtype=a2.dtype, device=a2.device)
            self.w_a2[:, :self.a_rank] = a2
            self.w_ba = get(n["beta"]).contiguous()
        else:
            self.w_ba = torch.cat([get(n["beta"]), get(n["a"])], dim=0).contiguous()
        if self.gate_rank:
            g2 = get(n["g2"])
            self.w_g2 = torch.zeros(g2.shape[0], self.a_col - self.gate_col if self.a_rank else self.proj_width - self.gate_col,
                                    dtype=g2.dtype, device=g2.device)
            self.w_g2[:, :self.gate_rank] = g2
        self.w_proj = w_proj.contiguous()
        self.w_o = get(n["o"]).contiguous()
        self.conv_w = torch.cat([get(n[x] + ".conv").float() for x in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = get(n["A_log"]).float().contiguous()
        self.dt_bias = get(n["dt_bias"]).float().contiguous()
        self.norm_w = get(n["norm"]).float().contiguous()

    def forward(self, x, batch, cache, writes_cache=True, then=None):
        T = x.shape[0]
        ws = self.ctx.workspace
        state = cache[0]
        conv_state = cache[1] if self.taps > 1 else state        # unused without taps to carry
        H, hw = self.nh, self.nh * self.dw
        proj = linear(x, self.w_proj, ws.get("delta_proj", T, self.proj_width))
        if self.a_rank:
            # beta straight from x; the decay's input through its two products (the inner values are columns of proj)
            ba = ws.get("delta_ba", T, H + hw)
            zb = linear(x, self.w_ba, ba.view(-1)[:T * H].view(T, H))
            za = linear(proj[:, self.a_col:], self.w_a2, ba.view(-1)[T * H:].view(T, hw))
        else:
            ba = linear(x, self.w_ba, ws.get("delta_ba", T, H + hw))
            zb, za = ba[:, :H], ba[:, H:]
        qkv = ws.get("delta_qkv", T, self.channels)
        beta, decay = ws.get("delta_beta", T, H), ws.get("delta_decay", T, hw)
        B = batch.num_seqs
        ops.delta_prep(proj, self.conv_w, conv_state, zb, za, self.a_log, self.dt_bias, batch.cu_q_lens, batch.context_lens,
                       batch.state_slots, B, self.nkv, self.nh, self.d, self.dv, qkv, beta, decay)
        o = ws.get("delta_o", T, self.nh * self.dv)
        ops.delta_recur(qkv, beta, decay, state, batch.cu_q_lens, batch.context_lens, batch.state_slots, B,
                        self.nkv, self.nh, self.d, self.dv, o)
        y = ws.get("delta_y", T, self.nh * self.dv)
        if self.gate_rank:
            gate = linear(proj[:, self.gate_col:self.a_col if self.a_rank else self.proj_width], self.w_g2,
                          ws.get("delta_gate", T, self.nh * self.dv))
        else:
            gate = proj[:, self.gate_col:self.gate_col + self.gate_cols]
        ops.delta_out(o, gate, self.norm_w, self.eps, self.nh, self.dv, y, self.gate_act)
        return linear(y, self.w_o, ws.get(self.out_buffer, T, self.hidden), then)


register_mixer("gated_delta", GatedDeltaRule)
