"""The SiLU-gated feed-forward: down( silu(x Wg^T) * (x Wu^T) ), no biases
(kernels/gollmgo_model.cu:746-776, kernels/gollmgo_ops.cu:361-374).  Gate and up
weights are stacked so one product makes both.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import WeightSpec
from .linear import NormedRows, fuses_norms, linear, use_mid_m, use_tc
from .registry import register_feed_forward


class GatedMLP:
    """params: hidden_size, intermediate_size, activation, names (optional: the local names of the
    gate, up and down tensors; default the Llama checkpoint's).  Activations: "silu" = silu(gate) * up;
    "clamped_swish" = g * sigmoid(alpha * g) * (u + shift) with g = min(gate, limit) and u = clamp(up,
    -limit, limit) (params limit, alpha = 1.702, shift = 1); "relu" and "gelu_tanh" = act(gate) * up.
    ``bias``: the three products have biases (tensors name + ".b"); ``defer_output_bias``: the last one's is
    left in ``deferred_bias`` for a block that adds it with the stream."""

    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        act = spec.get("activation", "silu")
        if act not in ("silu", "clamped_swish", "relu", "gelu_tanh"):
            raise ValueError(f"activation {act!r} is not supported (known: silu, clamped_swish, relu, gelu_tanh)")
        self.bias = bool(spec.get("bias", False))
        if self.bias and act == "clamped_swish":
            raise ValueError("the clamped activation takes no biases")
        self.defer_bias = bool(spec.get("defer_output_bias", False))
        self.b_gate_up = self.b_down = self.deferred_bias = None
        self.activation = act
        if act == "clamped_swish":
            self.limit = float(spec["limit"])
            self.alpha = float(spec.get("alpha", 1.702))
            self.shift = float(spec.get("shift", 1.0))
        self.names = tuple(spec.get("names") or ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("gate_up", T * 2 * self.inter, ctx.act_dtype)
        ws.reserve("ffn_act", T * self.inter, ctx.act_dtype)
        ws.reserve("ffn_out", T * self.hidden, ctx.act_dtype)
        self.w_gate_up = None
        self.w_down = None

    def weights(self):
        g, u, d = self.names
        w = {g: WeightSpec((self.inter, self.hidden)),
             u: WeightSpec((self.inter, self.hidden)),
             d: WeightSpec((self.hidden, self.inter))}
        if self.bias:
            w.update({g + ".b": WeightSpec((self.inter,), init="normal"), u + ".b": WeightSpec((self.inter,), init="normal"),
                      d + ".b": WeightSpec((self.hidden,), init="normal")})
        return w

    def load(self, get):
        g, u = get(self.names[0]), get(self.names[1])
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = get(self.names[2]).contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([get(self.names[0] + ".b").float(), get(self.names[1] + ".b").float()]).contiguous()
            self.b_down = get(self.names[2] + ".b").float().contiguous()
            self.deferred_bias = self.b_down if self.defer_bias else None

    # the optional protocol of parts/linear.py: the first product can take a norm's unnormalised
    # input, the last one can do the residual add and prepare the next norm
    def takes_normed_rows(self, num_tokens):
        return self.activation == "silu" and not self.bias and fuses_norms(num_tokens, self.w_gate_up, self.ctx.act_dtype)

    def fuses_next_norm(self, num_tokens):
        return not self.bias and fuses_norms(num_tokens, self.w_down, self.ctx.act_dtype)

    def forward(self, x, batch, then=None):
        T = x.shape[0]
        ws = self.ctx.workspace
        a = ws.get("ffn_act", T, self.inter)
        if self.activation == "clamped_swish":
            if self.limit > 0 and ops.small_m_ok(x, self.w_gate_up):
                ops.gemm_small_m_clamped(x, self.w_gate_up, a, self.limit, self.alpha, self.shift)   # product and activation in one
            else:
                gu = linear(x, self.w_gate_up, ws.get("gate_up", T, 2 * self.inter))
                ops.clamped_gate(gu, a, self.limit, self.alpha, self.shift)
        elif self.bias or self.activation != "silu":
            gu = linear(x, self.w_gate_up, ws.get("gate_up", T, 2 * self.inter))
            ops.gated_act(gu, self.b_gate_up, a, self.activation)
        elif isinstance(x, NormedRows):
            ops.gemm_small_m(x.scaled, self.w_gate_up, a, gated=True, in_partials=x.partials,
                             hidden=x.hidden, eps=x.eps)
        elif ops.small_m_ok(x, self.w_gate_up):
            ops.gemm_small_m(x, self.w_gate_up, a, gated=True)       # product and activation in one
        elif use_mid_m(x, self.w_gate_up, gated=True):
            ops.gemm_mid_m(x, self.w_gate_up, a, gated=True)          # the same for a few dozen tokens
        elif use_tc(x, self.w_gate_up, self.inter, True):
            ops.gemm_tc(x, self.w_gate_up, a, gated=True, pair=True)  # the same, on tcgen05 (CTA pairs)
        else:
            gu = ws.get("gate_up", T, 2 * self.inter)
            linear(x, self.w_gate_up, gu)
            ops.silu_mul(gu, a)
        y = ws.get("ffn_out", T, self.hidden)
        if self.bias:
            linear(a, self.w_down, y)
            if not self.defer_bias:
                ops.bias_add(y, self.b_down)
            return y
        return linear(a, self.w_down, y, then)


class PlainMLP:
    """down(act(up(x))), no gate, no biases.  params: hidden_size, intermediate_size, activation
    ("relu2" = the square of relu, "gelu_tanh", "silu"), names (local names of the up and down
    tensors)."""

    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.activation = spec.get("activation", "relu2")
        if self.activation not in ops.ACT_KINDS:
            raise ValueError(f"activation {self.activation!r} is not supported (known: {sorted(ops.ACT_KINDS)})")
        self.names = tuple(spec.get("names") or ("up", "down"))
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("ffn_up", T * self.inter, ctx.act_dtype)
        ws.reserve("ffn_out", T * self.hidden, ctx.act_dtype)
        self.w_up = None
        self.w_down = None

    def weights(self):
        return {self.names[0]: WeightSpec((self.inter, self.hidden)),
                self.names[1]: WeightSpec((self.hidden, self.inter))}

    def load(self, get):
        self.w_up = get(self.names[0]).contiguous()
        self.w_down = get(self.names[1]).contiguous()

    def forward(self, x, batch):
        T = x.shape[0]
        ws = self.ctx.workspace
        u = ws.get("ffn_up", T, self.inter)
        linear(x, self.w_up, u)
        ops.act(u, u, self.activation)
        return linear(u, self.w_down, ws.get("ffn_out", T, self.hidden))


register_feed_forward("gated_mlp", GatedMLP)
register_feed_forward("mlp", PlainMLP)
