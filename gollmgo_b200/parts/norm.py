"""RMSNorm and LayerNorm, fused with the residual add that precedes them, or (norm_scale_add)
with the scaling and the residual add that follow them.

y = x * rsqrt(mean(x^2) + eps) * w in float32 (kernels/gollmgo_ops.cu:593-629);
eps comes from config.json (the reference passes the literal 1e-5:
internal/backend/cuda/model_bridge.go:53).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import WeightSpec
from .registry import register_norm


class RMSNorm:
    """params: size, eps, scalar (bool: the weight is one number for all coordinates; the kernels then
    get it repeated ``size`` times)."""

    def __init__(self, spec, ctx):
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.scalar = bool(spec.get("scalar", False))
        self.ctx = ctx
        self.weight = None

    def weights(self):
        return {"": WeightSpec(() if self.scalar else (self.size,))}

    def load(self, get):
        w = get("").to(torch.float32)
        self.weight = (w.reshape(1).expand(self.size) if self.scalar else w).contiguous()

    def norm_in_place(self, resid):
        """resid <- norm(resid) * weight, float32 rows (the kernel holds a row in shared memory before it
        writes any of it)."""
        ops.add_rmsnorm(resid, None, self.weight, resid, self.eps, None, False)

    def rms_weight_eps(self):
        """(weight, eps) for a product that folds this norm in (parts/linear.py): only a norm
        that is exactly x * rsqrt(mean(x^2) + eps) * weight may offer this."""
        return self.weight, self.eps

    def add_norm(self, resid, delta, out, rows=None, write_back=True):
        """resid (+= delta); out = norm(resid) * weight.  With ``rows`` only those rows
        are normed (out[i] from resid[rows[i]])."""
        ops.add_rmsnorm(resid, delta, self.weight, out, self.eps, rows, write_back)
        return out


    def norm_scale_add(self, resid, y, scale, copy):
        """resid += scale * norm(y); copy = resid in the activation type (a block that norms what a
        sublayer returns: parts/block.py)."""
        ops.norm_scale_add(resid, y, self.weight, None, scale, copy, self.eps, layer=False)


class LayerNorm:
    """(x - mean) / sqrt(variance + eps) * weight + bias, the variance the mean of the squared
    deviations; statistics in float32.  params: size, eps.  Its tensors: "" (weight), ".b" (bias)."""

    def __init__(self, spec, ctx):
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.ctx = ctx
        self.weight = None
        self.bias = None

    def weights(self):
        return {"": WeightSpec((self.size,)), ".b": WeightSpec((self.size,))}

    def load(self, get):
        self.weight = get("").to(torch.float32).contiguous()
        self.bias = get(".b").to(torch.float32).contiguous()

    def add_norm(self, resid, delta, out, rows=None, write_back=True):
        ops.add_norm(resid, delta, self.weight, self.bias, out, self.eps, rows, write_back, layer=True)
        return out

    def norm_scale_add(self, resid, y, scale, copy):
        ops.norm_scale_add(resid, y, self.weight, self.bias, scale, copy, self.eps, layer=True)


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
