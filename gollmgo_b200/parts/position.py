"""Position encodings.  "rope": rotary, inverse frequencies from theta with the
optional llama3 or linear scaling of config.json's ``rope_scaling``; "none".

The reference rotates with f_p = theta^(-2p/d), theta fixed at 10000 and no
scaling (kernels/gollmgo_ops.cu:337, kernels/gollmgo_model.cu:603).  The table is
built once on the host in float64 and handed to the kernel that rotates q and k
and writes the cache.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..csrc import ops
from ..weights import WeightSpec
from .registry import register_position


def inverse_frequencies(rot: int, theta: float, scaling) -> torch.Tensor:
    p = torch.arange(0, rot, 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(theta, dtype=torch.float64), -p / rot)
    if scaling is None:
        return f
    if scaling.rope_type == "yarn":
        # Frequencies whose wave turns fewer than `slow` times over the original length are divided by
        # the factor, those that turn more than `fast` times are kept, and a linear ramp over the pair
        # index joins the two: with turns(i) = original * f_i / (2 pi), the pair index at which a wave
        # makes t turns is rot * ln(original / (2 pi t)) / (2 ln theta).
        def index_of(turns):
            return rot * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
        lo = max(math.floor(index_of(scaling.fast)), 0)
        hi = min(math.ceil(index_of(scaling.slow)), rot - 1)
        i = torch.arange(0, rot // 2, dtype=torch.float64)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / scaling.factor * ramp + f * (1.0 - ramp)
    if scaling.rope_type == "linear":
        return f / scaling.factor
    if scaling.rope_type == "llama3":
        orig = float(scaling.original_max_position_embeddings)
        lo_wl = orig / scaling.low_freq_factor        # longer than this: slowed by factor
        hi_wl = orig / scaling.high_freq_factor       # shorter than this: kept
        wl = 2.0 * math.pi / f
        smooth = (orig / wl - scaling.low_freq_factor) / (scaling.high_freq_factor - scaling.low_freq_factor)
        blended = (1.0 - smooth) * f / scaling.factor + smooth * f
        return torch.where(wl < hi_wl, f, torch.where(wl > lo_wl, f / scaling.factor, blended))
    raise ValueError(f"rope scaling {scaling.rope_type!r} is not supported")


@dataclass(frozen=True)
class YarnScaling:
    """Stretching of a rotary table for contexts beyond the ``original`` length by ``factor``:
    slow waves are slowed, fast ones kept, and every cosine and sine grows by 0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float
    rope_type: str = "yarn"

    @property
    def magnitude(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0


class RotaryEncoding:
    """params: head_dim, theta, scaling (config.RopeScaling, YarnScaling or None), interleaved,
    rotary_dim (defaults to head_dim).  ``magnitude`` is a factor on every cosine and sine (1 unless
    the scaling says otherwise); only the kernels of the general attention path apply it."""

    def __init__(self, spec, ctx):
        self.head_dim = int(spec["head_dim"])
        self.rot = int(spec.get("rotary_dim") or self.head_dim)
        if self.rot % 2 or self.rot > self.head_dim:
            raise ValueError(f"rotary width {self.rot} must be even and at most {self.head_dim}")
        self.interleaved = bool(spec.get("interleaved", False))
        self.magnitude = float(getattr(spec.get("scaling"), "magnitude", 1.0))
        self._table = inverse_frequencies(self.rot, float(spec["theta"]), spec.get("scaling")) \
            .to(ctx.device).contiguous()

    def rope_table(self):
        return self._table


class NoPositionEncoding:
    interleaved = False

    def __init__(self, spec, ctx):
        pass

    def rope_table(self):
        return None


class LearnedPositions:
    """A table of learned position vectors that is added to the embedded tokens (named in
    ``ModelSpec.embed_position``): x <- x * scale + table[position].  params: hidden_size,
    max_positions.  Its one tensor: "" (the prefix alone), [max_positions, hidden_size]."""
    interleaved = False

    def __init__(self, spec, ctx):
        self.hidden = int(spec["hidden_size"])
        self.max_positions = int(spec["max_positions"])
        self.table = None
        self.bad = torch.zeros(1, dtype=torch.int32, device=ctx.device) if ctx.device.type == "cuda" else None

    def rope_table(self):
        return None

    def weights(self):
        return {"": WeightSpec((self.max_positions, self.hidden))}

    def load(self, get):
        self.table = get("").contiguous()

    def add_to_embedding(self, resid, batch, scale: float = 1.0):
        ops.scale_add_rows(resid, scale, self.table, batch.positions, self.bad)


register_position("learned", LearnedPositions)
register_position("rope", RotaryEncoding)
register_position("none", NoPositionEncoding)
