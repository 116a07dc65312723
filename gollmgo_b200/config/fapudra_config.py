"""Typed configuration of the Fapudra decoder, read from its config.json.

The file names the design in ``architecture`` and lists the layers one by one: each entry has
``type`` (its mixer: "mamba2" = a state-space layer, "parallel" = a sigmoid attention and a delta
rule with a decay per key channel side by side), the mixer's sizes and constants in ``mixer`` and
its feed-forward in ``mlp`` (a mixture of experts, or null).  ``embedding.scale`` multiplies the
embedded tokens, ``max_positions`` is the length of the learned position table, ``norm.eps`` the
one epsilon, ``logit_softcap`` the cap of the logits (absent or 0: none).  Every size and constant
is taken from the file; three sizes are the checkpoint's tensors' (the rows of the distance table of
the attention, the inner widths of the delta rule's decay and gate): the optional keys ``bias_rows``,
``a_rank`` and ``gate_rank`` only say what random weights are made with.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .model_config import ConfigError
from .tekenex_config import _int, _num, _only


@dataclass(frozen=True)
class Mamba2Config:
    heads: int
    vdim: int            # values of a head
    state: int           # rows of a head's state matrix
    groups: int          # heads of one group share B and C
    conv: int            # taps of the short convolution
    norm_groups: int     # parts of the gated output that are normed on their own


@dataclass(frozen=True)
class SigmoidBranchConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: int                    # distance from which every key falls into the last bucket
    bias_rows: int                   # rows of the distance table where random weights are made (a checkpoint's tensor decides)
    window: Optional[int]            # None: every earlier key is seen
    keep_first: int                  # the first tokens stay visible behind the window


@dataclass(frozen=True)
class ChannelDeltaBranchConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    a_rank: int          # inner widths of the decay's and the gate's two products where random weights
    gate_rank: int       # are made (a checkpoint's tensors decide)


@dataclass(frozen=True)
class FapudraParallelConfig:
    left: SigmoidBranchConfig
    right: ChannelDeltaBranchConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class FapudraMoeConfig:
    ff: int
    limit: float
    experts: int
    top: int
    group_count: int
    group_keep: int


@dataclass(frozen=True)
class FapudraLayerConfig:
    type: str
    mixer: object                                # Mamba2Config | FapudraParallelConfig
    mlp: Optional[FapudraMoeConfig]


@dataclass(frozen=True)
class FapudraConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_softcap: float                         # 0 = none
    max_positions: int
    layers: Tuple[FapudraLayerConfig, ...]
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None

    @staticmethod
    def from_dict(d: dict) -> "FapudraConfig":
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' (with 'eps') is missing")
        eps = _num(norm, "eps", "norm")
        if eps < 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {eps}")
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            _only(e, ("type", "mixer", "mlp"), where)
            kind, m = e.get("type"), e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            if kind == "mamba2":
                mixer = _mamba2(m, where + ".mixer")
            elif kind == "parallel":
                _only(m, ("left", "right", "left_scale", "right_scale"), where + ".mixer")
                if not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                    raise ConfigError(f"config.json: {where}.mixer needs 'left' and 'right'")
                mixer = FapudraParallelConfig(_sigmoid_branch(m["left"], where + ".mixer.left"),
                                              _delta_branch(m["right"], where + ".mixer.right"),
                                              _num(m, "left_scale", where + ".mixer") if "left_scale" in m else 1.0,
                                              _num(m, "right_scale", where + ".mixer") if "right_scale" in m else 1.0)
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not known (known: mamba2, parallel)")
            layers.append(FapudraLayerConfig(kind, mixer, _moe(e.get("mlp"), where + ".mlp")))
        emb = d.get("embedding") or {}
        if not isinstance(emb, dict):
            raise ConfigError("config.json: 'embedding' must be an object")
        cap = d.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap < 0):
            raise ConfigError(f"config.json: logit_softcap must be a number >= 0 or null, got {cap!r}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return FapudraConfig(vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"), eps=eps,
                             embedding_scale=_num(emb, "scale", "embedding") if "scale" in emb else 1.0,
                             logit_softcap=float(cap or 0.0), max_positions=_int(d, "max_positions", "config"),
                             layers=tuple(layers), eos_token_ids=eos_ids, bos_token_id=d.get("bos_token_id"))


def _mamba2(m: dict, where: str) -> Mamba2Config:
    _only(m, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), where)
    heads, groups = _int(m, "heads", where), _int(m, "groups", where) if "groups" in m else 1
    if heads % groups:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {groups} groups")
    vdim = _int(m, "vdim", where)
    parts = _int(m, "norm_groups", where) if "norm_groups" in m else 1
    if (heads * vdim) % parts:
        raise ConfigError(f"config.json: {where}: {heads * vdim} inner values do not split into {parts} norm_groups")
    return Mamba2Config(heads, vdim, _int(m, "state", where), groups, _int(m, "conv", where), parts)


def _heads(m: dict, where: str):
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
    return heads, kv, _int(m, "dim", where), _int(m, "vdim", where)


def _sigmoid_branch(m: dict, where: str) -> SigmoidBranchConfig:
    _only(m, ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max", "bias_rows", "mask"), where)
    heads, kv, dim, vdim = _heads(m, where)
    if vdim != dim:
        raise ConfigError(f"config.json: {where}: the values are the keys, so vdim {vdim} must equal dim {dim}")
    window, keep = None, 0
    mask = m.get("mask")
    if mask is not None:
        if not isinstance(mask, dict):
            raise ConfigError(f"config.json: {where}.mask must be an object or null")
        _only(mask, ("size", "keep_first"), where + ".mask")
        window = _int(mask, "size", where + ".mask")
        k = mask.get("keep_first", 0)
        if isinstance(k, bool) or not isinstance(k, int) or k < 0:
            raise ConfigError(f"config.json: {where}.mask.keep_first must be an integer >= 0, got {k!r}")
        keep = k
    rows = _int(m, "bias_rows", where) if "bias_rows" in m else 32
    return SigmoidBranchConfig(heads, kv, dim, vdim, _num(m, "scale", where), _int(m, "bias_max", where), rows, window, keep)


def _delta_branch(m: dict, where: str) -> ChannelDeltaBranchConfig:
    _only(m, ("heads", "kv_heads", "dim", "vdim", "conv", "a_rank", "gate_rank"), where)
    heads, kv, dim, vdim = _heads(m, where)
    return ChannelDeltaBranchConfig(heads, kv, dim, vdim, _int(m, "conv", where),
                                    _int(m, "a_rank", where) if "a_rank" in m else 16,
                                    _int(m, "gate_rank", where) if "gate_rank" in m else 16)


def _moe(f, where: str) -> Optional[FapudraMoeConfig]:
    if f is None:
        return None
    if not isinstance(f, dict):
        raise ConfigError(f"config.json: {where} must be an object or null")
    if f.get("kind", "moe") != "moe":
        raise ConfigError(f"config.json: {where}.kind {f.get('kind')!r} is not known (known: moe)")
    _only(f, ("kind", "router", "expert"), where)
    r, ex = f.get("router"), f.get("expert")
    if not isinstance(r, dict) or not isinstance(ex, dict):
        raise ConfigError(f"config.json: {where} needs 'router' and 'expert'")
    _only(r, ("experts", "top", "groups"), where + ".router")
    _only(ex, ("ff", "limit"), where + ".expert")
    experts, top = _int(r, "experts", where + ".router"), _int(r, "top", where + ".router")
    count, keep = 1, 1
    g = r.get("groups")
    if g is not None:
        if not isinstance(g, dict):
            raise ConfigError(f"config.json: {where}.router.groups must be an object or null")
        _only(g, ("count", "keep"), where + ".router.groups")
        count, keep = _int(g, "count", where + ".router.groups"), _int(g, "keep", where + ".router.groups")
    if experts % count or keep > count:
        raise ConfigError(f"config.json: {where}.router: {experts} experts in {count} groups of which {keep} are kept")
    if top > keep * (experts // count):
        raise ConfigError(f"config.json: {where}.router: {top} choices from {keep} groups of {experts // count} experts")
    return FapudraMoeConfig(_int(ex, "ff", where + ".expert"), _num(ex, "limit", where + ".expert"), experts, top,
                            count, keep)
