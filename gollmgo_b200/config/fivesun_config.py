"""Typed configuration of the Fivesun decoder, read from its config.json.

The file names the design in ``architecture`` and lists the layers one by one: each entry has ``type``
(its mixer: "attention", "latent_attention" or "mlstm"), the mixer's sizes and constants in ``mixer``, and
its feed-forward in ``mlp`` (``kind`` "dense" with ``ff``, or null for a layer without one).  ``norm.eps``
is the one epsilon of every norm, ``embedding.scale`` multiplies the embedded tokens, ``vocab`` and
``width`` are the table's sizes.  A mixer's ``rot`` gives the rotation (``base``, ``dims`` and an optional
``scaling``: ``factor`` alone divides every frequency; with ``original``, ``fast`` and ``slow`` the
frequencies are blended between divided and kept), its ``mask`` the size of the chunks (attention) or of the
sliding window (latent attention); a mixer without ``mask`` sees every earlier token.  Every size and
constant is taken from the file; a key this engine does not know inside a layer is reported on standard
error and ignored.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .model_config import ConfigError
from .tekenex_config import _int, _num, _only


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    factor: Optional[float] = None                 # frequencies divided by this (alone: every one of them)
    blend: Optional[Tuple[float, float, float]] = None     # (original, fast, slow): divided, kept or in between


@dataclass(frozen=True)
class NormedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig]
    chunk: Optional[int]                           # a query sees the keys of its own chunk of this many positions
    v_mix: bool                                    # values blended with those of the first such layer


@dataclass(frozen=True)
class RotatedLatentConfig:
    heads: int
    dim: int                                       # unrotated values of a query / key head
    rot_dim: int                                   # rotated values (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    rot: Optional[RotationConfig]
    window: Optional[int]


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class FivesunLayerConfig:
    type: str
    mixer: Union[NormedAttentionConfig, RotatedLatentConfig, MatrixMemoryConfig]
    mlp: Optional[DenseMlpConfig]


def _rotation(r, where: str, width: int) -> Optional[RotationConfig]:
    if r is None:
        return None
    if not isinstance(r, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    _only(r, ("base", "dims", "scaling"), where)
    dims, base = _int(r, "dims", where), _num(r, "base", where)
    if dims % 2 or dims > width:
        raise ConfigError(f"config.json: {where}.dims must be even and at most {width}, got {dims}")
    if base <= 1.0:
        raise ConfigError(f"config.json: {where}.base must be above 1, got {base}")
    sc = r.get("scaling")
    if sc is None:
        return RotationConfig(base, dims)
    if not isinstance(sc, dict):
        raise ConfigError(f"config.json: {where}.scaling must be an object")
    _only(sc, ("factor", "original", "fast", "slow"), where + ".scaling")
    factor = _num(sc, "factor", where + ".scaling")
    if factor <= 0:
        raise ConfigError(f"config.json: {where}.scaling.factor must be positive, got {factor}")
    if not any(k in sc for k in ("original", "fast", "slow")):
        return RotationConfig(base, dims, factor)
    blend = tuple(_num(sc, k, where + ".scaling") for k in ("original", "fast", "slow"))
    if min(blend) <= 0:
        raise ConfigError(f"config.json: {where}.scaling original, fast and slow must be positive")
    return RotationConfig(base, dims, factor, blend)


def _mask(m: dict, where: str) -> Optional[int]:
    mk = m.get("mask")
    if mk is None:
        return None
    if not isinstance(mk, dict):
        raise ConfigError(f"config.json: {where}.mask must be an object")
    _only(mk, ("size",), where + ".mask")
    return _int(mk, "size", where + ".mask")


def _mixer(kind: str, m: dict, where: str):
    if kind == "attention":
        _only(m, ("heads", "kv_heads", "dim", "vdim", "scale", "rot", "mask", "v_mix"), where)
        heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
        dim = _int(m, "dim", where)
        return NormedAttentionConfig(heads, kv, dim, _int(m, "vdim", where), _num(m, "scale", where),
                                     _rotation(m.get("rot"), where + ".rot", dim), _mask(m, where), bool(m.get("v_mix", False)))
    if kind == "latent_attention":
        _only(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot", "mask"), where)
        rot_dim = _int(m, "rot_dim", where)
        rot = _rotation(m.get("rot"), where + ".rot", rot_dim)
        if rot is None or rot.dims != rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims must equal rot_dim ({rot_dim})")
        return RotatedLatentConfig(_int(m, "heads", where), _int(m, "dim", where), rot_dim, _int(m, "vdim", where),
                                   _int(m, "kv_rank", where), _num(m, "scale", where), rot, _mask(m, where))
    if kind == "mlstm":
        _only(m, ("heads", "dim", "vdim", "gate_cap"), where)
        cap = _num(m, "gate_cap", where)
        if cap <= 0:
            raise ConfigError(f"config.json: {where}.gate_cap must be positive, got {cap}")
        return MatrixMemoryConfig(_int(m, "heads", where), _int(m, "dim", where), _int(m, "vdim", where), cap)
    raise ConfigError(f"config.json: {where[:-6]}.type {kind!r} is not known (known: attention, latent_attention, mlstm)")


@dataclass(frozen=True)
class FivesunConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    layers: Tuple[FivesunLayerConfig, ...]
    max_position_embeddings: int
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None

    @staticmethod
    def from_dict(d: dict) -> "FivesunConfig":
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' (with 'eps') is missing")
        eps = _num(norm, "eps", "norm")
        if eps < 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {eps}")
        emb = d.get("embedding") or {}
        if not isinstance(emb, dict):
            raise ConfigError("config.json: 'embedding' must be an object")
        scale = _num(emb, "scale", "embedding") if "scale" in emb else 1.0
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            _only(e, ("type", "mixer", "mlp"), where)
            m = e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            f = e.get("mlp")
            mlp = None
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp must be null or an object of kind 'dense'")
                _only(f, ("kind", "ff"), where + ".mlp")
                mlp = DenseMlpConfig(_int(f, "ff", where + ".mlp"))
            layers.append(FivesunLayerConfig(e.get("type"), _mixer(e.get("type"), m, where + ".mixer"), mlp))
        blended = [l.mixer for l in layers if isinstance(l.mixer, NormedAttentionConfig) and l.mixer.v_mix]
        if any((b.kv_heads, b.vdim) != (blended[0].kv_heads, blended[0].vdim) for b in blended):
            raise ConfigError("config.json: layers that blend their values (v_mix) must agree in kv_heads and vdim")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return FivesunConfig(vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"), eps=eps,
                             embed_scale=scale, layers=tuple(layers),
                             max_position_embeddings=int(d.get("max_position_embeddings", 1 << 17)),
                             eos_token_ids=eos_ids, bos_token_id=d.get("bos_token_id"))
