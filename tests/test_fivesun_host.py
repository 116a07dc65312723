"""Fivesun without a device: the configuration (every key, absent keys, wrong values), the manifest against the
tensor names of a checkpoint, the rotation tables against the plain implementation, and the run of the spec."""
import copy

import numpy as np
import pytest
import torch

import fivesun_tools as ft
import plain_fivesun as P
from gollmgo_b200.config import ConfigError, resolve_architecture
from gollmgo_b200.config.fivesun_config import (FivesunConfig, MatrixMemoryConfig, NormedAttentionConfig,
                                                RotatedLatentConfig)
from gollmgo_b200.parts.model import manifest_for_config
from gollmgo_b200.parts.position import inverse_frequencies


@pytest.mark.parametrize("name", sorted(ft.TINY))
def test_manifest_is_the_checkpoint(name):
    cfg, _ = ft.get(name)
    manifest = manifest_for_config(cfg)
    assert {k: tuple(v.shape) for k, v in manifest.items()} == ft.tensor_shapes(cfg)


def test_every_key_is_read():
    cfg, _ = ft.get("fiv_a")
    c = FivesunConfig.from_dict(cfg)
    assert (c.vocab, c.width, c.eps, c.embed_scale, len(c.layers)) == (203, 64, 1e-5, 8.0, 5)
    lat, att, mem = c.layers[0].mixer, c.layers[1].mixer, c.layers[2].mixer
    assert isinstance(lat, RotatedLatentConfig) and isinstance(att, NormedAttentionConfig) and isinstance(mem, MatrixMemoryConfig)
    assert (lat.heads, lat.dim, lat.rot_dim, lat.vdim, lat.kv_rank, lat.scale, lat.window) == (3, 16, 8, 24, 24, 0.2, 20)
    assert (lat.rot.base, lat.rot.dims, lat.rot.factor, lat.rot.blend) == (10000.0, 8, 4.0, (64.0, 16.0, 1.0))
    assert (att.heads, att.kv_heads, att.dim, att.vdim, att.scale, att.chunk, att.v_mix) == (4, 2, 32, 16, 0.16, 24, True)
    assert (att.rot.dims, att.rot.factor, att.rot.blend) == (16, 2.0, None)
    assert (mem.heads, mem.dim, mem.vdim, mem.gate_cap) == (2, 16, 24, 8.0)
    assert c.layers[3].mlp is None and c.layers[0].mlp.ff == 40
    assert c.layers[4].mixer.rot.factor is None and not c.layers[4].mixer.v_mix


def test_absent_keys_switch_their_feature_off():
    cfg, _ = ft.get("fiv_c")
    c = FivesunConfig.from_dict(cfg)
    assert c.layers[3].mixer.chunk is None and c.layers[4].mixer.window is None
    del cfg["embedding"]
    del cfg["layers"][0]["mixer"]["rot"]
    c = FivesunConfig.from_dict(cfg)
    assert c.embed_scale == 1.0 and c.layers[0].mixer.rot is None
    spec = resolve_architecture(cfg).spec(c)
    assert spec.layers[0].mixer["position"].kind == "none" and spec.embed_scale == 1.0


def test_the_spec_names_the_first_blending_layer():
    cfg, _ = ft.get("fiv_a")
    spec = resolve_architecture(cfg).spec(FivesunConfig.from_dict(cfg))
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "normed_attention", "mlstm", "normed_attention",
                                                   "normed_attention"]
    assert [l.mixer.get("v_mix") for l in spec.layers] == [None, "first", None, "blend", None]
    assert [l.mixer.get("chunk") for l in spec.layers[1:]] == [24, None, 24, 40]
    assert spec.layers[3].feed_forward is None and spec.layers[3].ffn_norm is None
    assert all(l.block.kind == "sandwich" for l in spec.layers)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=15), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34), "at most"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot_dim"),
    (lambda c: c["layers"][2]["mixer"].update(gate_cap=0), "gate_cap"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=24), "agree"),
    (lambda c: c["layers"][0].update(mlp={"kind": "moe"}), "dense"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "positive"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_wrong_values_are_refused(change, message):
    cfg, _ = ft.get("fiv_a")
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        FivesunConfig.from_dict(cfg)


@pytest.mark.parametrize("name", sorted(ft.TINY))
def test_rotation_tables_match_the_plain_ones(name):
    cfg, _ = ft.get(name)
    spec = resolve_architecture(cfg).spec(FivesunConfig.from_dict(cfg))
    for lc, ls in zip(cfg["layers"], spec.layers):
        rot = lc["mixer"].get("rot")
        if rot is None:
            continue
        pos = ls.mixer["position"]
        f = inverse_frequencies(pos["rotary_dim"], pos["theta"], pos["scaling"]).numpy()
        want, mag = P.rotary_frequencies(rot)
        assert np.allclose(f, want, rtol=1e-14, atol=0)
        assert abs(float(getattr(pos["scaling"], "magnitude", 1.0)) - mag) < 1e-15
        assert pos["interleaved"] is True
