"""Fapudra without a device: registry and typed configuration, refused configurations, the manifest
against the design's naming rules, sizes that the checkpoint decides, the table of distance buckets,
pages with kept first tokens in the cache manager, and properties of the plain implementation
(causality, the window with its kept tokens, the grouped choice of experts)."""
import copy

import numpy as np
import pytest
import torch

import fapudra_tools as ft
import plain_fapudra as P


def test_registry_and_typed_config():
    from gollmgo_b200 import architectures  # noqa: F401
    from gollmgo_b200.config import resolve_architecture
    cfg, _ = ft.get("fap_a")
    arch = resolve_architecture(cfg)
    assert arch.name == "Fapudra"
    c = arch.parse(cfg)
    assert (c.vocab, c.width, c.eps, c.embedding_scale, c.logit_softcap, c.max_positions) == (203, 64, 1e-5, 8.0, 12.0, 512)
    left = c.layers[0].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.window, left.keep_first, left.bias_max) == (4, 2, 16, 40, 3, 60)
    assert (c.layers[0].mlp.group_count, c.layers[0].mlp.group_keep, c.layers[0].mlp.top) == (3, 2, 2)
    assert c.layers[2].mlp is None and c.layers[1].mixer.norm_groups == 2 and c.layers[1].mixer.groups == 2
    b = arch.parse(ft.get("fap_b")[0])
    assert b.logit_softcap == 0.0 and b.embedding_scale == 1.0
    assert b.layers[2].mixer.left.window is None and b.layers[2].mixer.left.keep_first == 0
    assert (b.layers[1].mlp.group_count, b.layers[1].mlp.group_keep) == (1, 1)
    spec = arch.spec(c)
    assert spec.embed_scale == 8.0 and spec.logit_softcap == 12.0 and spec.embed_norm.params["scalar"]
    assert [l.mixer.kind for l in spec.layers] == ["token_shift"] * 4
    assert [l.mixer.params["inner"].kind for l in spec.layers] == ["parallel", "mamba2", "parallel", "mamba2"]


def _broken():
    def edit(f):
        cfg, _ = ft.get("fap_a")
        f(cfg)
        return cfg
    return [
        edit(lambda c: c["layers"][0]["mixer"]["left"].update(vdim=24)),                    # the values are the keys
        edit(lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3)),
        edit(lambda c: c["layers"][0]["mixer"]["right"].update(kv_heads=3)),
        edit(lambda c: c["layers"][1].update(type="conv")),
        edit(lambda c: c["layers"][1]["mixer"].update(groups=3)),
        edit(lambda c: c["layers"][1]["mixer"].update(norm_groups=5)),
        edit(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4)),            # 6 experts in 4 groups
        edit(lambda c: c["layers"][0]["mlp"]["router"].update(top=5)),                        # more than the kept groups hold
        edit(lambda c: c["layers"][0]["mlp"].update(kind="dense")),
        edit(lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=-1)),
        edit(lambda c: c.pop("norm")),
        edit(lambda c: c.pop("max_positions")),
        edit(lambda c: c.update(logit_softcap=-1.0)),
    ]


@pytest.mark.parametrize("i", range(13))
def test_broken_configurations_are_refused(i):
    from gollmgo_b200 import architectures  # noqa: F401
    from gollmgo_b200.config import ConfigError, resolve_architecture
    cfg = _broken()[i]
    with pytest.raises(ConfigError):
        resolve_architecture(cfg).parse(cfg)


@pytest.mark.parametrize("name", sorted(ft.TINY))
def test_manifest_follows_the_naming_rules(name):
    from gollmgo_b200.parts import manifest_for_config
    cfg, _ = ft.get(name)
    manifest = manifest_for_config(cfg)
    want = ft.tensor_shapes(cfg)
    assert set(manifest) == set(want)
    assert {k: tuple(v.shape) for k, v in manifest.items()} == want


def test_sizes_that_the_checkpoint_decides():
    """The rows of the distance table and the inner widths of the low-rank products are not in
    config.json: a checkpoint that differs from the defaults in them fits, one that differs elsewhere
    does not."""
    from gollmgo_b200.parts import manifest_for_config
    from gollmgo_b200.weights.loader import WeightError, check_manifest
    cfg, _ = ft.get("fap_a")
    bare = copy.deepcopy(cfg)
    for layer in bare["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"].pop("bias_rows")
            layer["mixer"]["right"].pop("a_rank")
            layer["mixer"]["right"].pop("gate_rank")
    manifest = manifest_for_config(bare)
    found = {k: (v, torch.bfloat16) for k, v in ft.tensor_shapes(cfg).items()}
    check_manifest(manifest, found)
    found["l0.mix.left.rel"] = ((12, 5), torch.bfloat16)
    with pytest.raises(WeightError):
        check_manifest(manifest, found)


@pytest.mark.parametrize("rows,far", [(12, 60), (32, 120), (8, 33), (40, 250), (16, 17), (2, 5), (24, 48), (28, 128)])
def test_distance_buckets(rows, far):
    from gollmgo_b200.parts.sigmoid_attention import distance_buckets
    table = distance_buckets(rows, far).tolist()
    assert table == [P.distance_bucket(n, rows, far) for n in range(far + 1)]
    assert table[far] == rows - 1 and P.distance_bucket(10 * far, rows, far) == rows - 1
    assert table[:rows // 2] == list(range(rows // 2)) and all(b >= a for a, b in zip(table, table[1:]))
    with pytest.raises(ValueError):
        distance_buckets(rows, rows // 2)


def test_pages_of_kept_first_tokens_stay():
    from gollmgo_b200.cache import CacheManager, PagedKVNeed
    page = 8
    needs = [PagedKVNeed(2, 16, window=20, shared_kv=True, keep_first=11), PagedKVNeed(2, 16, window=20, shared_kv=True),
             PagedKVNeed(1, 8, window=6, keep_first=1)]
    cm = CacheManager(needs, page, 12, 2)
    assert len(cm.groups) == 3                       # a group per need: kept tokens make a need of its own
    cm.admit("a")
    for n in (30, 1, 1, 7, 25, 2):
        cm.append("a", n)
        cm.audit()
    held = cm.requests["a"].pages
    total = cm.num_tokens("a")
    first_needed = total - 20 + 1
    for idx, p in enumerate(held[0]):
        behind = (idx + 1) * page <= first_needed
        assert (p >= 0) == (not behind or idx < 2), (idx, p)      # 11 kept tokens lie in pages 0 and 1
    assert all((p >= 0) == ((idx + 1) * page > first_needed) for idx, p in enumerate(held[1]))
    assert held[2][0] >= 0 and held[2][1] < 0
    # what a scheduler plans with says the same
    assert cm.pages_held("a")[0] == sum(p >= 0 for p in held[0])
    cm.free("a")
    cm.audit()
    assert cm.free_pages_per_group() == [12, 12, 12]


def _one_layer(kind):
    cfg, _ = ft.get("fap_a")
    cfg["layers"] = [cfg["layers"][0 if kind == "parallel" else 1]]
    return cfg


def test_plain_model_is_causal_and_sees_what_the_mask_says():
    cfg = _one_layer("parallel")
    cfg["layers"][0]["mixer"]["right_scale"] = 0.0            # the attention alone (the recurrent branch sees everything)
    cfg["layers"][0]["mlp"] = None
    w = ft.as_numpy(ft.random_weights(cfg, 3))
    w["l0.shift"][:] = 0.0                                    # no look at the token before through the shift
    rng = np.random.default_rng(0)
    toks = rng.integers(0, cfg["vocab"], 120)
    base = P.forward(cfg, w, toks)
    other = toks.copy()
    other[60] = (other[60] + 1) % cfg["vocab"]
    d = np.abs(P.forward(cfg, w, other) - base).max(-1)
    assert d[:60].max() == 0 and d[60] > 0
    assert d[60 + 39] > 0 and d[60 + 40:].max() == 0          # a window of 40: seen by 39 more tokens, then gone
    kept = toks.copy()
    kept[2] = (kept[2] + 1) % cfg["vocab"]                    # one of the 3 kept first tokens: seen for ever
    assert np.abs(P.forward(cfg, w, kept) - base).max(-1)[100:].min() > 0
    fourth = toks.copy()
    fourth[3] = (fourth[3] + 1) % cfg["vocab"]                # the next one is not
    assert np.abs(P.forward(cfg, w, fourth) - base).max(-1)[3 + 40:].max() == 0


def test_plain_choice_of_experts_respects_the_groups():
    rng = np.random.default_rng(1)
    h, wr = rng.normal(size=(200, 16)), rng.normal(size=(12, 16))
    r = {"experts": 12, "top": 3, "groups": {"count": 4, "keep": 2}}
    gaps = []
    idx, wgt = P.route(h, wr, r, gaps)
    z = h @ wr.T
    for t in range(200):
        best = sorted(range(4), key=lambda g: -z[t, 3 * g:3 * g + 3].max())[:2]
        assert all(i // 3 in best for i in idx[t])
        allowed = sorted((e for g in best for e in range(3 * g, 3 * g + 3)), key=lambda e: -z[t, e])[:3]
        assert list(idx[t]) == allowed
    assert np.allclose(wgt.sum(-1), 1.0) and (gaps[0] >= 0).all()
    free = P.route(h, wr, {"experts": 12, "top": 3})[0]
    assert any(set(a) != set(b) for a, b in zip(free, idx))   # the groups change some choices


def test_cache_needs_of_the_model():
    from gollmgo_b200.cache import FixedStateNeed, PagedKVNeed
    from gollmgo_b200.config import resolve_architecture
    from gollmgo_b200.parts import BuildContext, build_model
    cfg, page = ft.get("fap_a")
    model = build_model(cfg, BuildContext(torch.float32, "cpu", 64, 4, page))[2]
    needs = model.cache_needs()
    assert len(needs) == 4
    shift, (left, right) = needs[0]
    assert shift == FixedStateNeed((64,), "float32")
    assert left == PagedKVNeed(2, 16, 40, shared_kv=True, keep_first=3)
    assert right == (FixedStateNeed((4, 24, 16), "float32"), FixedStateNeed((2, 2 * 2 * 16 + 4 * 24), "float32"))
    shift, ssm = needs[1]
    assert ssm == (FixedStateNeed((4, 16, 24), "float32"), FixedStateNeed((3, 4 * 16 + 2 * 2 * 24), "float32"))
