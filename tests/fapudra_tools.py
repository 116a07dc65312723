"""Small Fapudra configurations and weights for the tests.  The configurations differ in every size,
in the order of their layers and in which optional features they have: state-space layers with one
and several groups and norm parts; sigmoid attention with windows shorter and longer than a page,
with none, one and several kept first tokens (more than a page of them too), without a mask, with
one kv head and with as many as heads, distance tables of several sizes; delta rules with fewer q/k
heads than value heads, one to five taps, inner widths that are no multiple of 8; mixtures with one
and several choices, with and without groups; a layer without feed-forward; widths that are no
multiple of 8; with and without capped logits and scaled embeddings."""
import copy
import json
import os
import random

import numpy as np
import torch


def _ssm(heads, vdim, state, groups, conv, parts):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                       "norm_groups": parts}}


def _left(heads, kv, dim, scale, far, rows, window=None, first=0):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "bias_max": far, "bias_rows": rows}
    if window:
        m["mask"] = {"size": window, "keep_first": first}
    return m


def _right(heads, kv, dim, vdim, conv, a_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "a_rank": a_rank, "gate_rank": gate_rank}


def _par(left, right, ls, rs):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}}


def _moe(ff, limit, experts, top, count=None, keep=None):
    r = {"experts": experts, "top": top}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# a parallel layer first; windows of 40 and 24 with 3 and 1 kept tokens; groups of experts 3 of which 2 are kept
FAP_A = {"architecture": "Fapudra", "vocab": 203, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
         "max_positions": 512, "logit_softcap": 12.0, "layers": [
             _layer(_par(_left(4, 2, 16, 0.25, 60, 12, window=40, first=3), _right(4, 2, 16, 24, 3, 10, 6), 0.7, 0.4),
                    _moe(40, 1.5, 6, 2, 3, 2)),
             _layer(_ssm(4, 16, 24, 2, 4, 2), _moe(48, 2.0, 4, 1)),
             _layer(_par(_left(2, 1, 32, 0.18, 100, 20, window=24, first=1), _right(2, 1, 8, 40, 4, 8, 16), 1.0, 0.6), None),
             _layer(_ssm(2, 24, 16, 1, 2, 1), _moe(32, 0.8, 8, 3, 4, 2)),
         ]}
# no capped logits, no embedding scale; a window shorter than a page and no kept tokens; no mask at all; one tap
FAP_B = {"architecture": "Fapudra", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "max_positions": 400, "layers": [
    _layer(_ssm(8, 16, 32, 4, 3, 4), _moe(64, 1.0, 4, 2, 2, 2)),
    _layer(_par(_left(4, 4, 32, 0.15, 33, 8, window=5, first=0), _right(3, 3, 32, 32, 2, 16, 24), 0.5, 0.9), _moe(72, 1.2, 5, 2)),
    _layer(_par(_left(3, 1, 24, 0.2, 250, 40), _right(4, 1, 16, 16, 1, 5, 7), 0.6, 0.5), _moe(40, 3.0, 8, 2, 2, 1)),
]}
# sizes that are no multiple of 8; more kept first tokens than a page holds; a window of exactly four pages
FAP_C = {"architecture": "Fapudra", "vocab": 150, "width": 100, "norm": {"eps": 3e-6}, "embedding": {"scale": 3.5},
         "max_positions": 300, "logit_softcap": 30.0, "layers": [
             _layer(_par(_left(6, 2, 12, 0.3, 90, 16, window=32, first=11), _right(6, 2, 20, 36, 5, 12, 9), 0.9, 0.3),
                    _moe(28, 1.0, 9, 3, 3, 1)),
             _layer(_ssm(5, 12, 20, 5, 5, 1), None),
             _layer(_ssm(3, 20, 8, 1, 3, 3), _moe(52, 2.5, 3, 3)),
         ]}
# the widest kernels: heads of 128, states of 128 x 128, a window longer than most requests
FAP_D = {"architecture": "Fapudra", "vocab": 384, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 16.0},
         "max_positions": 1024, "logit_softcap": 20.0, "layers": [
             _layer(_ssm(4, 64, 128, 1, 4, 1), _moe(128, 1.0, 8, 2, 2, 1)),
             _layer(_par(_left(4, 2, 128, 0.09, 300, 64, window=200, first=6), _right(2, 1, 128, 128, 4, 32, 32), 0.75, 0.55),
                    _moe(96, 1.0, 16, 4, 4, 2)),
         ]}

# heads of 64 in groups of four with a window a little longer than a tile of keys and more kept tokens than a page;
# states whose columns a thread holds two of; a state that fills no whole register block
FAP_E = {"architecture": "Fapudra", "vocab": 300, "width": 192, "norm": {"eps": 2e-6}, "embedding": {"scale": 11.0},
         "max_positions": 640, "logit_softcap": 25.0, "layers": [
             _layer(_ssm(6, 32, 40, 2, 3, 2), _moe(80, 1.4, 6, 2, 2, 1)),
             _layer(_par(_left(8, 2, 64, 0.12, 150, 24, window=72, first=19), _right(4, 2, 32, 64, 3, 12, 20), 0.6, 0.7),
                    _moe(64, 2.0, 4, 2)),
             _layer(_ssm(3, 64, 16, 3, 2, 1), None),
         ]}

# name -> (config, page size)
TINY = {"fap_a": (FAP_A, 16), "fap_b": (FAP_B, 8), "fap_c": (FAP_C, 8), "fap_d": (FAP_D, 32), "fap_e": (FAP_E, 16)}


def get(name):
    cfg, page = TINY[name]
    return copy.deepcopy(cfg), page


def tensor_shapes(cfg):
    """Names and shapes of a checkpoint of ``cfg``, from the design's naming rules."""
    D, s = cfg["width"], {}
    s["embed"] = (cfg["vocab"], D)
    s["pos"] = (cfg["max_positions"], D)
    s["embed.norm"] = ()
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        s[p + "norm1"] = ()
        s[p + "shift"] = (D,)
        m = lc["mixer"]
        if lc["type"] == "mamba2":
            H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * P, H * P + 2 * G * N
            s.update({p + "mix.in": (2 * inner + 2 * G * N + H, D), p + "mix.conv": (ch, taps), p + "mix.conv.b": (ch,),
                      p + "mix.dt_bias": (H,), p + "mix.A_log": (H,), p + "mix.D": (H,), p + "mix.norm": (inner,),
                      p + "mix.o": (D, inner)})
        else:
            l, r = m["left"], m["right"]
            H, G, d = l["heads"], l["kv_heads"], l["dim"]
            s.update({p + "mix.left.q": (H * d, D), p + "mix.left.q.b": (H * d,), p + "mix.left.k": (G * d, D),
                      p + "mix.left.k.b": (G * d,), p + "mix.left.rel": (l["bias_rows"], H), p + "mix.left.pb": (H,),
                      p + "mix.left.g": (H * d, D), p + "mix.left.o": (D, H * d)})
            H, G, d, v, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            s.update({p + "mix.right.q": (G * d, D), p + "mix.right.q.conv": (G * d, taps),
                      p + "mix.right.k": (G * d, D), p + "mix.right.k.conv": (G * d, taps),
                      p + "mix.right.v": (H * v, D), p + "mix.right.v.conv": (H * v, taps),
                      p + "mix.right.b": (H, D), p + "mix.right.A_log": (H,), p + "mix.right.norm": (v,),
                      p + "mix.right.a1": (r["a_rank"], D), p + "mix.right.a2": (H * d, r["a_rank"]),
                      p + "mix.right.dt_bias": (H * d,), p + "mix.right.g1": (r["gate_rank"], D),
                      p + "mix.right.g2": (H * v, r["gate_rank"]), p + "mix.right.o": (D, H * v)})
        f = lc["mlp"]
        if f is not None:
            ff = f["expert"]["ff"]
            for e in range(f["router"]["experts"]):
                s.update({f"{p}mlp.e{e}.gate": (ff, D), f"{p}mlp.e{e}.up": (ff, D), f"{p}mlp.e{e}.down": (D, ff)})
            s[p + "mlp.router"] = (f["router"]["experts"], D)
    s["final.norm"] = ()
    s["head"] = (cfg["vocab"], D)
    return s


def random_weights(cfg, seed):
    """Float32 tensors whose values are exact in bfloat16, so that the same checkpoint serves both
    modes.  Matrices N(0, 1/fan_in) with a gain, norm weights around 1, biases away from 0, decays
    spread between fast and slow, taps of the size of an average with weight on the current token, a
    router with a wide spread of logits, biases of the sigmoid weights well below 0 (hundreds of keys
    add up)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "conv":
            t = torch.randn(shape, generator=g) / shape[1]
            t[:, -1] += 1.0
        elif name == "pos":
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "router":
            t = torch.randn(shape, generator=g) * 3.0 / shape[1] ** 0.5
        elif last == "rel":
            t = 0.8 * torch.randn(shape, generator=g)
        elif last in ("a2", "g2"):
            t = torch.randn(shape, generator=g) * 2.0 / shape[1] ** 0.5
        elif len(shape) == 2:
            gain = 1.0 if name == "embed" else 1.5
            t = torch.randn(shape, generator=g) * gain / (shape[1] ** 0.5 if name != "embed" else 1.0)
        elif last == "b" and name.endswith(("q.b", "k.b", "conv.b")):
            t = 0.2 * torch.randn(shape, generator=g)
        elif last == "pb":
            t = -3.0 + 0.5 * torch.randn(shape, generator=g)
        elif last == "A_log":
            t = torch.randn(shape, generator=g) - 1.0
        elif last == "dt_bias":
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "shift":
            t = torch.rand(shape, generator=g)
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w


def as_numpy(weights):
    return {k: v.double().numpy() for k, v in weights.items()}


def model_folder(tmp, name, cfg, weights, dtype="bfloat16"):
    from gollmgo_b200.weights import save_file
    d = os.path.join(str(tmp), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    td = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    save_file(((k, v.to(td)) for k, v in weights.items()), os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    return d


def steady_requests(cfg, weights, lengths, seed, min_gap=0.08):
    """Random requests in which no token's choice of experts is a close call (the plain
    implementation's router gaps all exceed ``min_gap``): a reduced-precision run then makes the
    same choices, and its logits can be compared with a tolerance of rounding.  A token that makes a
    close call is drawn again; tokens before it are not affected (the model is causal)."""
    import plain_fapudra as P
    rng = random.Random(seed)
    w = as_numpy(weights)
    out = {}
    for i, n in enumerate(lengths):
        toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
        for _ in range(40 * n):
            gaps = []
            P.forward(cfg, w, toks, gaps=gaps)
            if not gaps:
                break
            bad = np.nonzero(np.stack(gaps).min(0) < min_gap)[0]
            if bad.size == 0:
                break
            toks[int(bad[0])] = rng.randrange(cfg["vocab"])
        else:
            raise AssertionError("no request without close calls found")
        out[f"r{i}"] = toks
    return out
