"""Small Fivesun configurations and weights for the tests.  The configurations differ in every size, in the
order of their layers and in which optional features they have: attention with chunks shorter and longer
than a page and with none, partial and full rotation, scaled and unscaled frequencies, one kv head and as
many as heads, values of another size than keys, with and without blended values (the first blending layer
not being the model's first layer); latent attention with windows shorter than a page and with none, ranks
that need padding and one beyond what a cache row holds, one to five heads; matrix memories whose values are
no multiple of four; a layer without feed-forward; widths that are no multiple of 8; with and without a scaled
embedding."""
import copy
import json
import os

import torch


def _rot(dims, base, factor=None, blend=None):
    r = {"dims": dims, "base": base}
    if factor is not None:
        r["scaling"] = {"factor": factor}
        if blend is not None:
            r["scaling"].update({"original": blend[0], "fast": blend[1], "slow": blend[2]})
    return r


def _att(heads, kv, dim, vdim, scale, chunk=None, rot=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = rot
    return {"type": "attention", "mixer": m}


def _lat(heads, dim, rot_dim, vdim, rank, scale, window=None, base=10000.0, factor=None, blend=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": _rot(rot_dim, base, factor, blend)}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def _mem(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def _layer(mixer, ff):
    return dict(mixer, mlp={"kind": "dense", "ff": ff} if ff else None)


# latent attention first; the first blending layer is the model's second; an attention layer without blending
FIV_A = {"architecture": "Fivesun", "vocab": 203, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0}, "layers": [
    _layer(_lat(3, 16, 8, 24, 24, 0.2, window=20, base=10000.0, factor=4.0, blend=(64, 16.0, 1.0)), 40),
    _layer(_att(4, 2, 32, 16, 0.16, chunk=24, rot=_rot(16, 10000.0, 2.0), v_mix=True), 48),
    _layer(_mem(2, 16, 24, 8.0), 56),
    _layer(_att(4, 2, 32, 16, 0.16, chunk=24, rot=_rot(16, 10000.0, 2.0), v_mix=True), None),
    _layer(_att(3, 1, 24, 40, 0.2, chunk=40, rot=_rot(24, 500000.0)), 32),
]}
# no embedding scale; heads of 64 (bfloat16 runs the tensor-core kernels of the general path); a chunk that is no multiple
# of a page or a tile; a latent whose row is 64 values; a window longer than most requests
FIV_B = {"architecture": "Fivesun", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "layers": [
    _layer(_mem(4, 32, 32, 15.0), 64),
    _layer(_att(2, 2, 64, 64, 0.11, chunk=100, rot=_rot(64, 1000000.0, 8.0), v_mix=True), 72),
    _layer(_lat(4, 32, 16, 32, 48, 0.14, window=150, base=1000000.0, factor=2.0, blend=(128, 32.0, 2.0)), 96),
    _layer(_att(2, 2, 64, 64, 0.11, chunk=100, rot=_rot(64, 1000000.0, 8.0), v_mix=True), 40),
    _layer(_att(2, 2, 64, 64, 0.11, chunk=100, rot=_rot(32, 1000000.0), v_mix=True), None),
]}
# sizes that are no multiple of 8; a chunk and a window shorter than a page; an attention layer and a latent layer
# that see every earlier token; one blending layer alone
FIV_C = {"architecture": "Fivesun", "vocab": 150, "width": 100, "norm": {"eps": 3e-6}, "embedding": {"scale": 3.5}, "layers": [
    _layer(_att(6, 2, 12, 20, 0.3, chunk=7, rot=_rot(8, 10000.0, 1.5), v_mix=True), 28),
    _layer(_lat(5, 12, 4, 20, 40, 0.25, window=5, base=5000.0), 52),
    _layer(_mem(3, 20, 11, 5.0), None),
    _layer(_att(2, 2, 20, 12, 0.22, rot=_rot(20, 10000.0, 3.0)), 36),
    # a latent too wide to be cached as one row of at most 256 values: per-head keys and values are cached instead
    _layer(_lat(1, 24, 12, 16, 264, 0.2, base=10000.0, factor=8.0, blend=(32, 8.0, 1.0)), 44),
]}
# the widest kernels: heads of 128, a latent row of 128, a memory of 128 x 64; chunks of exactly four pages
FIV_D = {"architecture": "Fivesun", "vocab": 384, "width": 192, "norm": {"eps": 1e-6}, "embedding": {"scale": 12.0}, "layers": [
    _layer(_att(4, 2, 128, 64, 0.09, chunk=128, rot=_rot(64, 1000000.0, 2.0), v_mix=True), 128),
    _layer(_mem(2, 128, 64, 10.0), 96),
    _layer(_lat(4, 64, 32, 64, 96, 0.1, window=100, base=1000000.0, factor=4.0, blend=(256, 32.0, 1.0)), 112),
    _layer(_att(6, 2, 128, 64, 0.09, chunk=128, rot=_rot(128, 1000000.0, 2.0), v_mix=True), 80),
]}

# name -> (config, page size)
TINY = {"fiv_a": (FIV_A, 16), "fiv_b": (FIV_B, 8), "fiv_c": (FIV_C, 8), "fiv_d": (FIV_D, 32)}


def get(name):
    cfg, page = TINY[name]
    return copy.deepcopy(cfg), page


def tensor_shapes(cfg):
    """Names and shapes of a checkpoint of ``cfg``, from the design's naming rules."""
    D, s = cfg["width"], {}
    s["embed"] = (cfg["vocab"], D)
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = lc["mixer"]
        s.update({p + "norm1": (D,), p + "norm1b": (D,), p + "rg1": (D, D), p + "rg1.b": (D,)})
        if lc["type"] == "attention":
            H, G, d, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            s.update({p + "mix.q": (H * d, D), p + "mix.k": (G * d, D), p + "mix.v": (G * v, D), p + "mix.q.norm": (d,),
                      p + "mix.k.norm": (d,), p + "mix.sink": (H,), p + "mix.g": (H, D), p + "mix.o": (D, H * v)})
            if m.get("v_mix"):
                s[p + "mix.vmix"] = ()
        elif lc["type"] == "latent_attention":
            H, d, r, v, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            s.update({p + "mix.q": (H * (d + r), D), p + "mix.dkv": (R + r, D), p + "mix.dkv.norm": (R,),
                      p + "mix.uk": (H * d, R), p + "mix.uv": (H * v, R), p + "mix.g": (H * v, D), p + "mix.o": (D, H * v)})
        else:
            H, d, v = m["heads"], m["dim"], m["vdim"]
            s.update({p + "mix.q": (H * d, D), p + "mix.k": (H * d, D), p + "mix.v": (H * v, D), p + "mix.g": (H * v, D),
                      p + "mix.o": (D, H * v), p + "mix.norm": (H * v,), p + "mix.i": (H, D), p + "mix.i.b": (H,),
                      p + "mix.f": (H, D), p + "mix.f.b": (H,)})
        if lc["mlp"] is not None:
            ff = lc["mlp"]["ff"]
            s.update({p + "norm2": (D,), p + "norm2b": (D,), p + "rg2": (D, D), p + "rg2.b": (D,),
                      p + "mlp.gate": (ff, D), p + "mlp.gate.b": (ff,), p + "mlp.up": (ff, D), p + "mlp.up.b": (ff,),
                      p + "mlp.down": (D, ff), p + "mlp.down.b": (D,)})
    s["final.norm"] = (D,)
    s["head"] = (cfg["vocab"], D)
    return s


def random_weights(cfg, seed):
    """Float32 tensors whose values are exact in bfloat16, so that the same checkpoint serves both modes.
    Matrices N(0, 1/fan_in) with a gain, norm weights around 1, biases away from 0, sinks of the size of a
    large score, blend factors between 0.2 and 0.8, forget-gate biases that make the memory last."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "vmix":
            t = 0.2 + 0.6 * torch.rand(shape, generator=g)
        elif last == "sink":
            t = 1.0 + torch.randn(shape, generator=g)
        elif name.endswith("f.b"):
            t = 3.0 + torch.randn(shape, generator=g)
        elif name.endswith("i.b"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif len(shape) == 2:
            gain = 1.0 if name == "embed" else 1.5
            t = torch.randn(shape, generator=g) * gain / (shape[1] ** 0.5 if name != "embed" else 1.0)
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)
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
