"""Fivesun as a ModelSpec: sandwich blocks (an RMS norm before and after every sublayer, and between
them a learned sigmoid gate on the sublayer's result, computed from the sublayer's own input), three kinds
of mixer listed layer by layer (grouped-query attention with normed heads, interleaved rotary positions
with linearly scaled frequencies, a chunked mask, a sink in the softmax, values blended with the first such
layer's and a gate per head; latent attention with a rotated key part shared by the heads, stretched
rotary frequencies, a sliding window and a gate per channel; a matrix memory with exponential gates), a
ReLU-gated feed-forward with biases, a scaled embedding, an RMS norm and an untied head.
Tensor names: layer i's start with "l<i>.", the mixer's with "l<i>.mix.", the feed-forward's with
"l<i>.mlp."; the norms are "l<i>.norm1", "norm1b", "norm2", "norm2b", the gates "l<i>.rg1", "rg2" (+ ".b").
"""
from __future__ import annotations

from ..config import RopeScaling, register_architecture
from ..config.fivesun_config import FivesunConfig, MatrixMemoryConfig, NormedAttentionConfig, RotatedLatentConfig
from ..parts.position import YarnScaling
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _position(rot, dim: int) -> PartSpec:
    if rot is None:
        return PartSpec("none")
    scaling = None
    if rot.blend is not None:
        scaling = YarnScaling(rot.factor, *rot.blend)
    elif rot.factor is not None:
        scaling = RopeScaling("linear", factor=rot.factor)
    return PartSpec("rope", {"head_dim": dim, "rotary_dim": rot.dims, "theta": rot.base, "scaling": scaling,
                             "interleaved": True})


def _mixer(cfg: FivesunConfig, m, first_blend: bool) -> PartSpec:
    if isinstance(m, NormedAttentionConfig):
        return PartSpec("normed_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
            "v_head_dim": m.vdim, "position": _position(m.rot, m.dim), "scale": m.scale, "eps": cfg.eps,
            "qk_norm": True, "v_norm": True, "chunk": m.chunk, "sink": True,
            "v_mix": ("first" if first_blend else "blend") if m.v_mix else None, "head_gate": True})
    if isinstance(m, RotatedLatentConfig):
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
            "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.eps, "gate": "element", "rot_dim": m.rot_dim,
            "position": _position(m.rot, m.rot_dim), "window": m.window})
    if isinstance(m, MatrixMemoryConfig):
        return PartSpec("mlstm", {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim,
                                  "v_head_dim": m.vdim, "gate_cap": m.gate_cap, "eps": cfg.eps})
    raise TypeError(type(m).__name__)


def fivesun_spec(cfg: FivesunConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps})
    block = PartSpec("sandwich", {"eps": cfg.eps, "gated": True, "post_names": ("norm1b", "norm2b"),
                                  "gate_names": ("rg1", "rg2")})
    layers, ignorable, blended = [], [], False
    for i, lc in enumerate(cfg.layers):
        p = f"l{i}."
        blends = isinstance(lc.mixer, NormedAttentionConfig) and lc.mixer.v_mix
        mixer = _mixer(cfg, lc.mixer, first_blend=blends and not blended)
        blended = blended or blends
        ff = None
        if lc.mlp is not None:
            ff = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": lc.mlp.ff, "activation": "relu",
                                        "bias": True, "defer_output_bias": True, "names": ("gate", "up", "down")})
        else:
            ignorable += [p + "norm2", p + "norm2b", p + "rg2", p + "rg2.b"]
        layers.append(LayerSpec(block, mixer, ff, norm, norm if ff is not None else None, mixer_prefix=p + "mix.",
                                ffn_prefix=p + "mlp.", mixer_norm_name=p + "norm1", ffn_norm_name=p + "norm2",
                                block_prefix=p))
    n = len(layers)
    return ModelSpec(architecture="Fivesun", vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
                     run_order=tuple(RunEntry(i, i) for i in range(n)), final_norm=norm, tie_embeddings=False,
                     embed_name="embed", final_norm_name="final.norm", head_name="head",
                     max_positions=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids,
                     bos_token_id=cfg.bos_token_id, ignorable_tensors=tuple(ignorable), embed_scale=cfg.embed_scale)


register_architecture("Fivesun", FivesunConfig.from_dict, fivesun_spec)
