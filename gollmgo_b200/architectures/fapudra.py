"""Fapudra as a ModelSpec: token embeddings times a constant plus learned positions, an RMS norm on
that; parallel blocks (one RMS norm whose weight is a single number; the mixer reads a token-shifted
copy of its output, the feed-forward the output itself; both are added to the stream); two kinds of
mixer (a state-space layer; or a sigmoid attention whose values are its keys beside a delta rule with
a decay per key channel, summed with a factor each); a mixture of experts with grouped choice and a
clamped activation; an RMS norm, an untied head and capped logits.
Tensor names: "embed", "pos", "embed.norm", "final.norm", "head"; layer i's start with "l<i>.":
"l<i>.norm1", "l<i>.shift", the mixer's "l<i>.mix.", the feed-forward's "l<i>.mlp.".
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.fapudra_config import FapudraConfig, Mamba2Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mixer(cfg: FapudraConfig, m) -> PartSpec:
    if isinstance(m, Mamba2Config):
        return PartSpec("mamba2", {"hidden_size": cfg.width, "num_heads": m.heads, "v_head_dim": m.vdim, "state": m.state,
                                   "groups": m.groups, "conv": m.conv, "norm_groups": m.norm_groups, "eps": cfg.eps})
    left, right = m.left, m.right
    attn = PartSpec("sigmoid_attention", {"hidden_size": cfg.width, "num_heads": left.heads, "num_kv_heads": left.kv_heads,
                                          "head_dim": left.dim, "window": left.window, "keep_first": left.keep_first,
                                          "scale": left.scale, "bias_max": left.bias_max, "bias_rows": left.bias_rows})
    delta = PartSpec("gated_delta", {"hidden_size": cfg.width, "num_heads": right.heads, "num_kv_heads": right.kv_heads,
                                     "head_dim": right.dim, "v_head_dim": right.vdim, "conv": right.conv, "eps": cfg.eps,
                                     "decay": "channel", "a_rank": right.a_rank, "gate_rank": right.gate_rank,
                                     "gate_act": "sigmoid"})
    return PartSpec("parallel", {"hidden_size": cfg.width, "eps": cfg.eps, "branch_norm": False,
                                 "scales": (m.left_scale, m.right_scale),
                                 "branches": ((attn, "left.", ""), (delta, "right.", ""))})


def fapudra_spec(cfg: FapudraConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "scalar": True})
    block = PartSpec("parallel", {})
    layers = []
    for i, lc in enumerate(cfg.layers):
        p = f"l{i}."
        ff = None
        if lc.mlp is not None:
            f = lc.mlp
            ff = PartSpec("moe", {"hidden_size": cfg.width, "intermediate_size": f.ff, "experts": f.experts, "top": f.top,
                                  "router_bias": False, "router_weigh": "softmax_all",
                                  "groups": (f.group_count, f.group_keep), "activation": "clamped_swish", "limit": f.limit})
        shifted = PartSpec("token_shift", {"hidden_size": cfg.width, "inner": _mixer(cfg, lc.mixer), "inner_prefix": "mix.",
                                           "name": "shift"})
        layers.append(LayerSpec(block, shifted, ff, norm, None, mixer_prefix=p, ffn_prefix=p + "mlp.",
                                mixer_norm_name=p + "norm1", block_prefix=p))
    return ModelSpec(architecture="Fapudra", vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers),
                     run_order=tuple(RunEntry(i, i) for i in range(len(layers))), final_norm=norm, tie_embeddings=False,
                     embed_name="embed", final_norm_name="final.norm", head_name="head",
                     max_positions=cfg.max_positions, eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id,
                     embed_position=PartSpec("learned", {"hidden_size": cfg.width, "max_positions": cfg.max_positions}),
                     embed_position_prefix="pos", embed_scale=cfg.embedding_scale, embed_norm=norm,
                     embed_norm_name="embed.norm", logit_softcap=cfg.logit_softcap)


register_architecture("Fapudra", FapudraConfig.from_dict, fapudra_spec)
