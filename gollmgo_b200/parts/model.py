"""The generic decoder: embedding, the layers in run order, final norm, LM head.

Built from a ``ModelSpec`` alone.  Data flow per step (reference:
kernels/gollmgo_model.cu:796-858 and run_layer): ids -> float32 residual stream
-> blocks -> rows whose logits are wanted -> final norm -> head product ->
float32 logits.  The reference computes the head for every token of a prompt;
here only the wanted rows reach the final norm and the head.
"""
from __future__ import annotations

from typing import Callable, Dict, List

import torch

from ..config import read_config_json, resolve_architecture
from ..csrc import ops
from ..weights import WeightSpec
from .block import ResidualRows
from .context import BuildContext
from .linear import linear
from .registry import build_block, build_feed_forward, build_mixer, build_norm, build_position
from .spec import ModelSpec


def _prefixed(prefix: str, weights: Dict[str, WeightSpec], single_name: str = "") -> Dict[str, WeightSpec]:
    """Checkpoint names of a part's tensors.  A mixer or feed-forward: prefix + local name.  A norm
    (``single_name`` given): its one tensor "" has that name, any further tensor (a bias ".b") that
    name with the local name appended."""
    if single_name:
        return {single_name + local: spec for local, spec in weights.items()}
    return {prefix + local: spec for local, spec in weights.items()}


def spec_manifest(spec: ModelSpec, parts=None, embed_position=None, blocks=None, final_norm=None,
                  embed_norm=None) -> Dict[str, WeightSpec]:
    """Checkpoint tensors the model expects.  ``parts`` = per layer
    (mixer, feed_forward, mixer_norm, ffn_norm) if already built; ``blocks`` = the layers' blocks
    (one that has tensors of its own offers ``weights()`` and ``load(get)``)."""
    m: Dict[str, WeightSpec] = {spec.embed_name: WeightSpec((spec.vocab_size, spec.hidden_size))}
    for ls, (mixer, ff, n1, n2) in zip(spec.layers, parts):
        m.update(_prefixed(ls.mixer_prefix, mixer.weights()))
        if ff is not None:
            m.update(_prefixed(ls.ffn_prefix, ff.weights()))
        if n1 is not None:
            m.update(_prefixed("", n1.weights(), ls.mixer_norm_name))
        if n2 is not None:
            m.update(_prefixed("", n2.weights(), ls.ffn_norm_name))
    for ls, block in zip(spec.layers, blocks or ()):
        if hasattr(block, "weights"):
            m.update(_prefixed(ls.block_prefix, block.weights()))
    if final_norm is not None:
        m.update(_prefixed("", final_norm.weights(), spec.final_norm_name))
    else:
        m[spec.final_norm_name] = WeightSpec((spec.hidden_size,))
    if embed_position is not None:
        m.update(_prefixed(spec.embed_position_prefix, embed_position.weights()))
    if embed_norm is not None:
        m.update(_prefixed("", embed_norm.weights(), spec.embed_norm_name))
    if spec.input_mix_name:
        m[spec.input_mix_name] = WeightSpec((spec.hidden_size, 2 * spec.hidden_size))
    m[spec.head_name] = WeightSpec((spec.vocab_size, spec.hidden_size), optional=spec.tie_embeddings)
    return m


class DecoderModel:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.parts = []
        self.blocks = []
        for ls in spec.layers:
            mixer = build_mixer(ls.mixer, ctx)
            # a layer may have no feed-forward (and then no norm for it)
            ff = build_feed_forward(ls.feed_forward, ctx) if ls.feed_forward is not None else None
            n1 = build_norm(ls.mixer_norm, ctx)
            n2 = build_norm(ls.ffn_norm, ctx) if ls.ffn_norm is not None else None
            self.parts.append((mixer, ff, n1, n2))
            self.blocks.append(build_block(ls, mixer, ff, n1, n2, ctx))
        self.final_norm = build_norm(spec.final_norm, ctx)
        self.embed_position = build_position(spec.embed_position, ctx) if spec.embed_position else None
        self.embed_norm = build_norm(spec.embed_norm, ctx) if spec.embed_norm else None
        if self.embed_norm is not None and not hasattr(self.embed_norm, "norm_in_place"):
            raise TypeError(f"norm {type(self.embed_norm).__name__} cannot sit on the embedding output (no norm_in_place)")
        ws = ctx.workspace
        ws.reserve("residual", ctx.max_tokens * spec.hidden_size, torch.float32)
        ws.reserve("head_in", ctx.max_tokens * spec.hidden_size, ctx.act_dtype)
        self.mixes_input = any(e.mix_input for e in spec.run_order)
        if self.mixes_input:
            if not spec.input_mix_name:
                raise ValueError("a run entry mixes the embedding output in, but the model names no tensor for it")
            ws.reserve("embed_out", ctx.max_tokens * spec.hidden_size, torch.float32)
            ws.reserve("mix_in", ctx.max_tokens * 2 * spec.hidden_size, ctx.act_dtype)
        self.w_input_mix = None
        self.embed = None
        self.head = None
        self.bad_id = torch.zeros(1, dtype=torch.int32, device=ctx.device) \
            if ctx.device.type == "cuda" else None

    # ------------------------------------------------------------------ weights
    def manifest(self) -> Dict[str, WeightSpec]:
        return spec_manifest(self.spec, self.parts, self.embed_position, self.blocks, self.final_norm, self.embed_norm)

    def load(self, get: Callable[[str], torch.Tensor]) -> None:
        """Bind weights: ``get(name)`` delivers a checkpoint tensor on the device."""
        s = self.spec
        self.embed = get(s.embed_name).contiguous()
        for ls, (mixer, ff, n1, n2) in zip(s.layers, self.parts):
            mixer.load(lambda local, p=ls.mixer_prefix: get(p + local))
            if ff is not None:
                ff.load(lambda local, p=ls.ffn_prefix: get(p + local))
            if n1 is not None:
                n1.load(lambda local, n=ls.mixer_norm_name: get(n + local))
            if n2 is not None:
                n2.load(lambda local, n=ls.ffn_norm_name: get(n + local))
        for ls, block in zip(s.layers, self.blocks):
            if hasattr(block, "load"):
                block.load(lambda local, p=ls.block_prefix: get(p + local))
        self.final_norm.load(lambda local: get(s.final_norm_name + local))
        if self.embed_position is not None:
            self.embed_position.load(lambda local, p=s.embed_position_prefix: get(p + local))
        if self.embed_norm is not None:
            self.embed_norm.load(lambda local: get(s.embed_norm_name + local))
        if self.mixes_input:
            self.w_input_mix = get(s.input_mix_name).contiguous()
        head = None if s.tie_embeddings else get(s.head_name)
        self.head = self.embed if head is None else head.contiguous()

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.embed), add(self.head), add(self.w_input_mix)
        add(getattr(self.embed_position, "table", None))
        def add_part(part, depth=0):
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.is_cuda:
                    add(v)
                elif depth < 2 and hasattr(v, "weights") and hasattr(v, "load"):     # a part inside a part
                    add_part(v, depth + 1)
                elif depth < 2 and isinstance(v, (list, tuple)):                     # ... or parts and tensors in a list
                    for item in v:
                        if isinstance(item, torch.Tensor) and item.dim() >= 1 and item.is_cuda:
                            add(item)
                        elif hasattr(item, "weights") and hasattr(item, "load"):
                            add_part(item, depth + 1)
        add_part(self.final_norm)
        for parts, block in zip(self.parts, self.blocks):
            for part in parts:
                if part is not None:
                    add_part(part)
            for name in ("scale1", "scale2"):
                add(getattr(block, name, None))
        return total

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> List[object]:
        """Per cache entry of the run order, what it needs of the cache manager."""
        needs: List[object] = [None] * self.spec.num_cache_entries
        for e in self.spec.run_order:
            need = self.parts[e.layer][0].cache_need()
            if needs[e.cache] is not None and needs[e.cache] != need:
                raise ValueError(f"cache entry {e.cache} is used by layers with different needs")
            needs[e.cache] = need
        return needs

    # ------------------------------------------------------------------ what the parts ask of a step
    def query_tiles(self) -> list:
        """The index lists (QueryTiles) the mixers want in every step's batch."""
        wanted = []
        for mixer, _, _, _ in self.parts:
            for need in getattr(mixer, "query_tiles", lambda: ())():
                if need not in wanted:
                    wanted.append(need)
        return wanted

    def step_tags(self, facts) -> tuple:
        """The step's kind: the tags of every part that offers ``step_tags(facts)``, sorted."""
        tags = set()
        for parts in self.parts:
            for part in parts:
                f = getattr(part, "step_tags", None) if part is not None else None
                if f is not None:
                    tags.update(f(facts))
        return tuple(sorted(tags))

    # ------------------------------------------------------------------ forward
    def forward(self, batch, caches) -> torch.Tensor:
        """Run the batch's tokens; return float32 logits [len(logit_rows), vocab].
        ``caches[i]`` is what the cache manager holds for cache entry i."""
        T, H = batch.num_tokens, self.spec.hidden_size
        ws = self.ctx.workspace
        resid = ws.get("residual", T, H)
        ops.embed_gather(batch.token_ids, self.embed, resid, self.bad_id,
                         getattr(batch, "token_src", None), getattr(batch, "prev_tokens", None))
        scale = float(self.spec.embed_scale)
        if self.embed_position is not None:
            if scale != 1.0:
                self.embed_position.add_to_embedding(resid, batch, scale=scale)     # scale and positions in one pass
            else:
                self.embed_position.add_to_embedding(resid, batch)
        elif scale != 1.0:
            resid.mul_(scale)
        if self.embed_norm is not None:
            self.embed_norm.norm_in_place(resid)
        delta = None
        order = self.spec.run_order
        x0 = None
        if self.mixes_input:
            x0 = ws.get("embed_out", T, H)
            x0.copy_(resid)
        for i, e in enumerate(order):
            block = self.blocks[e.layer]
            if e.mix_input:
                # x <- W [x; x0]: both halves rounded to the activation type for the product, the
                # result float32 straight into the stream (what the block before still owes is added first)
                if not (delta is None or isinstance(delta, ResidualRows) or torch.is_tensor(delta)):
                    raise ValueError("the block before an input mix handed on a norm's input instead of its output")
                cat = ws.get("mix_in", T, 2 * H)
                ops.concat_cast(resid, delta if torch.is_tensor(delta) else None, x0, cat)
                linear(cat, self.w_input_mix, resid)
                delta = None
            if getattr(block, "chains_norms", False):
                # such a block may fold the first norm of the block that runs next into its last product
                nxt = self.blocks[order[i + 1].layer] if i + 1 < len(order) and not order[i + 1].mix_input else None
                delta = block.forward(resid, delta, batch, caches[e.cache], e.writes_cache, next_block=nxt)
            else:
                delta = block.forward(resid, delta, batch, caches[e.cache], e.writes_cache)
        R = batch.num_logit_rows
        logits = torch.empty(R, self.spec.vocab_size, dtype=torch.float32, device=self.ctx.device)
        if R == 0:
            return logits
        h = ws.get("head_in", R, H)
        if isinstance(delta, ResidualRows):
            delta = None                       # the last block has added everything to the residual itself
        self.final_norm.add_norm(resid, delta, h, rows=batch.logit_rows, write_back=False)
        linear(h, self.head, logits)
        if self.spec.logit_softcap > 0:
            ops.softcap(logits, float(self.spec.logit_softcap))
        return logits


def build_model(config_dict: dict, ctx: BuildContext):
    """config.json dict -> (typed config, ModelSpec, DecoderModel) via the registry."""
    arch = resolve_architecture(config_dict)
    cfg = arch.parse(config_dict)
    spec = arch.spec(cfg)
    return cfg, spec, DecoderModel(spec, ctx)


def manifest_for_config(config_dict: dict) -> Dict[str, WeightSpec]:
    """Tensors a checkpoint of this configuration holds (no device needed)."""
    ctx = BuildContext(torch.float32, "cpu", 1, 1, 16)
    return build_model(config_dict, ctx)[2].manifest()
