"""What a model is made of, as data.

An architecture turns its typed configuration into a ``ModelSpec``: one
``LayerSpec`` per layer (which mixer, which feed-forward, which norms, arranged
by which block, each with its sizes and constants as parameters) and a run
order.  The generic ``DecoderModel`` builds the parts named here from the parts
registry; no part knows which model it is in.

The run order is a list of ``RunEntry``.  An entry names the layer to run and the
cache entry it uses; a layer may be named twice (each occurrence with a cache
entry of its own), and an entry with ``writes_cache=False`` reads the cache that
another entry wrote instead of writing its own.  An entry with ``mix_input`` first
remakes the stream from itself and the embedding output (``ModelSpec.input_mix_name``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part by registry name with its parameters (sizes, constants)."""
    kind: str
    params: Dict[str, object] = field(default_factory=dict)

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec                    # arrangement, e.g. "pre_norm"
    mixer: PartSpec                    # e.g. "attention"
    feed_forward: Optional[PartSpec]   # e.g. "gated_mlp"; None: the layer has no feed-forward
    mixer_norm: PartSpec               # norm before (or, in a post-norm block, after) the mixer
    ffn_norm: Optional[PartSpec]       # norm before (or, in a post-norm block, after) the feed-forward
    # checkpoint names: prefix of the mixer's and feed-forward's tensors, full
    # names of the two norm weights
    mixer_prefix: str = ""
    ffn_prefix: str = ""
    mixer_norm_name: str = ""
    ffn_norm_name: str = ""
    # prefix of the tensors that belong to the block itself (per-channel scales of its two
    # branches, say); a block without tensors ignores it
    block_prefix: str = ""


@dataclass(frozen=True)
class RunEntry:
    layer: int
    cache: int                         # index of the cache entry this occurrence uses
    writes_cache: bool = True
    # before this entry runs, the stream is remade from itself and the embedding output:
    # x <- W [x; x0] with the tensor ModelSpec.input_mix_name ([width, 2 width], x first)
    mix_input: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    tie_embeddings: bool
    embed_name: str
    final_norm_name: str
    head_name: str
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    # a position encoding that acts on the embedded tokens, before the first layer (a table of
    # learned positions, say), with the prefix of its checkpoint tensors; None = the layers'
    # mixers do all the position encoding there is (rotary: inside attention)
    embed_position: Optional[PartSpec] = None
    embed_position_prefix: str = ""
    # name patterns (fnmatch) of checkpoint tensors that this model does not use and a
    # checkpoint may still hold
    ignorable_tensors: Tuple[str, ...] = ()
    # the tensor of the run entries' mix_input (a model that runs some of its layers several
    # times feeds the embedding output back in at the start of every pass); "" = none
    input_mix_name: str = ""
    # the embedded tokens are multiplied by this before anything else is done with them
    embed_scale: float = 1.0
    # a norm on the embedding output (after the scale and an ``embed_position``), with its tensor's name
    embed_norm: Optional[PartSpec] = None
    embed_norm_name: str = ""
    # > 0: logits <- cap * tanh(logits / cap)
    logit_softcap: float = 0.0

    @property
    def num_cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.run_order), default=-1)
