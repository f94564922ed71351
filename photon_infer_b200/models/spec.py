"""A model as data: which parts each layer has, and in which order layers run.

An architecture's ``build_spec(config)`` returns a ``ModelSpec``; ``CausalLM`` builds
the parts from it, the weight loader and the random-weights mode read the tensor
list from it, and the cache manager reads the cache needs from it.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional


@dataclasses.dataclass
class PartSpec:
    kind: str                               # a name in the matching registry of parts.registry
    params: Dict[str, Any]                  # constructor parameters (sizes and constants)
    prefix: str = ""                        # weight-name prefix inside the layer, e.g. "self_attn."


@dataclasses.dataclass
class LayerSpec:
    block: PartSpec                         # arrangement, e.g. kind "pre_norm"
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    feed_forward: PartSpec
    prefix: str                             # e.g. "model.layers.3."


@dataclasses.dataclass
class RunEntry:
    """One step of the run list.  ``layer`` indexes ``ModelSpec.layers`` and may occur in
    several entries (shared weights, a cache of its own for each entry).  ``kv_from``
    names an EARLIER entry of the run list whose cache this entry reads instead of
    writing one."""
    layer: int
    kv_from: Optional[int] = None


@dataclasses.dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding_name: str                     # e.g. "model.embed_tokens.weight"
    head_name: Optional[str]                # None: the output head is the embedding table (tied)
    final_norm: PartSpec
    position_encodings: Dict[str, PartSpec]  # shared by name between the mixers that ask for one
    layers: List[LayerSpec]
    run: List[RunEntry]
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    # name patterns of tensors that weight files of this architecture may carry and the model does not use
    ignored_tensors: tuple = ()
    # optional factors: the embedded rows are multiplied by ``embedding_scale`` before the first block, the
    # logits by ``logit_scale`` after the head (architectures that scale either; None: untouched)
    embedding_scale: Optional[float] = None
    logit_scale: Optional[float] = None

    def validate(self) -> None:
        from ..errors import ErrorCode, PhotonError
        for i, e in enumerate(self.run):
            if not 0 <= e.layer < len(self.layers):
                raise PhotonError(ErrorCode.INVALID_CONFIG, f"run entry {i} names layer {e.layer}, which does not exist")
            if e.kv_from is not None:
                if not 0 <= e.kv_from < i:
                    raise PhotonError(ErrorCode.INVALID_CONFIG,
                                      f"run entry {i} reads the cache of entry {e.kv_from}, which does not run before it")
                if self.run[e.kv_from].kv_from is not None:
                    raise PhotonError(ErrorCode.INVALID_CONFIG,
                                      f"run entry {i} reads the cache of entry {e.kv_from}, which has none of its own")
