"""A causal language model built from a ``ModelSpec``: embedding, the run list of
blocks, final norm and output head.  It knows nothing of Llama; the spec does.

``forward`` runs exactly the tokens of one step (``StepContext``) against the cache
and returns 32-bit logits for the wanted rows only; the reference computes logits
for every token of the step (include/photon/scheduler/continuous_batch_engine.hpp:
226-237).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..errors import ErrorCode, PhotonError
from ..kernels import ops
from ..parts.base import (Block, LayerCache, Mixer, PagedCacheSpec, Part, StateSpec, StepContext,
                          TensorSpec)
from ..parts.registry import create_part
from .spec import LayerSpec, ModelSpec


def _build_position_encodings(spec: ModelSpec) -> Dict[str, Part]:
    return {name: create_part("position_encoding", ps.kind, ps.params)
            for name, ps in spec.position_encodings.items()}


def _build_layer(ls: LayerSpec, encodings: Dict[str, Part]) -> Block:
    mixer_params = dict(ls.mixer.params)
    if "position_encoding" in mixer_params and isinstance(mixer_params["position_encoding"], str):
        key = mixer_params["position_encoding"]
        if key not in encodings:
            raise PhotonError(ErrorCode.INVALID_CONFIG, f"mixer asks for position encoding {key!r}, which the model does not define")
        mixer_params["position_encoding"] = encodings[key]
    norm1 = create_part("norm", ls.norm1.kind, ls.norm1.params)
    mixer = create_part("mixer", ls.mixer.kind, mixer_params)
    norm2 = create_part("norm", ls.norm2.kind, ls.norm2.params)
    ff = create_part("feed_forward", ls.feed_forward.kind, ls.feed_forward.params)
    return create_part("block", ls.block.kind, dict(ls.block.params, norm1=norm1, mixer=mixer, norm2=norm2,
                                                    feed_forward=ff))


def _layer_part_prefixes(ls: LayerSpec) -> Dict[str, str]:
    return {"norm1": ls.prefix + ls.norm1.prefix, "mixer": ls.prefix + ls.mixer.prefix,
            "norm2": ls.prefix + ls.norm2.prefix, "feed_forward": ls.prefix + ls.feed_forward.prefix}


class _Skeleton:
    """Parts of a model built without weights or a device: enough to list tensors and cache needs."""

    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.encodings = _build_position_encodings(spec)
        self.blocks: List[Block] = [_build_layer(ls, self.encodings) for ls in spec.layers]
        self.final_norm = create_part("norm", spec.final_norm.kind, spec.final_norm.params)

    def named_parts(self) -> List[Tuple[str, Part]]:
        out: List[Tuple[str, Part]] = []
        for name, pe in self.encodings.items():
            out.append((self.spec.position_encodings[name].prefix, pe))
        for ls, block in zip(self.spec.layers, self.blocks):
            prefixes = _layer_part_prefixes(ls)
            for key, part in block.parts().items():
                out.append((prefixes[key], part))
        out.append((self.spec.final_norm.prefix, self.final_norm))
        return out

    def declared(self) -> Dict[str, TensorSpec]:
        s = self.spec
        d: Dict[str, TensorSpec] = {s.embedding_name: TensorSpec(s.embedding_name, (s.vocab_size, s.hidden_size))}
        for prefix, part in self.named_parts():
            for ts in part.tensor_specs():
                full = prefix + ts.name
                if full in d:
                    raise PhotonError(ErrorCode.INVALID_CONFIG, f"two parts declare the tensor {full!r}")
                d[full] = ts
        if s.head_name is not None:
            d[s.head_name] = TensorSpec(s.head_name, (s.vocab_size, s.hidden_size))
        return d


def declared_tensors(spec: ModelSpec) -> Dict[str, TensorSpec]:
    """Full tensor name -> spec, for the loader and the random-weights mode."""
    return _Skeleton(spec).declared()


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        sk = _Skeleton(spec)
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.encodings = sk.encodings
        self.blocks = sk.blocks
        self.final_norm = sk.final_norm
        self._skeleton = sk
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ weights
    def declared(self) -> Dict[str, TensorSpec]:
        return self._skeleton.declared()

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[s.embedding_name]
        self.head = self.embedding if s.head_name is None else tensors[s.head_name]   # tied: alias, no copy
        for prefix, part in self._skeleton.named_parts():
            local = {ts.name: tensors[prefix + ts.name] for ts in part.tensor_specs()}
            part.load(local)
        for pe in self.encodings.values():
            if hasattr(pe, "to_device"):
                pe.to_device(self.device)

    def kernel_modules(self) -> List[object]:
        """What this model launches in this dtype: module names and (name, definitions) pairs."""
        mods: List[object] = ["elementwise", "sampling"]
        if self.dtype == torch.float32:
            mods.append("gemm_f32")
        for _, part in self._skeleton.named_parts():
            for m in part.required_kernels(self.dtype):
                if m not in mods:
                    mods.append(m)
        return mods

    def step_weight_bytes(self) -> int:
        """Bytes of weights one step reads: every matrix of every run-list entry once, the output
        head, no embedding rows."""
        total = self.head.numel() * self.head.element_size() + self.final_norm.weight_bytes()
        for e in self.spec.run:
            total += sum(p.weight_bytes() for p in self.blocks[e.layer].parts().values())
        return total

    # ------------------------------------------------------------------ cache needs
    def cache_needs(self) -> List[Tuple[Optional[PagedCacheSpec], Optional[StateSpec]]]:
        """One pair per entry of the run list; entries that read another entry's cache report None pages."""
        out = []
        for e in self.spec.run:
            m: Mixer = self.blocks[e.layer].mixer()
            out.append((m.cache_spec() if e.kv_from is None else None, m.state_spec()))
        return out

    # ------------------------------------------------------------------ one step
    def forward(self, ctx: StepContext, caches: List[LayerCache], logit_rows: torch.Tensor) -> torch.Tensor:
        """``caches[i]`` belongs to entry ``i`` of the run list.  ``logit_rows``: int32 indices of the
        tokens of the step whose logits are wanted.  Returns float32 ``[len(logit_rows), vocab]``."""
        T = ctx.num_tokens
        residual = torch.empty((T, self.spec.hidden_size), dtype=torch.float32, device=self.device)
        ops.embedding(ctx.token_ids, self.embedding, residual, ctx.error_flag)
        if self.spec.embedding_scale is not None:
            residual.mul_(self.spec.embedding_scale)
        delta = None
        for entry, cache in zip(self.spec.run, caches):
            residual, delta = self.blocks[entry.layer].forward(residual, delta, ctx, cache)
        n = logit_rows.numel()
        if n == 0:
            # the blocks still ran: their cache writes are the step's effect
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        y = self.final_norm.add_forward_rows(delta, residual, logit_rows, self.dtype)
        logits = ops.linear(y, self.head, out_dtype=torch.float32)
        if self.spec.logit_scale is not None:
            logits.mul_(self.spec.logit_scale)
        return logits
