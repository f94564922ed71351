"""Grouped-query attention over the paged cache.

Order of work as src/arch/transformer_block.cpp:204-266: q, k, v projections (one
fused product here), rotation of q and k, keys and values into the cache, attention
of every token over the keys up to its own position, output projection.  The
reference's batched path rotates every row with the first token's position and lets
a token see later tokens of its own portion (src/arch/transformer_block.cpp:442-445,
486-509); here each token has its own position and its own causal limit.

``window`` None is full attention; an integer makes the same mixer a sliding-window
one, whose cache group gives pages back once the window has passed them.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, PagedCacheSpec, StepContext, TensorSpec
from .linear import project
from .registry import register_mixer
from .rope import RotaryEncoding


class PagedAttention(Mixer):
    kernel_modules = ("rope_kv", "attention")

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, head_dim: int,
                 position_encoding=None, window: Optional[int] = None, scale: Optional[float] = None):
        self.hidden_size = hidden_size
        self.n_q = n_q_heads
        self.n_kv = n_kv_heads
        self.head_dim = head_dim
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position_encoding = position_encoding
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.pairs_adjacent = False             # set at load: the convention the rotation kernel runs in
        self._max_groups: Optional[int] = None  # groups of warps per block of the split-key kernel, asked once

    def required_kernels(self, dtype):
        mods = list(self.kernel_modules)
        if dtype == torch.bfloat16:
            mods.extend(["gemm_skinny", "gemm_skinny_fused", "gemm_tc", "gemm_tc2"])
        if ops.flash_attention_supported(dtype, self.head_dim):
            mods.append(("attention_flash", {"HEAD_DIM": self.head_dim}))
        if dtype == torch.bfloat16 and self.head_dim in (64, 128) and ops.USE_ATTENTION_TC and self.n_q // self.n_kv <= 128:
            mods.append(("attention_tc", {"HEAD_DIM": self.head_dim}))
        if dtype == torch.bfloat16 and self.head_dim in (64, 128) and self.n_q // self.n_kv <= 16:
            mods.append(("attention_decode", {"HEAD_DIM": self.head_dim}))
        return mods

    # -- weights: separate q/k/v in the file, one fused matrix on the device
    def tensor_specs(self) -> List[TensorSpec]:
        d, H = self.head_dim, self.hidden_size
        return [TensorSpec("q_proj.weight", (self.n_q * d, H)),
                TensorSpec("k_proj.weight", (self.n_kv * d, H)),
                TensorSpec("v_proj.weight", (self.n_kv * d, H)),
                TensorSpec("o_proj.weight", (H, self.n_q * d))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        wq, wk = tensors["q_proj.weight"], tensors["k_proj.weight"]
        pe = self.position_encoding
        self.pairs_adjacent = bool(getattr(pe, "interleaved", False))
        if isinstance(pe, RotaryEncoding) and not pe.interleaved:
            # Files in the half-split convention pair feature j with j + d/2.  The rows of the q and k
            # projections are reordered inside every head to [0, d/2, 1, d/2 + 1, ...], which makes the
            # partners neighbours (the same rotation then runs in the neighbour convention) and leaves
            # every score q.k unchanged, because q and k are permuted alike.  Values are untouched.
            d = self.head_dim
            order = torch.stack([torch.arange(d // 2), torch.arange(d // 2) + d // 2], dim=1).reshape(-1)
            wq = wq.view(self.n_q, d, -1)[:, order.to(wq.device), :].reshape(self.n_q * d, -1)
            wk = wk.view(self.n_kv, d, -1)[:, order.to(wk.device), :].reshape(self.n_kv * d, -1)
            self.pairs_adjacent = True
        self.w_qkv = torch.cat([wq, wk, tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return PagedCacheSpec(self.n_kv, self.head_dim, self.window)

    # -- decode steps: residual sum, norm, q/k/v products, rotation and cache write in one kernel
    def fuses_norm(self, norm, residual, ctx, cache) -> bool:
        from .norm import RMSNorm
        return (isinstance(norm, RMSNorm) and ctx.dtype == torch.bfloat16 and not cache.shared
                and isinstance(self.position_encoding, RotaryEncoding) and self.pairs_adjacent
                and cache.k is not None and ops.skinny_fused_supported(residual, self.w_qkv))

    def forward_with_norm(self, residual, delta, norm, ctx, cache):
        group = ctx.groups[cache.group]
        pe = self.position_encoding
        q, residual = ops.skinny_fused(
            residual, delta, norm.weight, norm.eps, self.w_qkv, "qkv",
            rope=dict(positions=ctx.positions, inv_freq=pe.inv_freq, slot_mapping=group.slot_mapping, k_cache=cache.k,
                      v_cache=cache.v, n_q=self.n_q, n_kv=self.n_kv, head_dim=self.head_dim),
            err=ctx.error_flag)
        attn = torch.empty((q.shape[0], self.n_q * self.head_dim), dtype=q.dtype, device=q.device)
        self.attend(q, attn, ctx, cache)
        return project(attn, self.w_o), residual

    # -- one step
    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        d = self.head_dim
        group = ctx.groups[cache.group]
        pe = self.position_encoding
        if (not cache.shared and cache.k is not None and isinstance(pe, RotaryEncoding) and self.pairs_adjacent
                and h.dtype == torch.bfloat16 and ops.gemm_tc_qkv_supported(h, self.w_qkv, d)):
            # a long prompt portion: rotation and cache write ride in the epilogue of the q/k/v product
            q = torch.empty((T, self.n_q * d), dtype=h.dtype, device=h.device)
            ops.gemm_tc_qkv(h, self.w_qkv, q, ctx.positions, group.slot_mapping, pe.inv_freq,
                            pe.table(ctx.max_context_len), cache.k, cache.v, self.n_q, self.n_kv, d, ctx.error_flag)
            attn = torch.empty((T, self.n_q * d), dtype=h.dtype, device=h.device)
            self.attend(q, attn, ctx, cache)
            return project(attn, self.w_o)
        if cache.shared:
            # keys and values come from another entry's pages: only the queries are computed
            q = project(h, self.w_qkv[: self.n_q * d])
            k = v = None
        else:
            qkv = project(h, self.w_qkv)                              # [T, (n_q + 2 n_kv) d]
            q = qkv[:, : self.n_q * d]
            k = qkv[:, self.n_q * d: (self.n_q + self.n_kv) * d]
            v = qkv[:, (self.n_q + self.n_kv) * d:]
        pe = self.position_encoding
        k_cache, v_cache = (None, None) if cache.shared else (cache.k, cache.v)
        if isinstance(pe, RotaryEncoding):
            # rotation and cache write in one pass over the row
            ops.rope_kv_write(q, k, v, ctx.positions,
                              pe.inv_freq, self.pairs_adjacent, group.slot_mapping, k_cache, v_cache,
                              self.n_q, self.n_kv, d, ctx.error_flag)
        else:
            if pe is not None:
                pe.apply(q.view(T, self.n_q, d), None if k is None else k.view(T, self.n_kv, d), ctx.positions)
            if k_cache is not None:
                ops.rope_kv_write(None, k, v, None, None, False, group.slot_mapping, k_cache, v_cache,
                                  self.n_q, self.n_kv, d, ctx.error_flag)
        attn = torch.empty((T, self.n_q * d), dtype=h.dtype, device=h.device)
        self.attend(q, attn, ctx, cache)
        return project(attn, self.w_o)

    def attend(self, q: torch.Tensor, out: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        """bfloat16 with a head size the tensor-core kernel is compiled for: that kernel.  float32 and
        other sizes: the general kernel, whose sums depend only on a token's position."""
        group = ctx.groups[cache.group]
        gsize = self.n_q // self.n_kv
        if ops.flash_attention_supported(q.dtype, self.head_dim):
            # tensor cores: requests with many rows walk their keys in one block per 128 rows, requests
            # with few rows (decoded tokens) split their keys over blocks
            T = q.shape[0]
            few = [n * gsize <= 16 for n in ctx.host_query_lens]
            keys_mode, rows_mode = any(few), not all(few)
            splits, groups, scratch = 1, 1, None
            keys = ctx.max_context_len if self.window is None else min(self.window + ctx.max_query_len, ctx.max_context_len)
            # decoded tokens with long contexts: the persistent TMA kernel
            plan = None
            pairs = sum(few) * self.n_kv
            if keys_mode and (keys >= DECODE_TMA_MIN_KEYS.get(self.head_dim, 1 << 30)
                              or pairs * keys >= DECODE_TMA_MIN_WORK.get(self.head_dim, 1 << 60)) \
                    and ops.attention_decode_supported(q.dtype, self.head_dim, gsize, cache.k.shape[2], ctx.num_seqs):
                plan = ops.attention_decode_plan(sum(few), self.n_kv, keys, self.head_dim, cache.k.shape[2])
            decode_tma = plan is not None
            if keys_mode and not decode_tma:
                if self._max_groups is None:
                    self._max_groups = ops.flash_attention_max_groups(self.head_dim)
                splits, groups = choose_key_shares(sum(few) * self.n_kv, keys, self._max_groups, sms=ops.sm_count(q.device))
                # the kernel indexes its partial results by the token's place in the step, so beside a long prompt
                # portion every share costs T rows: no more shares than 64 MB of them
                per_share = T * self.n_q * (self.head_dim + 2) * 4
                splits = max(1, min(splits, (64 << 20) // per_share))
                if splits > 1:
                    scratch = torch.empty(T * self.n_q * splits * (self.head_dim + 2), dtype=torch.float32, device=q.device)
            if rows_mode and ops.USE_ATTENTION_TC and \
                    ops.attention_tc_supported(q.dtype, self.head_dim, gsize, cache.k.shape[2]):
                # prompt portions: tensor memory and TMA; the split-key kernel keeps the decoded tokens
                ops.attention_tc(q, out, cache.k, cache.v, group.block_table, ctx.cu_tokens, ctx.positions,
                                 ctx.num_seqs, ctx.max_query_len, self.n_q, self.n_kv, self.head_dim, self.window,
                                 self.scale, ctx.error_flag)
                rows_mode = False
            if decode_tma:
                chunk, chunks, items = plan
                # one scratch buffer per device, shared by the layers and steps (they run one after the other) and never
                # freed: a captured decode step keeps its address
                scratch = ops.attention_decode_scratch(q.device, chunks * self.n_kv * 16 * (self.head_dim + 2))
                ops.attention_decode(q, out, cache.k, cache.v, group.block_table, ctx.cu_tokens, ctx.context_lens,
                                     ctx.num_seqs, self.n_q, self.n_kv, self.head_dim, self.window, self.scale, chunk,
                                     scratch, chunks, items, ctx.error_flag)
                keys_mode = False
            if rows_mode or keys_mode:
                ops.flash_attention(q, out, cache.k, cache.v, group.block_table, ctx.cu_tokens, ctx.positions,
                                    ctx.num_seqs, ctx.max_query_len, self.n_q, self.n_kv, self.head_dim, self.window,
                                    self.scale, splits, scratch, rows_mode, keys_mode, ctx.error_flag,
                                    ctx.context_lens, groups)
            return
        ops.paged_attention(q, out, cache.k, cache.v, group.block_table, ctx.token_seq, ctx.positions,
                            self.n_q, self.n_kv, self.head_dim, self.window, self.scale, ctx.error_flag)


#: Contexts (keys a decoded token may see) from which the persistent TMA kernel takes the decoded tokens, by head
#: size.  Measured on B200 against the split-key kernel: heads of 128 are 20 to 45 % faster from 1,000 keys on at
#: every batch size tried (8 x 16,500 keys: 95 us against 156 us; 56 x 1,300: 63 against 112); heads of 64 move
#: half the bytes per tile and only gain with very long contexts (4 x 32,000 keys: 53 us against 68 us).
DECODE_TMA_MIN_KEYS = {128: 1000, 64: 8192}
#: ... or from this many (request, key/value head) pairs x keys on: with many requests the persistent kernel wins
#: earlier, because the split-key kernel has one block per pair and each block keeps a single tile in flight.
#: Measured with cold caches at 24/8 heads of 128: 64 requests x 256 keys 25 us against 30 us, x 768 keys 45 against
#: 73; 32 x 512: 23 against 24; 16 x 768: 23 against 18 (still the split-key kernel).  Heads of 64, 64 requests:
#: x 1,024 keys 36 against 34, x 2,048 keys 59 against 62.
DECODE_TMA_MIN_WORK = {128: 128 * 1024, 64: 1024 * 1024}


def choose_key_shares(pairs: int, max_keys: int, max_groups: int, tile: int = 64, sms: int = 148):  # sms: the caller passes the device's count
    """How the keys of a decoded token are shared out: (blocks per (request, key/value head), groups of
    four warps per block).  Measured on B200 (148 SMs) at 32/8 heads of 64:

    * up to one (request, key/value head) pair per SM: every block runs ``max_groups`` groups, each with a ring
      of stages of its own, merged through shared memory (batch 8, 640 keys: 9.2 us against 10.9 us for four
      blocks merged through global memory; batch 16: 9.4 against 14.8).  The keys are split over blocks as
      well only while a group keeps four tiles or more and the blocks do not outnumber the SMs (batch 8,
      4,096 keys: two blocks, 20.6 us against 28.0 us);
    * more pairs than SMs: one group per block, about 256 blocks, no share below one tile; more shares cost
      more in the merge than they gain.
    """
    tiles = -(-max(max_keys, 1) // tile)
    pairs = max(pairs, 1)
    if max_groups > 1 and pairs <= sms:
        by_fill = sms // pairs
        by_tiles = (tiles // max_groups) // 4
        return max(1, min(by_fill, by_tiles, 64)), max_groups
    by_fill = -(-256 // pairs)
    return max(1, min(by_fill, tiles, 64)), 1


register_mixer("full_attention", PagedAttention)
register_mixer("sliding_attention", PagedAttention)
