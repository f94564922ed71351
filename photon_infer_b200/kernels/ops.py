"""Python side of the CUDA kernels: argument checks, pointers, the current stream.

Every function takes CUDA tensors and launches on ``torch.cuda.current_stream()``.
There is no CPU path: a tensor that is not on a CUDA device raises, and so does a
missing or failing extension (``csrc/build.py``).  A kernel that cannot run a size
correctly refuses it (``UNSUPPORTED_SIZE``) instead of giving a wrong result.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from ..csrc.build import load_module
from ..errors import ErrorCode, PhotonError

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_launch_count = 0


def launch_count() -> int:
    """Kernels of this package launched so far in this process."""
    return _launch_count


_sm_counts = {}


def sm_count(device) -> int:
    """Streaming multiprocessors of ``device`` (asked once)."""
    key = (device.type, device.index)
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[key]


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT,
                              "a tensor on the CPU was passed to a CUDA kernel; there is no CPU path")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(t.data_ptr() if t is not None else 0)


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, what: str) -> None:
    global _launch_count
    if status == 0:
        _launch_count += 1
        return
    if status == -2:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, f"{what}: this size is not supported by the kernel")
    if status == -3:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"{what}: invalid argument")
    raise PhotonError(ErrorCode.CUDA_ERROR, f"{what}: CUDA error {status}")


_sigs_done = set()


def _fn(module: str, name: str, argtypes, defines=None):
    lib = load_module(module, defines)
    f = getattr(lib, name)
    key = (id(lib), name)
    if key not in _sigs_done:
        f.argtypes = argtypes
        f.restype = c_int
        _sigs_done.add(key)
    return f


def _int32(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"{what} must be a contiguous int32 tensor")


# ----------------------------------------------------------------------------- row kernels

def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor]) -> None:
    """``out[t, :] = table[ids[t], :]`` as float32; ids outside the table set the error word."""
    _cuda(ids, table, out, err)
    _int32(ids, "ids")
    T, (V, H) = ids.numel(), table.shape
    if out.dtype != torch.float32 or out.shape != (T, H) or not out.is_contiguous() or not table.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "embedding: out must be contiguous float32 [T, H]")
    f = _fn("elementwise", "photon_embedding",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(ids), _ptr(table), _dtype_code(table), _ptr(out), T, H, V, _ptr(err), _stream()), "embedding")


def add_rmsnorm(delta: Optional[torch.Tensor], residual: torch.Tensor, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """``residual += delta`` in float32 (in place; skipped when ``rows`` is given), then
    ``out = weight * (residual / sqrt(mean(residual^2) + eps))``.  With ``rows`` (int32 list)
    only those rows are read and ``out`` has one row per list entry."""
    _cuda(delta, residual, weight, out, rows)
    H = residual.shape[-1]
    n = rows.numel() if rows is not None else residual.shape[0]
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "add_rmsnorm: the residual stream must be contiguous float32")
    if delta is not None and (delta.shape != residual.shape or not delta.is_contiguous()):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "add_rmsnorm: delta must match the residual stream")
    if out.shape != (n, H) or not out.is_contiguous() or weight.numel() != H:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "add_rmsnorm: out must be [rows, H] and weight [H]")
    if rows is not None:
        _int32(rows, "rows")
    f = _fn("elementwise", "photon_add_rmsnorm",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(delta), _dtype_code(delta) if delta is not None else F32, _ptr(residual), _ptr(weight),
             _dtype_code(weight), _ptr(out), _dtype_code(out), _ptr(rows), n, H, float(eps), _stream()),
           "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]``."""
    _cuda(gate_up, out)
    T, I2 = gate_up.shape
    if I2 % 2 or out.shape != (T, I2 // 2) or out.dtype != gate_up.dtype \
            or not gate_up.is_contiguous() or not out.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "swiglu: gate_up [T, 2I] and out [T, I] of one dtype")
    f = _fn("elementwise", "photon_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), _dtype_code(out), T, I2 // 2, _stream()), "swiglu")


# ----------------------------------------------------------------------------- rope and cache write

def rope_kv_write(q: Optional[torch.Tensor], k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                  positions: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], interleaved: bool,
                  slot_mapping: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                  v_cache: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int,
                  err: Optional[torch.Tensor]) -> None:
    """Rotates ``q [T, n_q * d]`` and ``k [T, n_kv * d]`` in place (when ``inv_freq`` is given)
    and stores ``k`` and ``v [T, n_kv * d]`` at ``slot_mapping`` in the paged cache
    ``[pages, n_kv, page_size, d]`` (when the caches are given).  The three inputs may be
    views with any row stride, e.g. sections of one fused row."""
    _cuda(q, k, v, positions, inv_freq, slot_mapping, k_cache, v_cache, err)
    ref = q if q is not None else k
    if ref is None:
        return
    T = ref.shape[0]
    for name, t, heads in (("q", q, n_q), ("k", k, n_kv), ("v", v, n_kv)):
        if t is None:
            continue
        if t.dim() == 3:
            ok = t.shape == (T, heads, head_dim) and t.stride(2) == 1 and t.stride(1) == head_dim
        else:
            ok = t.shape == (T, heads * head_dim) and t.stride(1) == 1
        if not ok or t.dtype != ref.dtype:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH,
                              f"rope_kv_write: {name} must be [T, {heads} * {head_dim}] with contiguous heads")
    rotate = inv_freq is not None
    write = k_cache is not None
    page_size, num_slots = 1, 0
    if rotate:
        _int32(positions, "positions")
        if inv_freq.dtype != torch.float32 or inv_freq.numel() != head_dim // 2 or head_dim % 2:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "rope_kv_write: inv_freq must be float32 [head_dim / 2]")
    if write:
        if k is None or v is None:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "rope_kv_write: storing needs k and v")
        _int32(slot_mapping, "slot_mapping")
        if k_cache.dtype != ref.dtype or v_cache.dtype != ref.dtype or k_cache.shape != v_cache.shape \
                or k_cache.dim() != 4 or k_cache.shape[1] != n_kv or k_cache.shape[3] != head_dim \
                or not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH,
                              "rope_kv_write: caches must be contiguous [pages, n_kv, page_size, head_dim] of the run dtype")
        page_size = k_cache.shape[2]
        num_slots = k_cache.shape[0] * page_size
    f = _fn("rope_kv", "photon_rope_kv_write",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_void_p, c_int, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_long, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0) if q is not None else 0, _ptr(k), k.stride(0) if k is not None else 0,
             _ptr(v), v.stride(0) if v is not None else 0, _dtype_code(ref), _ptr(positions), _ptr(inv_freq),
             int(interleaved), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), T, n_q, n_kv, head_dim,
             page_size, num_slots, int(rotate), int(write), _ptr(err), _stream()), "rope_kv_write")


# ----------------------------------------------------------------------------- attention

def paged_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, token_seq: torch.Tensor, positions: torch.Tensor,
                    n_q: int, n_kv: int, head_dim: int, window: Optional[int], scale: float,
                    err: Optional[torch.Tensor]) -> None:
    """General paged causal attention.  ``q`` is a ``[T, n_q * d]`` view (row stride free),
    ``out [T, n_q * d]``; the token at position ``p`` of request ``token_seq[t]`` sees keys
    ``max(0, p - window + 1) .. p`` through ``block_table[seq]``."""
    _cuda(q, out, k_cache, v_cache, block_table, token_seq, positions, err)
    T = q.shape[0]
    if q.shape[1] != n_q * head_dim or q.stride(1) != 1 or out.shape != (T, n_q * head_dim) or out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "paged_attention: q and out must be [T, n_q * head_dim]")
    if q.dtype != out.dtype or q.dtype != k_cache.dtype or q.dtype != v_cache.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "paged_attention: q, out and the caches must share one dtype")
    if n_kv <= 0 or n_q % n_kv or head_dim % 2:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "paged_attention: n_q must be a multiple of n_kv and head_dim even")
    if (n_q // n_kv) * head_dim > 4096:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE,
                          f"paged_attention: heads per group x head_dim = {(n_q // n_kv) * head_dim} exceeds 4096")
    for name, t in (("block_table", block_table), ("token_seq", token_seq), ("positions", positions)):
        _int32(t, name)
    f = _fn("attention", "photon_paged_attention",
            [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _dtype_code(q), _ptr(k_cache), _ptr(v_cache),
             _ptr(block_table), block_table.shape[1], _ptr(token_seq), _ptr(positions), T, n_q, n_kv, head_dim,
             k_cache.shape[2], k_cache.shape[0], int(window) if window else 0, float(scale), _ptr(err), _stream()),
           "paged_attention")


_ticket_buffers = {}


def _attention_tickets(device) -> torch.Tensor:
    """Zeroed tickets, one per (token, key/value head); the kernel puts them back to zero."""
    key = (device.type, device.index)
    if key not in _ticket_buffers:
        _ticket_buffers[key] = torch.zeros(1 << 16, dtype=torch.int32, device=device)
    return _ticket_buffers[key]


def reset_tickets(device) -> None:
    """Puts the ticket counters of the split-key attention and of the split-K products back to zero.  The
    kernels do that themselves after every launch; a launch that gave up (the error word says so) may not."""
    key = (device.type, device.index)
    if key in _ticket_buffers:
        _ticket_buffers[key].zero_()
    if key in _skinny_buffers:
        _skinny_buffers[key][1].zero_()


def flash_attention_supported(dtype: torch.dtype, head_dim: int) -> bool:
    """The tensor-core kernel takes bfloat16 and head sizes that are a multiple of 16 up to 128."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128


def flash_attention_max_groups(head_dim: int) -> int:
    """Groups of four warps that the split-key kernel can run in one block at this head size (4, 2 or 1)."""
    lib = load_module("attention_flash", {"HEAD_DIM": head_dim})
    return int(lib.photon_flash_attention_max_groups())


def flash_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, cu_tokens: torch.Tensor, positions: torch.Tensor,
                    num_seqs: int, max_tokens_per_seq: int, n_q: int, n_kv: int, head_dim: int,
                    window: Optional[int], scale: float, num_splits: int, scratch: Optional[torch.Tensor],
                    rows_mode: bool, keys_mode: bool, err: Optional[torch.Tensor],
                    context_lens: Optional[torch.Tensor] = None, key_groups: int = 1) -> None:
    """Paged causal attention on the tensor cores.  ``cu_tokens [S + 1]`` gives each request's
    tokens in the step.  ``rows_mode``: run requests with more than 16 rows (tokens x heads per
    group); ``keys_mode``: run the others, their keys split over ``num_splits`` blocks.
    ``scratch``: float32, at least ``T * n_q * num_splits * (head_dim + 2)`` when ``num_splits > 1``.
    ``context_lens [S]`` (optional): tokens of each request after this step; the split-key kernel then
    derives positions from it (a request's tokens of the step are its last ones) and saves a round trip.
    ``key_groups``: 1, 2 or 4 groups of four warps per block of the split-key kernel, each walking its own
    share of the block's keys (``flash_attention_max_groups`` bounds it); their results are merged in shared
    memory, which is far cheaper than the merge of ``num_splits`` blocks through global memory."""
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, positions, scratch, err, context_lens)
    if context_lens is not None:
        _int32(context_lens, "context_lens")
        if context_lens.numel() < num_seqs:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "flash_attention: context_lens must cover every request")
    T = q.shape[0]
    if not flash_attention_supported(q.dtype, head_dim) or n_kv <= 0 or n_q % n_kv:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, f"flash_attention: head_dim {head_dim} in {q.dtype} is not supported")
    if q.shape[1] != n_q * head_dim or q.stride(1) != 1 or out.shape != (T, n_q * head_dim) or not out.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "flash_attention: q and out must be [T, n_q * head_dim]")
    if out.dtype != q.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "flash_attention: q, out and the caches must be bfloat16")
    for name, t in (("block_table", block_table), ("cu_tokens", cu_tokens), ("positions", positions)):
        _int32(t, name)
    if cu_tokens.numel() < num_seqs + 1 or block_table.shape[0] < num_seqs:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "flash_attention: cu_tokens and block_table must cover every request")
    part_acc = part_ml = tickets = None
    splits = int(num_splits) if keys_mode else 1
    if splits > 1:
        need = T * n_q * splits * (head_dim + 2)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need or not scratch.is_contiguous():
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"flash_attention: scratch must hold {need} float32 values")
        part_acc = scratch
        part_ml = scratch[T * n_q * splits * head_dim:]
        tickets = _attention_tickets(q.device)
        if tickets.numel() < num_seqs * n_kv:
            raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "flash_attention: too many requests for the ticket buffer")
    mode = (1 if rows_mode else 0) | (2 if keys_mode else 0)
    f = _fn("attention_flash", "photon_flash_attention",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
             c_int, c_void_p, c_void_p],
            defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(cu_tokens), _ptr(positions), _ptr(context_lens), _ptr(part_acc), _ptr(part_ml),
             _ptr(tickets),
             int(num_seqs), int(max_tokens_per_seq), n_q, n_kv, head_dim, k_cache.shape[2], k_cache.shape[0],
             int(window) if window else 0, float(scale), splits, int(key_groups) if keys_mode else 1, mode, _ptr(err),
             _stream()), "flash_attention")
    if rows_mode and keys_mode:
        global _launch_count
        _launch_count += 1


def attention_decode_supported(dtype: torch.dtype, head_dim: int, group: int, page_size: int, num_seqs: int) -> bool:
    """The persistent TMA kernel for decoded tokens: bfloat16, head size 64 or 128, up to 16 heads per
    key/value head, pages of 8, 16, 32 or a multiple of 64 tokens, up to 512 requests in the step."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and 1 <= group <= 16 and num_seqs <= 512
            and page_size % 8 == 0 and page_size >= 8 and (64 % page_size == 0 or page_size % 64 == 0))


def attention_decode_slots(head_dim: int) -> int:
    """Blocks of the persistent decode-attention kernel that the current device holds at once."""
    lib = load_module("attention_decode", {"HEAD_DIM": head_dim})
    return int(lib.photon_attention_decode_slots())


def attention_decode_plan(num_seqs: int, n_kv: int, max_keys: int, head_dim: int, page_size: int):
    """(tiles of 64 keys per work item, chunks to reserve scratch for, upper bound of the work items) for a step of
    ``num_seqs`` requests of at most ``max_keys`` visible keys; None when a request has more keys than the kernel
    takes (min(120, head size) chunks of 64 tiles of 64 keys: about 490,000 at heads of 128, 260,000 at heads of 64).

    A request's keys are cut into ``p`` chunks; a (chunk, key/value head) is a work item that one of the resident
    blocks draws.  ``p`` minimises ``rounds * (tiles per item + 5) + 0.3 * p`` with ``rounds = ceil(items / blocks)``:
    an item costs about five tile times beside its tiles (Q, the first round trip, the merge of its four warps), a
    chunk a partial result written and merged, and what decides most is how many items the busiest block gets.
    Measured on B200: 64 requests of 640 keys run best whole (26 us against 45 us in chunks of four tiles); 8
    requests x 8 heads of 16,500 keys: five chunks each are 320 items for 296 blocks, two rounds of 52 tiles (95
    us), chunks of four tiles 154 us."""
    slots = attention_decode_slots(head_dim)
    tiles = -(-max(max_keys, 1) // 64) + 1              # a window may start inside a tile
    most = 64                                           # tiles an item may have
    pairs = max(1, num_seqs * n_kv)
    best = None
    for p in range(-(-tiles // most), min(120, head_dim, tiles) + 1):     # the kernel merges up to min(120, head_dim) chunks
        chunk = -(-tiles // p)
        if -(-tiles // chunk) != p:
            continue                                    # the same chunk length as a smaller p
        rounds = -(-(pairs * p) // slots)
        cost = rounds * (chunk + 5) + (0.3 * p if p > 1 else 0.0)
        if best is None or cost < best[0]:
            best = (cost, chunk, p)
    if best is None:
        return None                                     # more keys than 120 chunks of 64 tiles hold
    _, chunk, per_seq = best
    return chunk, num_seqs * per_seq, num_seqs * per_seq * n_kv


_decode_scratch = {}


def attention_decode_scratch(device, floats: int) -> torch.Tensor:
    """The partial results of ``attention_decode``: one float32 buffer per device of at least ``floats`` elements.
    It grows by doubling and the buffers it outgrew are kept, because a captured CUDA graph holds the address it
    was captured with; a tensor that died with the step would leave the graph writing into memory that has a
    new owner."""
    key = (device.type, device.index)
    buffers = _decode_scratch.setdefault(key, [])
    if not buffers or buffers[-1].numel() < floats:
        size = max(int(floats), 2 * buffers[-1].numel() if buffers else 0, 1 << 20)
        buffers.append(torch.empty(size, dtype=torch.float32, device=device))
    return buffers[-1]


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_table: torch.Tensor, cu_tokens: torch.Tensor, context_lens: torch.Tensor, num_seqs: int,
                     n_q: int, n_kv: int, head_dim: int, window: Optional[int], scale: float, chunk_tiles: int,
                     scratch: torch.Tensor, scratch_chunks: int, max_items: int, err: Optional[torch.Tensor]) -> None:
    """Attention of the requests that bring at most 16 rows (tokens x heads per group) in this step, by the
    persistent TMA kernel (``attention_decode.cu``); the rows of the other requests are left untouched.
    ``context_lens [S]``: tokens of each request after this step (a request's tokens of the step are its last).
    ``scratch``: float32, at least ``scratch_chunks * n_kv * 16 * (head_dim + 2)``; ``scratch_chunks`` at least the
    chunks of ``chunk_tiles`` tiles that all requests have together (``attention_decode_plan``)."""
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, context_lens, scratch, err)
    T = q.shape[0]
    if n_kv <= 0 or n_q % n_kv or not attention_decode_supported(q.dtype, head_dim, n_q // n_kv, k_cache.shape[2], num_seqs):
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE,
                          f"attention_decode: head_dim {head_dim}, {n_q}/{n_kv} heads, pages of {k_cache.shape[2]} in {q.dtype} is not supported")
    if q.shape[1] != n_q * head_dim or q.stride(1) != 1 or out.shape != (T, n_q * head_dim) or not out.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "attention_decode: q and out must be [T, n_q * head_dim]")
    if out.dtype != q.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "attention_decode: q, out and the caches must be bfloat16")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "attention_decode: the caches must be contiguous [pages, n_kv, page, d]")
    for name, t in (("block_table", block_table), ("cu_tokens", cu_tokens), ("context_lens", context_lens)):
        _int32(t, name)
    if cu_tokens.numel() < num_seqs + 1 or block_table.shape[0] < num_seqs or context_lens.numel() < num_seqs:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "attention_decode: cu_tokens, context_lens and block_table must cover every request")
    need = scratch_chunks * n_kv * 16 * (head_dim + 2)
    if scratch.dtype != torch.float32 or scratch.numel() < need or not scratch.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"attention_decode: scratch must hold {need} float32 values")
    tickets = _attention_tickets(q.device)
    if tickets.numel() < num_seqs * n_kv + 2:      # the tickets, then the kernel's two work counters
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "attention_decode: too many requests for the ticket buffer")
    part_ml = scratch[scratch_chunks * n_kv * 16 * head_dim:]
    f = _fn("attention_decode", "photon_attention_decode",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
             c_long, c_void_p, c_void_p],
            defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(cu_tokens), _ptr(context_lens), _ptr(scratch), _ptr(part_ml), int(scratch_chunks),
             _ptr(tickets), int(num_seqs), T, n_q, n_kv, head_dim, k_cache.shape[2], k_cache.shape[0],
             int(window) if window else 0, float(scale), int(chunk_tiles), max(1, -(-int(scratch_chunks) // max(num_seqs, 1))),
             int(max_items), _ptr(err), _stream()),
           "attention_decode")


# PHOTON_ATTENTION_TC=0 keeps prompt portions on the mma.sync kernel (for comparisons)
USE_ATTENTION_TC = os.environ.get("PHOTON_ATTENTION_TC", "1") != "0"


def attention_tc_supported(dtype: torch.dtype, head_dim: int, group: int, page_size: int) -> bool:
    """The tcgen05 kernel for prompt portions: bfloat16, head size 64 or 128, up to 128 heads per
    key/value head and pages of 8, 16, 32 or a multiple of 64 tokens."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and 1 <= group <= 128
            and page_size % 8 == 0 and page_size >= 8 and (64 % page_size == 0 or page_size % 64 == 0))


def attention_tc(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 block_table: torch.Tensor, cu_tokens: torch.Tensor, positions: torch.Tensor,
                 num_seqs: int, max_tokens_per_seq: int, n_q: int, n_kv: int, head_dim: int,
                 window: Optional[int], scale: float, err: Optional[torch.Tensor]) -> None:
    """Paged causal attention of the requests that bring more than 16 rows (tokens x heads per
    group) in this step, on the tcgen05 tensor cores; the rows of the other requests are left
    untouched (``flash_attention`` with ``keys_mode`` takes them)."""
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, positions, err)
    T = q.shape[0]
    if n_kv <= 0 or n_q % n_kv or not attention_tc_supported(q.dtype, head_dim, n_q // n_kv, k_cache.shape[2]):
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE,
                          f"attention_tc: head_dim {head_dim}, {n_q}/{n_kv} heads, pages of {k_cache.shape[2]} in {q.dtype} is not supported")
    if q.shape[1] != n_q * head_dim or q.stride(1) != 1 or out.shape != (T, n_q * head_dim) or not out.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "attention_tc: q and out must be [T, n_q * head_dim]")
    if out.dtype != q.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "attention_tc: q, out and the caches must be bfloat16")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "attention_tc: the caches must be contiguous [pages, n_kv, page, d]")
    for name, t in (("block_table", block_table), ("cu_tokens", cu_tokens), ("positions", positions)):
        _int32(t, name)
    if cu_tokens.numel() < num_seqs + 1 or block_table.shape[0] < num_seqs:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "attention_tc: cu_tokens and block_table must cover every request")
    f = _fn("attention_tc", "photon_attention_tc",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
            defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(cu_tokens), _ptr(positions), int(num_seqs), int(max_tokens_per_seq), T,
             n_q, n_kv, head_dim, k_cache.shape[2], k_cache.shape[0], int(window) if window else 0, float(scale),
             _ptr(err), _stream()), "attention_tc")


# ----------------------------------------------------------------------------- matrix products

SKINNY_MAX_ROWS = 8         # up to this many rows the weight-streaming kernel runs instead of the library


def skinny_gemm_supported(x: torch.Tensor, weight: torch.Tensor, swiglu: bool = False) -> bool:
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 1 <= M <= (32 if swiglu else 64)
            and K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


_skinny_buffers = {}


def _skinny_scratch(device):
    """One scratch buffer and one ticket array per device for the split of K over blocks; launches
    on one stream use them one after the other."""
    key = (device.type, device.index)
    if key not in _skinny_buffers:
        _skinny_buffers[key] = (torch.empty(1 << 20, dtype=torch.float32, device=device),
                                torch.zeros(8192, dtype=torch.int32, device=device))
    return _skinny_buffers[key]


def skinny_gemm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "bf16") -> None:
    """``out = x @ weight^T`` for few rows, the weights streamed once.  ``epilogue``: ``"bf16"``,
    ``"f32"`` (float output) or ``"swiglu"`` (``weight`` holds gate rows then up rows; ``out`` is
    ``[M, I]`` with ``silu(gate) * up``)."""
    _cuda(x, weight, out)
    M, K = x.shape
    N = weight.shape[0]
    code = {"bf16": 0, "f32": 1, "swiglu": 2}[epilogue]
    cols = N // 2 if epilogue == "swiglu" else N
    want = torch.float32 if epilogue == "f32" else torch.bfloat16
    if not skinny_gemm_supported(x, weight, epilogue == "swiglu") or weight.shape[1] != K:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "skinny_gemm: needs bfloat16, K a multiple of 8, aligned rows, few rows of x")
    if out.shape != (M, cols) or out.dtype != want or out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"skinny_gemm: out must be {want} [{M}, {cols}]")
    scratch, tickets = _skinny_scratch(x.device)
    f = _fn("gemm_skinny", "photon_skinny_gemm",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p, c_long,
             c_void_p, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, code,
             _ptr(scratch), scratch.numel(), _ptr(tickets), tickets.numel(), _stream()), "skinny_gemm")


def skinny_fused_supported(residual: torch.Tensor, weight: torch.Tensor) -> bool:
    """The decode-step product with the residual add and the norm folded in: up to 8 rows of a contiguous
    float32 residual stream, bfloat16 weights, K a multiple of 8."""
    M, K = residual.shape
    return (residual.dtype == torch.float32 and residual.is_contiguous() and weight.dtype == torch.bfloat16
            and weight.is_contiguous() and 1 <= M <= 8 and K % 8 == 0 and weight.shape[1] == K
            and weight.data_ptr() % 16 == 0 and residual.data_ptr() % 16 == 0)


def skinny_fused(residual: torch.Tensor, delta: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                 weight: torch.Tensor, epilogue: str, rope: Optional[dict] = None,
                 err: Optional[torch.Tensor] = None):
    """``x = residual + delta``; ``out = epilogue(rmsnorm(x; norm_weight, eps) @ weight^T)`` in one kernel.
    Returns ``(out, new_residual)``; the input residual is left untouched (the sum goes to a new tensor).
    ``epilogue``: ``"bf16"``, ``"swiglu"`` (``weight`` = gate rows then up rows) or ``"qkv"`` with
    ``rope = dict(positions, inv_freq, slot_mapping, k_cache, v_cache, n_q, n_kv, head_dim)``: q and k are
    rotated (partners must be neighbouring rows of ``weight``), q is returned ``[M, n_q * d]`` wide in
    ``out[:, :n_q * d]``, k and v go into the paged cache."""
    _cuda(residual, delta, norm_weight, weight, err)
    M, K = residual.shape
    N = weight.shape[0]
    if not skinny_fused_supported(residual, weight):
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "skinny_fused: needs <= 8 float32 rows, bfloat16 weights, K % 8 == 0")
    if delta is not None and (delta.shape != residual.shape or delta.dtype != torch.bfloat16 or not delta.is_contiguous()
                              or delta.data_ptr() % 16):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "skinny_fused: delta must be contiguous bfloat16 like the residual")
    if norm_weight.numel() != K or norm_weight.data_ptr() % 16:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "skinny_fused: norm weight must be [K]")
    code = {"bf16": 0, "swiglu": 2, "qkv": 3}[epilogue]
    new_residual = torch.empty_like(residual) if delta is not None else residual
    r = rope or {}
    if epilogue == "qkv":
        n_q, n_kv, d = r["n_q"], r["n_kv"], r["head_dim"]
        if N != (n_q + 2 * n_kv) * d or d % 2:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "skinny_fused: weight must hold q, k and v rows")
        k_cache, v_cache = r["k_cache"], r["v_cache"]
        if k_cache.dtype != torch.bfloat16 or k_cache.shape != v_cache.shape or k_cache.dim() != 4 \
                or k_cache.shape[1] != n_kv or k_cache.shape[3] != d or not k_cache.is_contiguous() \
                or not v_cache.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "skinny_fused: caches must be contiguous bfloat16 [pages, n_kv, page, d]")
        _int32(r["positions"], "positions")
        _int32(r["slot_mapping"], "slot_mapping")
        out = torch.empty((M, n_q * d), dtype=torch.bfloat16, device=residual.device)
        page_size, num_slots = k_cache.shape[2], k_cache.shape[0] * k_cache.shape[2]
    else:
        n_q = n_kv = d = 0
        k_cache = v_cache = None
        page_size, num_slots = 1, 0
        out = torch.empty((M, N // 2 if epilogue == "swiglu" else N), dtype=torch.bfloat16, device=residual.device)
    if err is None:
        err = _error_word(residual.device)
    f = _fn("gemm_skinny_fused", "photon_skinny_fused",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
             c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_long,
             c_void_p, c_void_p])
    _check(f(_ptr(residual), _ptr(new_residual if delta is not None else None), _ptr(delta), _ptr(norm_weight),
             _dtype_code(norm_weight), float(eps), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K,
             code, _ptr(r.get("positions")), _ptr(r.get("inv_freq")), _ptr(r.get("slot_mapping")), _ptr(k_cache),
             _ptr(v_cache), n_q, n_kv, d, page_size, num_slots, _ptr(err), _stream()), "skinny_fused")
    return out, new_residual


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)`` with ``w_gate_up = [Wg; Wu]``: one kernel for few rows, else the
    product followed by the SwiGLU kernel."""
    M = x.shape[0]
    I = w_gate_up.shape[0] // 2
    out = torch.empty((M, I), dtype=x.dtype, device=x.device)
    if M <= SKINNY_MAX_ROWS and skinny_gemm_supported(x, w_gate_up, swiglu=True):
        skinny_gemm(x, w_gate_up, out, "swiglu")
        return out
    if gemm_tc_supported(x, w_gate_up) and gemm_tc_tiles(M, 2 * I, swiglu=True) >= TC_MIN_TILES:
        gemm_tc(x, w_gate_up, out, "swiglu", pair=M >= TC_PAIR_MIN_ROWS)
        return out
    swiglu(linear(x, w_gate_up), out)
    return out


_error_words = {}


def set_error_word(flag: torch.Tensor) -> None:
    """The int32[4] word in which kernels called without an explicit one report a wait that ran out."""
    _error_words[(flag.device.type, flag.device.index)] = flag


def _error_word(device) -> Optional[torch.Tensor]:
    return _error_words.get((device.type, device.index))


TC_MIN_TILES = 96           # below this many 128 x 256 tiles the tcgen05 product leaves too many SMs idle
TC_PAIR_MIN_ROWS = 256      # from here on tiles of 256 x 256 on pairs of SMs (gemm_tc2.cu): a third less operand traffic


def gemm_tc_tiles(M: int, N: int, swiglu: bool = False) -> int:
    """Tiles the tcgen05 product would run; 0 when a tile of 128 rows would be mostly padding."""
    if M < 128:
        return 0
    cols = N // 2 if swiglu else N
    return -(-M // 128) * -(-cols // (128 if swiglu else 256))


def gemm_tc_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """The tcgen05 product takes bfloat16, K a multiple of 8 and 16-byte aligned rows (TMA)."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "bf16",
            err: Optional[torch.Tensor] = None, pair: bool = False) -> None:
    """``out = x @ weight^T`` on the tcgen05 tensor cores (TMA operands, accumulator in tensor memory).
    ``epilogue``: ``"bf16"``, ``"f32"`` or ``"swiglu"`` (``weight`` holds gate rows then up rows; ``out``
    is ``[M, I]``).  ``pair``: tiles of 256 x 256 on pairs of SMs (``gemm_tc2.cu``) instead of 128 x 256
    on one."""
    _cuda(x, weight, out, err)
    M, K = x.shape
    N = weight.shape[0]
    code = {"bf16": 0, "f32": 1, "swiglu": 2}[epilogue]
    cols = N // 2 if epilogue == "swiglu" else N
    want = torch.float32 if epilogue == "f32" else torch.bfloat16
    if not gemm_tc_supported(x, weight) or weight.shape[1] != K:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "gemm_tc: needs bfloat16, K a multiple of 8 and aligned rows")
    if out.shape != (M, cols) or out.dtype != want or out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"gemm_tc: out must be {want} [{M}, {cols}]")
    module, entry = ("gemm_tc2", "photon_gemm_tc2") if pair else ("gemm_tc", "photon_gemm_tc")
    f = _fn(module, entry,
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    if err is None:
        err = _error_word(x.device)
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, code,
             _ptr(err), _stream()), module)


def rope_table(inv_freq: torch.Tensor, count: int) -> torch.Tensor:
    """``(cos, sin)`` of ``position * inv_freq[j]`` for positions below ``count``, float32
    ``[count, len(inv_freq), 2]``, computed on the device with the expression the rotary kernels use."""
    _cuda(inv_freq)
    if inv_freq.dtype != torch.float32 or not inv_freq.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "rope_table: inv_freq must be contiguous float32")
    half = inv_freq.numel()
    out = torch.empty((int(count), half, 2), dtype=torch.float32, device=inv_freq.device)
    f = _fn("rope_kv", "photon_rope_table", [c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(inv_freq), half, int(count), _ptr(out), _stream()), "rope_table")
    return out


def gemm_tc_qkv_supported(x: torch.Tensor, w_qkv: torch.Tensor, head_dim: int) -> bool:
    """The q/k/v product with rotation and cache write in its epilogue: the tcgen05 kernel on pairs of SMs with
    enough tiles, heads that are a multiple of 32 wide."""
    M = x.shape[0]
    return (gemm_tc_supported(x, w_qkv) and M >= TC_PAIR_MIN_ROWS and head_dim % 32 == 0
            and gemm_tc_tiles(M, w_qkv.shape[0]) >= TC_MIN_TILES)


def gemm_tc_qkv(x: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                slot_mapping: torch.Tensor, inv_freq: torch.Tensor, table: Optional[torch.Tensor],
                k_cache: torch.Tensor, v_cache: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                err: Optional[torch.Tensor] = None) -> None:
    """``x @ w_qkv^T`` (rows of q, then k, then v; rotation partners of q and k as neighbours) with the
    rotation and the cache write in the epilogue: rotated queries to ``q_out [M, n_q * d]``, rotated keys and
    the values to ``slot_mapping`` of the paged cache ``[pages, n_kv, page_size, d]``.  ``table``: from
    ``rope_table`` (positions beyond it are computed in place)."""
    _cuda(x, w_qkv, q_out, positions, slot_mapping, inv_freq, table, k_cache, v_cache, err)
    M, K = x.shape
    if not gemm_tc_supported(x, w_qkv) or w_qkv.shape != ((n_q + 2 * n_kv) * head_dim, K) or head_dim % 32:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "gemm_tc_qkv: needs bfloat16, K a multiple of 8, aligned rows, "
                          "head_dim a multiple of 32 and a weight of (n_q + 2 n_kv) * head_dim rows")
    if q_out.shape != (M, n_q * head_dim) or q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"gemm_tc_qkv: q_out must be bfloat16 [{M}, {n_q * head_dim}]")
    for name, t in (("positions", positions), ("slot_mapping", slot_mapping)):
        _int32(t, name)
        if t.numel() < M:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"gemm_tc_qkv: {name} must have an entry per row")
    if k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16 or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape or k_cache.shape[1] != n_kv \
            or k_cache.shape[3] != head_dim:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "gemm_tc_qkv: the caches must be contiguous bfloat16 [pages, n_kv, page, d]")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != head_dim // 2:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "gemm_tc_qkv: inv_freq must be float32 [head_dim / 2]")
    count = 0
    if table is not None:
        if table.dtype != torch.float32 or table.dim() != 3 or table.shape[1:] != (head_dim // 2, 2) or not table.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "gemm_tc_qkv: table must be float32 [positions, head_dim / 2, 2]")
        count = table.shape[0]
    f = _fn("gemm_tc2", "photon_gemm_tc2_qkv",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_long, c_void_p, c_void_p])
    if err is None:
        err = _error_word(x.device)
    _check(f(_ptr(x), x.stride(0), _ptr(w_qkv), w_qkv.stride(0), _ptr(q_out), q_out.stride(0), M, K, _ptr(positions),
             _ptr(slot_mapping), _ptr(inv_freq), _ptr(table), count, _ptr(k_cache), _ptr(v_cache), n_q, n_kv, head_dim,
             k_cache.shape[2], k_cache.shape[0] * k_cache.shape[2], _ptr(err), _stream()), "gemm_tc_qkv")


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M, K] @ weight[N, K]^T``.  float32: this package's FMA kernel (true 32-bit).
    bfloat16: up to 8 rows the weight-streaming kernel; with enough 128 x 256 tiles to fill the
    GPU the tcgen05 kernel; in between the library product (cuBLAS through torch), where the
    reference's engine also calls the library (src/ops/kernels/cuda/matmul_dequant_cached.cu:193-207)."""
    _cuda(x, weight, out)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or x.stride(1) != 1 or not weight.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"linear: x [M, {K}] against weight {tuple(weight.shape)}")
    if x.dtype != weight.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"linear: x is {x.dtype}, weight is {weight.dtype}")
    want = out_dtype or x.dtype
    if M <= SKINNY_MAX_ROWS and want in (torch.bfloat16, torch.float32) and skinny_gemm_supported(x, weight):
        if out is None:
            out = torch.empty((M, N), dtype=want, device=x.device)
        skinny_gemm(x, weight, out, "f32" if want == torch.float32 else "bf16")
        return out
    if want in (torch.bfloat16, torch.float32) and gemm_tc_supported(x, weight) \
            and gemm_tc_tiles(M, N) >= TC_MIN_TILES and (out is None or out.stride(1) == 1):
        if out is None:
            out = torch.empty((M, N), dtype=want, device=x.device)
        gemm_tc(x, weight, out, "f32" if want == torch.float32 else "bf16", pair=M >= TC_PAIR_MIN_ROWS)
        return out
    if x.dtype == torch.float32:
        if want != torch.float32:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "linear: a float32 product gives float32")
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        f = _fn("gemm_f32", "photon_sgemm_nt",
                [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_void_p])
        _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, _stream()),
               "sgemm")
        return out
    if want == torch.float32:
        res = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is None:
        return torch.mm(x, weight.t())
    torch.mm(x, weight.t(), out=out)
    return out


# ----------------------------------------------------------------------------- sampling

def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], u: Optional[torch.Tensor],
           out: torch.Tensor) -> None:
    """Row-wise: first-maximum argmax where ``temperature <= 0`` (or None), else the first
    index whose running sum of ``softmax(logits / temperature)`` reaches ``u``."""
    _cuda(logits, temperature, u, out)
    rows, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "sample: logits must be float32 with unit inner stride")
    _int32(out, "out")
    if temperature is not None and (temperature.dtype != torch.float32 or temperature.numel() != rows
                                    or u is None or u.dtype != torch.float32 or u.numel() != rows):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "sample: temperature and u must be float32 [rows]")
    scratch = None
    if V > 16384:
        # long rows are cut into 32 spans that separate blocks reduce; their results meet here
        scratch = torch.empty(rows * 32 * 4, dtype=torch.float32, device=logits.device)
    f = _fn("sampling", "photon_sample", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), _ptr(temperature), _ptr(u), _ptr(out), rows, V, _ptr(scratch), _stream()),
           "sample")
    if scratch is not None:
        global _launch_count
        _launch_count += 1
