"""The step function: one batch of (request, its next tokens) through the model.

A step may hold portions of prompts beside single decoded tokens, cut anywhere.  It
runs only the tokens it is given, as one batch, against the cache that earlier steps
left, and returns 32-bit logits at the wanted places.  The reference's counterpart is
``LLaMAModel::forward_batched`` (src/arch/llama_model.cpp:483-605), which rebuilds and
uploads block tables in every layer (src/arch/transformer_block.cpp:455-465,496-509);
here all indices of a step are built once on the host and reach the device in one copy.
"""
from __future__ import annotations

import collections
import dataclasses
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..errors import ErrorCode, PhotonError
from ..models.model import CausalLM
from ..parts.base import GroupView, StepContext


@dataclasses.dataclass
class StepEntry:
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()            # indices into ``tokens`` whose logits are wanted


@dataclasses.dataclass
class StepResult:
    logits: torch.Tensor                # float32 [n_wanted, vocab] on the device
    rows: List[tuple]                   # (request_id, position in the request) of each row
    tokens: Optional[torch.Tensor] = None   # int32 [n_wanted]: sampled ids, when sampling was asked for


@dataclasses.dataclass
class _DecodeGraph:
    graph: "torch.cuda.CUDAGraph"
    static_input: torch.Tensor
    logits: torch.Tensor
    kernels: int                        # kernels of this package inside one replay
    tokens: Optional[torch.Tensor] = None


#: Batch sizes that decode graphs are captured for.  A step of single tokens is padded up to the next of
#: these with copies of its first entry (same token, position, cache slot and block-table row: the copy
#: computes and stores exactly what the original does, and its logits are dropped), so that a batch that
#: shrinks by one request replays a graph it already has instead of capturing a new one.
GRAPH_BATCH_SIZES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)


def graph_batch_size(n: int) -> int:
    for b in GRAPH_BATCH_SIZES:
        if b >= n:
            return b
    return n


_DEVICE_ERRORS = {1: "token id {1} at token {0} of the step is outside the vocabulary of {2}",
                  2: "token {0} of the step was given cache slot {1}, outside the pool of {2} slots",
                  3: "token {0} of the step needs key {1}, whose block-table entry is {2}",
                  4: "a kernel gave up waiting (stage {0}, {1}, {2})"}


class ModelRunner:
    def __init__(self, model: CausalLM, cache: CacheManager, max_model_len: Optional[int] = None,
                 use_cuda_graphs: bool = False, max_graph_batch: int = 256, max_graphs: int = 48):
        self.model = model
        # A captured step is run once before its capture and replayed with padding rows that repeat a
        # request; both would advance a mixer's per-request state twice.  Models with such state run
        # their decode steps as plain launches.
        self.use_cuda_graphs = use_cuda_graphs and not cache.states.specs
        self.max_graph_batch = max_graph_batch
        self.max_graphs = max_graphs        # graphs kept; the one replayed longest ago goes first
        self._graphs: "collections.OrderedDict[tuple, _DecodeGraph]" = collections.OrderedDict()
        self._graph_pool = None
        self._pad_indices: Dict[tuple, torch.Tensor] = {}
        self.cache = cache
        self.device = model.device
        self.max_model_len = max_model_len or model.spec.max_position
        self.error_flag = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._layer_caches = cache.layer_caches()
        from ..kernels import ops as _ops
        _ops.set_error_word(self.error_flag)
        self._pinned: Optional[torch.Tensor] = None
        self._copy_done: Optional[torch.cuda.Event] = None
        self.steps = 0
        self.tokens = 0
        self.h2d_bytes = 0                  # bytes of step inputs copied from pinned host memory
        self.graph_kernel_launches = 0      # kernels of this package replayed inside CUDA graphs

    # ------------------------------------------------------------------ host buffers
    def _staging(self, n: int) -> torch.Tensor:
        if self._pinned is None or self._pinned.numel() < n:
            self._pinned = torch.empty(max(n, 1 << 14), dtype=torch.int32, pin_memory=True)
        return self._pinned

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], pages_taken: bool = False,
             sampling: Optional[tuple] = None, device_tokens: Optional[torch.Tensor] = None) -> StepResult:
        """``pages_taken``: the caller (the scheduler) has already taken the pages these tokens need.
        ``sampling``: (temperatures, uniform numbers), one of each per wanted row in order; the step then
        also samples on the device (inside the captured graph for decode steps) and returns the ids.
        ``device_tokens``: int32 ids on the device, one per entry, that replace the entries' (single) tokens;
        a decode step can then be enqueued before the host has seen the ids the previous step sampled."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return StepResult(torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device), [])
        cache = self.cache
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if not cache.has_request(e.request_id):
                raise PhotonError(ErrorCode.INVALID_STATE, f"request {e.request_id!r} is not registered with the cache")
            if cache.length(e.request_id) + len(e.tokens) > self.max_model_len:
                raise PhotonError(ErrorCode.INVALID_ARGUMENT,
                                  f"request {e.request_id!r} would exceed the longest request of {self.max_model_len} tokens")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise PhotonError(ErrorCode.INVALID_INDEX, f"wanted place {w} is outside the {len(e.tokens)} tokens given")
        # pages first: all or nothing over the whole step
        need = [0] * len(cache.groups)
        if pages_taken:
            entries_to_extend = []
        else:
            entries_to_extend = entries
        for e in entries_to_extend:
            for g, n in enumerate(cache.pages_needed(e.request_id, len(e.tokens))):
                need[g] += n
        for g, n in enumerate(need):
            if n > cache.groups[g].pool.num_free:
                raise PhotonError(ErrorCode.OUT_OF_MEMORY,
                                  f"the step needs {n} more cache pages in group {g}, "
                                  f"{cache.groups[g].pool.num_free} of {cache.groups[g].num_pages} are free")
        for e in entries_to_extend:
            cache.extend(e.request_id, len(e.tokens))

        tokens = None
        if device_tokens is not None and not all(len(e.tokens) == 1 for e in entries):
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "device_tokens needs entries of one token each")
        if self.use_cuda_graphs and len(entries) <= self.max_graph_batch and all(len(e.tokens) == 1 for e in entries):
            logits, ctx, rows, tokens = self._graph_step(entries, sampling, device_tokens)
        else:
            ctx, logit_rows, rows = self._build_context(entries, sampling=sampling)
            if device_tokens is not None:
                ctx.token_ids.copy_(device_tokens[: ctx.num_tokens])
            logits = self.model.forward(ctx, self._layer_caches, logit_rows)
            if sampling is not None:
                tokens = self._sample(logits)
        for e in entries:
            cache.commit(e.request_id, len(e.tokens))
        self.steps += 1
        self.tokens += sum(len(e.tokens) for e in entries)
        return StepResult(logits, rows, tokens)

    def _sample(self, logits: torch.Tensor) -> torch.Tensor:
        """Samples every row of ``logits`` with the temperatures and uniform numbers of the last built step."""
        from ..kernels import ops
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        if logits.shape[0]:
            ops.sample(logits, self._temps, self._uniforms, out)
        return out

    def _build_context(self, entries: Sequence[StepEntry], widths: Optional[List[int]] = None,
                       static_input: Optional[torch.Tensor] = None, bound_context: Optional[int] = None,
                       sampling: Optional[tuple] = None):
        """Builds every index array of the step in one pinned buffer and copies it to the device once.
        ``widths``: block-table widths to use (default: what the requests need).  ``static_input``: a
        device buffer of the same layout to copy into (for a captured graph).  ``bound_context``: the
        context length that kernels may assume as an upper bound when they size their grids."""
        cache = self.cache
        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        starts = [cache.length(e.request_id) for e in entries]
        T = sum(q_lens)
        rids = [e.request_id for e in entries]
        n_want = sum(len(e.want) for e in entries)
        if widths is None:
            widths = cache.table_width(rids)
        G = len(cache.groups)
        # layout of the one staging buffer (int32 counts)
        n_samp = n_want if sampling is not None else 0
        sizes = [T, T, T, S + 1, S, S, n_want] + [T] * G + [S * w for w in widths] + [n_samp, n_samp]
        offs = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])]).astype(np.int64)
        total = int(offs[-1])
        self._last_total = total
        if self._copy_done is not None:
            self._copy_done.synchronize()
        stage = self._staging(total)
        host = stage.numpy()
        seg = lambda i: host[offs[i]: offs[i] + sizes[i]]
        tok, pos, tseq, cu, ctxl, slots, lrows = (seg(i) for i in range(7))
        rows: List[tuple] = []
        if T == S:
            # every request brings one token (a decode step): whole arrays at once
            tok[:] = [e.tokens[0] for e in entries]
            pos[:] = starts
            tseq[:] = range(S)
            cu[:] = range(S + 1)
            ctxl[:] = [p + 1 for p in starts]
            slots[:] = [cache.states.slot_of(r) for r in rids]
            w = 0
            for s, e in enumerate(entries):
                for k in e.want:
                    lrows[w] = s + k
                    rows.append((e.request_id, starts[s] + k))
                    w += 1
            for g in range(G):
                grp = cache.groups[g]
                ps = grp.page_size
                seg(7 + g)[:] = [grp.tables[r][p // ps] * ps + p % ps for r, p in zip(rids, starts)]
                cache.fill_block_table(g, rids, seg(7 + G + g).reshape(S, widths[g]))
        else:
            t = 0
            w = 0
            for s, e in enumerate(entries):
                n = q_lens[s]
                tok[t:t + n] = np.asarray(e.tokens, dtype=np.int64)
                pos[t:t + n] = np.arange(starts[s], starts[s] + n)
                tseq[t:t + n] = s
                cu[s] = t
                ctxl[s] = starts[s] + n
                slots[s] = cache.states.slot_of(e.request_id)
                for k in e.want:
                    lrows[w] = t + k
                    rows.append((e.request_id, starts[s] + k))
                    w += 1
                t += n
            cu[S] = T
            for g in range(G):
                sm = seg(7 + g)
                t = 0
                for s, e in enumerate(entries):
                    cache.fill_slot_mapping(g, e.request_id, starts[s], q_lens[s], sm[t:t + q_lens[s]])
                    t += q_lens[s]
                cache.fill_block_table(g, rids, seg(7 + G + g).reshape(S, widths[g]))
        if sampling is not None and n_samp:
            seg(7 + 2 * G).view(np.float32)[:] = sampling[0]
            seg(8 + 2 * G).view(np.float32)[:] = sampling[1]
        if static_input is not None:
            dev = static_input
            dev[:total].copy_(stage[:total], non_blocking=True)
        else:
            dev = stage[:total].to(self.device, non_blocking=True)
        self.h2d_bytes += 4 * total
        dseg = lambda i: dev[offs[i]: offs[i] + sizes[i]]
        groups = [GroupView(block_table=dseg(7 + G + g).view(S, widths[g]), slot_mapping=dseg(7 + g),
                            page_size=cache.groups[g].page_size, num_pages=cache.groups[g].num_pages,
                            max_pages_per_seq=widths[g]) for g in range(G)]
        ctx = StepContext(
            num_tokens=T, num_seqs=S, dtype=self.model.dtype,
            token_ids=dseg(0), positions=dseg(1), token_seq=dseg(2), cu_tokens=dseg(3),
            context_lens=dseg(4), state_slots=dseg(5), groups=groups,
            host_query_lens=q_lens, host_context_lens=[a + b for a, b in zip(starts, q_lens)],
            host_start_positions=starts, max_query_len=max(q_lens),
            max_context_len=bound_context or max(a + b for a, b in zip(starts, q_lens)), error_flag=self.error_flag)
        if sampling is not None:
            self._temps = dseg(7 + 2 * G).view(torch.float32)
            self._uniforms = dseg(8 + 2 * G).view(torch.float32)
        # the staging buffer is reused by the next step, which waits for this copy first
        self._copy_done = torch.cuda.Event()
        self._copy_done.record()
        return ctx, dseg(6), rows

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    def _graph_step(self, entries: Sequence[StepEntry], sampling: Optional[tuple] = None,
                    device_tokens: Optional[torch.Tensor] = None):
        """A step of single tokens replays a captured graph: same kernels, one launch.  A graph is
        captured per (padded batch size, block-table width, wanted rows); the width is a power of two
        of pages, so a graph serves until a request outgrows it, and the batch is padded to one of
        ``GRAPH_BATCH_SIZES`` with copies of its first entry.  The logits it returns live in the graph's
        memory and are overwritten by the next step of the same shape."""
        cache = self.cache
        real = len(entries)
        n_want = sum(len(e.want) for e in entries)
        pad = graph_batch_size(real) - real
        if pad:
            entries = list(entries) + [entries[0]] * pad
            if sampling is not None:
                extra = pad * len(entries[0].want)
                sampling = (list(sampling[0]) + [0.0] * extra, list(sampling[1]) + [0.0] * extra)
        rids = [e.request_id for e in entries]
        widths = []
        for w in cache.table_width(rids):
            b = 8
            while b < w:
                b *= 2
            widths.append(b)
        key = (len(entries), tuple(widths), sum(len(e.want) for e in entries), sampling is not None)
        bound = max(w * g.page_size for w, g in zip(widths, cache.groups)) if widths else 1
        graph = self._graphs.get(key)
        if graph is None:
            graph = self._capture(entries, widths, bound, sampling)
            self._graphs[key] = graph
            while len(self._graphs) > self.max_graphs:
                self._graphs.popitem(last=False)
        else:
            self._graphs.move_to_end(key)
        ctx, _, rows = self._build_context(entries, widths, graph.static_input, bound, sampling)
        if device_tokens is not None:
            # into a view of the graph's input buffer; padding rows repeat the first request's id
            if pad:
                torch.index_select(device_tokens, 0, self._pad_index(real, pad), out=ctx.token_ids)
            else:
                ctx.token_ids.copy_(device_tokens[:real])
        graph.graph.replay()
        self.graph_kernel_launches += graph.kernels
        tokens = graph.tokens[:n_want] if graph.tokens is not None else None
        return graph.logits[:n_want], ctx, rows[:n_want], tokens

    def _pad_index(self, real: int, pad: int) -> torch.Tensor:
        key = (real, pad)
        idx = self._pad_indices.get(key)
        if idx is None:
            idx = self._pad_indices[key] = torch.tensor(list(range(real)) + [0] * pad, dtype=torch.int64,
                                                        device=self.device)
        return idx

    def _capture(self, entries: Sequence[StepEntry], widths: List[int], bound: int,
                 sampling: Optional[tuple] = None) -> "_DecodeGraph":
        from ..kernels import ops
        # the layout depends only on (batch, widths, wanted rows): one build gives the buffer's size
        self._build_context(entries, widths, None, bound, sampling)
        size = self._last_total
        static_input = torch.zeros(size, dtype=torch.int32, device=self.device)
        ctx, logit_rows, _ = self._build_context(entries, widths, static_input, bound, sampling)
        # once outside the capture: modules load, cuBLAS makes its workspace
        warm = self.model.forward(ctx, self._layer_caches, logit_rows)
        if sampling is not None:
            self._sample(warm)
        torch.cuda.synchronize()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        g = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(g, pool=self._graph_pool):
            logits = self.model.forward(ctx, self._layer_caches, logit_rows)
            tokens = self._sample(logits) if sampling is not None else None
        kernels = ops.launch_count() - before
        return _DecodeGraph(g, static_input, logits, kernels, tokens)

    # ------------------------------------------------------------------ errors from the device
    def check_device_errors(self) -> None:
        """Reads the error word the kernels write (a device-to-host copy and a wait)."""
        self.raise_device_error(self.error_flag.cpu().tolist())

    def raise_device_error(self, flag: Sequence[int]) -> None:
        """``flag``: a host copy of the error word.  Non-zero: clears the word and the tickets that a
        kernel which gave up may have left behind, and raises."""
        if flag[0] == 0:
            return
        from ..kernels import ops
        self.error_flag.zero_()
        ops.reset_tickets(self.device)
        msg = _DEVICE_ERRORS.get(flag[0], "device error code {0}").format(flag[1], flag[2], flag[3])
        code = ErrorCode.CUDA_ERROR if flag[0] == 4 else ErrorCode.INVALID_INDEX
        raise PhotonError(code, msg)
