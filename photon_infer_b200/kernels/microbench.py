"""Times single kernels of this package at chosen sizes, with CUDA events.

    python -m photon_infer_b200.kernels.microbench products [--rows 2048 4096]
    python -m photon_infer_b200.kernels.microbench decode-products [--rows 1 8 16]
    python -m photon_infer_b200.kernels.microbench attention-prefill [--tokens 2048 8192]
    python -m photon_infer_b200.kernels.microbench attention-decode [--batch 1 8 64] [--context 640 4096]

The shapes are those of the Llama 3.2 1B layer unless ``--hidden/--intermediate/--heads/--kv-heads/
--head-dim`` say otherwise.  Decode kernels are timed inside a CUDA graph of ten launches over ten
different weight (or cache) buffers, with a buffer larger than L2 written before every timed replay, so
that neither host gaps nor a warm L2 flatter them; the library product (cuBLAS through ``torch.mm``) is
timed the same way beside ours.
"""
from __future__ import annotations

import argparse
import math

import torch

from . import ops


def _events(fn, reps: int = 20, warm: int = 3) -> float:
    """Mean microseconds of ``fn()`` over ``reps`` back-to-back calls."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def _graph(fn, copies: int, reps: int = 10) -> float:
    """Mean microseconds of one ``fn(i)`` when ``copies`` of them replay as one CUDA graph."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(copies):
            fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(copies):
            fn(i)
    g.replay()
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    times = []
    for _ in range(reps):
        _flush.zero_()                                   # 256 MB: what the last replay left in L2 is gone
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / copies)
    times.sort()
    return times[len(times) // 2]


_flush = None


def _shapes(a):
    qkv = (a.heads + 2 * a.kv_heads) * a.head_dim
    return {"qkv": (qkv, a.hidden), "o": (a.hidden, a.heads * a.head_dim),
            "gate_up": (2 * a.intermediate, a.hidden), "down": (a.hidden, a.intermediate)}


def products(a) -> None:
    """The four products of a layer at many rows: one SM per tile, pairs of SMs, the library."""
    dev = torch.device("cuda", 0)
    for M in a.rows or [2048, 4096]:
        for name, (N, K) in _shapes(a).items():
            x = torch.randn(M, K, device=dev).bfloat16()
            w = (torch.randn(N, K, device=dev) / math.sqrt(K)).bfloat16()
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            fl = 2.0 * M * N * K
            t_lib = _events(lambda: torch.mm(x, w.t(), out=out))
            t_one = _events(lambda: ops.gemm_tc(x, w, out, "bf16"))
            t_two = _events(lambda: ops.gemm_tc(x, w, out, "bf16", None, True))
            line = (f"rows {M:5d} {name:8s} library {t_lib:7.1f} us ({fl / t_lib / 1e6:5.0f} TFLOP/s)  "
                    f"one SM {t_one:7.1f} us ({fl / t_one / 1e6:5.0f})  pairs {t_two:7.1f} us ({fl / t_two / 1e6:5.0f})")
            if name == "gate_up":
                act = torch.empty(M, N // 2, device=dev, dtype=torch.bfloat16)
                t_f = _events(lambda: ops.gemm_tc(x, w, act, "swiglu", None, True))
                t_l = _events(lambda: (torch.mm(x, w.t(), out=out), ops.swiglu(out, act)))
                line += f"  with SwiGLU: pairs {t_f:7.1f} us, library + kernel {t_l:7.1f} us"
            print(line, flush=True)


def decode_products(a) -> None:
    """The weight-streaming product for few rows against the library, weights never twice from L2."""
    dev = torch.device("cuda", 0)
    for name, (N, K) in _shapes(a).items():
        ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(10)]
        for M in a.rows or [1, 8, 16]:
            x = torch.randn(M, K, device=dev).bfloat16()
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            t_lib = _graph(lambda i: torch.mm(x, ws[i].t(), out=out), 10)
            t_own = _graph(lambda i: ops.skinny_gemm(x, ws[i], out, "bf16"), 10)
            mb = N * K * 2 / 1e6
            print(f"{name:8s} rows {M:3d}  library {t_lib:6.1f} us ({mb / t_lib:5.2f} TB/s)   "
                  f"weight streaming {t_own:6.1f} us ({mb / t_own:5.2f} TB/s)", flush=True)


def _paged(batch: int, context: int, a, dev):
    ps = a.page_size
    pages_per = -(-context // ps)
    kc = torch.randn(batch * pages_per + 4, a.kv_heads, ps, a.head_dim, device=dev).bfloat16()
    vc = torch.randn_like(kc)
    table = torch.randperm(batch * pages_per).to(torch.int32).reshape(batch, pages_per).to(dev)
    return kc, vc, table


def attention_prefill(a) -> None:
    """One causal prompt portion from position 0: the tcgen05 kernel against the mma.sync kernel."""
    dev = torch.device("cuda", 0)
    n_q, n_kv, d = a.heads, a.kv_heads, a.head_dim
    for T in a.tokens or [2048, 8192]:
        kc, vc, table = _paged(1, T, a, dev)
        q = torch.randn(T, n_q * d, device=dev).bfloat16()
        out = torch.empty_like(q)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        err = torch.zeros(4, dtype=torch.int32, device=dev)
        sc = 1.0 / math.sqrt(d)
        fl = 4.0 * n_q * d * T * (T + 1) / 2
        t_old = _events(lambda: ops.flash_attention(q, out, kc, vc, table, cu, pos, 1, T, n_q, n_kv, d, None, sc, 1,
                                                    None, True, False, err))
        line = f"tokens {T:6d}  mma.sync {t_old:8.1f} us ({fl / t_old / 1e6:4.0f} TFLOP/s)"
        if ops.attention_tc_supported(q.dtype, d, n_q // n_kv, a.page_size):
            t_new = _events(lambda: ops.attention_tc(q, out, kc, vc, table, cu, pos, 1, T, n_q, n_kv, d, None, sc, err))
            line += f"   tcgen05 {t_new:8.1f} us ({fl / t_new / 1e6:4.0f} TFLOP/s)"
        print(line, flush=True)


def attention_decode(a) -> None:
    """One token per request over a paged context, with the shares the engine would choose."""
    from ..parts.attention import choose_key_shares
    dev = torch.device("cuda", 0)
    n_q, n_kv, d = a.heads, a.kv_heads, a.head_dim
    max_groups = ops.flash_attention_max_groups(d)
    for B in a.batch or [1, 8, 64]:
        for ctx in a.context or [640, 4096]:
            caches = [_paged(B, ctx, a, dev) for _ in range(10 if B * ctx <= 65536 else 3)]
            q = torch.randn(B, n_q * d, device=dev).bfloat16()
            out = torch.empty_like(q)
            cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
            pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
            lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
            err = torch.zeros(4, dtype=torch.int32, device=dev)
            splits, groups = choose_key_shares(B * n_kv, ctx, max_groups, sms=ops.sm_count(dev))
            scratch = torch.empty(B * n_q * splits * (d + 2), device=dev)

            def one(i):
                kc, vc, table = caches[i % len(caches)]
                ops.flash_attention(q, out, kc, vc, table, cu, pos, B, 1, n_q, n_kv, d, None, 1.0 / math.sqrt(d),
                                    splits, scratch, False, True, err, lens, groups)
            t = _graph(one, 10)
            mb = B * ctx * n_kv * d * 2 * 2 / 1e6
            line = (f"batch {B:3d} context {ctx:6d}  {mb:7.1f} MB of keys and values: split-key kernel ({splits} blocks per pair, "
                    f"{groups} groups) {t:7.2f} us ({mb / t:5.2f} TB/s)")
            plan = None
            if ops.attention_decode_supported(q.dtype, d, n_q // n_kv, a.page_size, B):
                plan = ops.attention_decode_plan(B, n_kv, ctx, d, a.page_size)
            if plan is not None:
                chunk, chunks, items = plan
                scratch2 = torch.empty(chunks * n_kv * 16 * (d + 2), device=dev)

                def two(i):
                    kc, vc, table = caches[i % len(caches)]
                    ops.attention_decode(q, out, kc, vc, table, cu, lens, B, n_q, n_kv, d, None, 1.0 / math.sqrt(d), chunk,
                                         scratch2, chunks, items, err)
                t2 = _graph(two, 10)
                line += f"   persistent TMA kernel (chunks of {chunk} tiles) {t2:7.2f} us ({mb / t2:5.2f} TB/s)"
            print(line, flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["products", "decode-products", "attention-prefill", "attention-decode"])
    ap.add_argument("--rows", type=int, nargs="*")
    ap.add_argument("--tokens", type=int, nargs="*")
    ap.add_argument("--batch", type=int, nargs="*")
    ap.add_argument("--context", type=int, nargs="*")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--intermediate", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=16)
    a = ap.parse_args(argv)
    torch.manual_seed(0)
    {"products": products, "decode-products": decode_products, "attention-prefill": attention_prefill,
     "attention-decode": attention_decode}[a.what](a)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
