"""Each CUDA kernel alone against a plain float32/float64 reference of the same op, at
sizes other than the engine's tests use."""
import math

import pytest
import torch

from plain.llama_plain import (causal_attention, inverse_cdf_sample, rms_norm, rope_apply,
                               rope_inverse_frequencies, swiglu, temperature_probabilities)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    # float32: summation order only.  bfloat16: one rounding of the output (2^-9 relative) plus
    # the same on inputs that the reference reads after rounding, so nothing else.
    return 2e-6 if dtype == torch.float32 else 6e-3


def _close(got, want, dtype, scale=None):
    want = want.double().cpu()
    got = got.double().cpu()
    s = float(want.abs().max()) if scale is None else scale
    assert float((got - want).abs().max()) <= _tol(dtype) * max(s, 1e-30), \
        f"max diff {float((got - want).abs().max()):.3g} at scale {s:.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,V", [(1, 24, 7), (13, 200, 101), (5, 2050, 33)])
def test_embedding(dtype, T, H, V):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(0)
    table = torch.randn(V, H).to(dtype).to(DEV)
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    out = torch.empty(T, H, dtype=torch.float32, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.embedding(ids, table, out, err)
    assert torch.equal(out.cpu(), table.float().cpu()[ids.cpu().long()])
    assert err.cpu().tolist()[0] == 0


def test_embedding_reports_bad_token():
    from photon_infer_b200.kernels import ops
    table = torch.randn(10, 8, device=DEV)
    ids = torch.tensor([1, 12, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(3, 8, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.embedding(ids, table, out, err)
    assert err.cpu().tolist() == [1, 1, 12, 10]
    assert float(out[1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H", [(1, 16), (7, 200), (3, 2048), (2, 5000), (2, 14000), (300, 2048), (70, 200), (65, 4100)])
@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(dtype, T, H, w_dtype):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(1)
    res = torch.randn(T, H)
    delta = torch.randn(T, H).to(dtype)
    w = (1 + 0.1 * torch.randn(H)).to(w_dtype)
    eps = 3e-6
    want_res = res + delta.float()
    want = rms_norm(want_res.double(), w.double(), eps)
    r = res.to(DEV).clone()
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(delta.to(DEV), r, w.to(DEV), eps, out)
    assert torch.equal(r.cpu(), want_res)
    _close(out, want, dtype)
    # without a delta, and on listed rows only
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, dtype=dtype, device=DEV)
    r2 = res.to(DEV).clone()
    ops.add_rmsnorm(delta.to(DEV), r2, w.to(DEV), eps, out2, rows=rows)
    assert torch.equal(r2.cpu(), res)                       # listed rows are only read
    _close(out2, want[[T - 1, 0]], dtype)
    out3 = torch.empty(T, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(None, r2, w.to(DEV), eps, out3)
    _close(out3, rms_norm(res.double(), w.double(), eps), dtype)
    if T >= 64:
        # many listed rows: every row twice, backwards
        many = torch.arange(T - 1, -1, -1, dtype=torch.int32, device=DEV).repeat(2)
        out4 = torch.empty(2 * T, H, dtype=dtype, device=DEV)
        ops.add_rmsnorm(delta.to(DEV), r2, w.to(DEV), eps, out4, rows=many)
        assert torch.equal(r2.cpu(), res)
        _close(out4, want[many.cpu().long()], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 8), (9, 200), (300, 1111)])
def test_swiglu(dtype, T, I):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(2)
    gu = (3 * torch.randn(T, 2 * I)).to(dtype)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    ops.swiglu(gu.to(DEV), out)
    _close(out, swiglu(gu[:, :I].double(), gu[:, I:].double()), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("n_q,n_kv,d,ps", [(4, 2, 16, 16), (3, 1, 32, 8), (6, 2, 48, 16), (2, 2, 128, 4), (5, 5, 80, 32)])
def test_rope_and_cache_write(dtype, interleaved, n_q, n_kv, d, ps):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(3)
    T, pages = 11, 9
    qkv = torch.randn(T, (n_q + 2 * n_kv) * d).to(dtype)
    positions = torch.tensor([0, 1, 2, 3, 77, 500, 4095, 9, 10, 70000, 12], dtype=torch.int32)
    scaling = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                   original_max_position_embeddings=64)
    inv = rope_inverse_frequencies(d, 500000.0, scaling)
    slots = torch.randperm(pages * ps)[:T].to(torch.int32)
    kc = torch.zeros(pages, n_kv, ps, d, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    buf = qkv.to(DEV).clone()
    q = buf[:, : n_q * d]
    k = buf[:, n_q * d: (n_q + n_kv) * d]
    v = buf[:, (n_q + n_kv) * d:]
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.rope_kv_write(q, k, v, positions.to(DEV), inv.to(DEV), interleaved, slots.to(DEV), kc, vc, n_q, n_kv, d, err)
    assert err.cpu().tolist()[0] == 0
    src = qkv.double()
    want_q = rope_apply(src[:, : n_q * d].view(T, n_q, d), positions, inv, interleaved)
    want_k = rope_apply(src[:, n_q * d: (n_q + n_kv) * d].view(T, n_kv, d), positions, inv, interleaved)
    # the angle is a float32 product of a large position: allow its rounding (|x| * 2^-24 * pos ~ 1e-3 at 70000)
    big = 4e-3 if dtype == torch.float32 else None
    if dtype == torch.float32:
        small = positions < 5000
        _close(q.view(T, n_q, d)[small], want_q[small], dtype, scale=float(want_q.abs().max()) * 20)
        assert float((q.view(T, n_q, d).cpu().double() - want_q).abs().max()) < big * float(want_q.abs().max())
    else:
        _close(q.view(T, n_q, d), want_q, dtype)
    got_k = torch.stack([kc.cpu()[int(s) // ps, :, int(s) % ps, :] for s in slots])
    got_v = torch.stack([vc.cpu()[int(s) // ps, :, int(s) % ps, :] for s in slots])
    assert torch.equal(got_v, qkv[:, (n_q + n_kv) * d:].view(T, n_kv, d))
    assert torch.equal(got_k, k.view(T, n_kv, d).cpu())
    if dtype == torch.bfloat16:
        _close(got_k, want_k, dtype)
    # slots that were not named stay untouched
    untouched = torch.ones(pages * ps, dtype=torch.bool)
    untouched[slots.long()] = False
    assert float(kc.cpu().permute(0, 2, 1, 3).reshape(pages * ps, -1)[untouched].abs().max()) == 0.0


def test_rope_float32_matches_plain_exactly_enough():
    """Same 32-bit angle as the plain implementation: agreement to float32 rounding at small positions."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(4)
    T, n_q, n_kv, d = 64, 2, 1, 64
    positions = torch.arange(T, dtype=torch.int32)
    inv = rope_inverse_frequencies(d, 10000.0, None)
    x = torch.randn(T, (n_q + 2 * n_kv) * d)
    buf = x.to(DEV).clone()
    ops.rope_kv_write(buf[:, : n_q * d], buf[:, n_q * d:(n_q + n_kv) * d], None, positions.to(DEV), inv.to(DEV),
                      False, None, None, None, n_q, n_kv, d, None)
    want = rope_apply(x[:, : n_q * d].view(T, n_q, d), positions, inv, False)
    assert float((buf[:, : n_q * d].view(T, n_q, d).cpu() - want).abs().max()) < 2e-6 * float(want.abs().max())


def _paged(k, v, ps, pages, seed):
    """Scatter dense [L, n_kv, d] keys/values into a paged cache with a shuffled block table."""
    L, n_kv, d = k.shape
    n_logical = (L + ps - 1) // ps
    g = torch.Generator().manual_seed(seed)
    table = torch.randperm(pages, generator=g)[:n_logical]
    kc = torch.full((pages, n_kv, ps, d), float("nan"), dtype=k.dtype)     # unwritten slots must never be read
    vc = torch.full((pages, n_kv, ps, d), float("nan"), dtype=k.dtype)
    for t in range(L):
        kc[table[t // ps], :, t % ps] = k[t]
        vc[table[t // ps], :, t % ps] = v[t]
    return kc, vc, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,ps,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 2, 48, 16, 24), (8, 1, 64, 4, None), (2, 2, 128, 32, 70),
    (5, 5, 80, 16, None), (16, 2, 256, 16, None), (7, 7, 16, 8, 5)])
def test_paged_attention_two_requests(dtype, n_q, n_kv, d, ps, window):
    """Two requests in one batch: a portion in the middle of one, a single late token of the other."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(5)
    lens = [150, 97]
    pages = sum((L + ps - 1) // ps for L in lens) + 5
    qs, ks, vs, outs = [], [], [], []
    kc = vc = None
    tables = []
    for i, L in enumerate(lens):
        q = torch.randn(L, n_q, d).to(dtype)
        k = torch.randn(L, n_kv, d).to(dtype)
        v = torch.randn(L, n_kv, d).to(dtype)
        outs.append(causal_attention(q.double(), k.double(), v.double(), window=window))
        qs.append(q); ks.append(k); vs.append(v)
    # one shared pool: request 0 takes even pages, request 1 odd ones, shuffled
    kc = torch.full((pages, n_kv, ps, d), float("nan"), dtype=dtype)
    vc = torch.full_like(kc, float("nan"))
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(9)).tolist()
    width = max((L + ps - 1) // ps for L in lens) + 3
    table = torch.full((2, width), -1, dtype=torch.int32)
    for i, L in enumerate(lens):
        for lp in range((L + ps - 1) // ps):
            table[i, lp] = perm.pop()
        for t in range(L):
            kc[table[i, t // ps], :, t % ps] = ks[i][t]
            vc[table[i, t // ps], :, t % ps] = vs[i][t]
    # request 0: tokens 60..99 ; request 1: its last token
    tok_seq = torch.tensor([0] * 40 + [1], dtype=torch.int32)
    positions = torch.tensor(list(range(60, 100)) + [lens[1] - 1], dtype=torch.int32)
    q = torch.cat([qs[0][60:100], qs[1][-1:]]).reshape(41, n_q * d)
    want = torch.cat([outs[0][60:100], outs[1][-1:]]).reshape(41, n_q * d)
    out = torch.empty(41, n_q * d, dtype=dtype, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.paged_attention(q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV), tok_seq.to(DEV), positions.to(DEV),
                        n_q, n_kv, d, window, 1.0 / math.sqrt(d), err)
    assert err.cpu().tolist()[0] == 0
    assert not torch.isnan(out).any()
    _close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_far_key_stands_out(dtype):
    """One key among hundreds is made to dominate: the output must be that key's value."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(6)
    n_q, n_kv, d, ps, L = 4, 1, 64, 16, 700
    for far in (0, 15, 16, 333, 511, 512, 699):
        q = 0.1 * torch.randn(1, n_q, d)
        k = 0.1 * torch.randn(L, n_kv, d)
        v = torch.randn(L, n_kv, d)
        k[far] = 0
        k[far, 0, 0] = 40.0
        q[0, :, 0] = 40.0                                    # score 1600/8 = 200 against O(1) elsewhere
        kc, vc, table = _paged(k.to(dtype), v.to(dtype), ps, 50, seed=far)
        out = torch.empty(1, n_q * d, dtype=dtype, device=DEV)
        ops.paged_attention(q.to(dtype).reshape(1, -1).to(DEV), out, kc.to(DEV), vc.to(DEV),
                            table.to(torch.int32).reshape(1, -1).to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                            torch.tensor([L - 1], dtype=torch.int32, device=DEV), n_q, n_kv, d, None,
                            1.0 / math.sqrt(d), None)
        want = v[far, 0].to(dtype).float().repeat(n_q)
        assert float((out.float().cpu()[0] - want).abs().max()) < 1e-3, f"far key {far}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_window_edge(dtype):
    """The key just outside the window dominates in score but must be invisible."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(7)
    n_q, n_kv, d, ps, L, window = 2, 1, 32, 8, 100, 24
    q = 0.1 * torch.randn(1, n_q, d)
    k = 0.1 * torch.randn(L, n_kv, d)
    v = torch.randn(L, n_kv, d)
    outside = L - 1 - window                                  # first invisible key
    k[outside] = 0; k[outside, 0, 0] = 50.0
    q[0, :, 0] = 50.0
    kc, vc, table = _paged(k.to(dtype), v.to(dtype), ps, 20, seed=1)
    args = (kc.to(DEV), vc.to(DEV), table.to(torch.int32).reshape(1, -1).to(DEV),
            torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([L - 1], dtype=torch.int32, device=DEV))
    out = torch.empty(1, n_q * d, dtype=dtype, device=DEV)
    ops.paged_attention(q.to(dtype).reshape(1, -1).to(DEV), out, *args, n_q, n_kv, d, window, 1.0 / math.sqrt(d), None)
    want = causal_attention(q.to(dtype).double().expand(L, n_q, d).clone(), k.to(dtype).double(), v.to(dtype).double(),
                            window=window)[-1].reshape(-1)
    _close(out[0], want, dtype)
    # with a window one larger the key is visible and takes over
    ops.paged_attention(q.to(dtype).reshape(1, -1).to(DEV), out, *args, n_q, n_kv, d, window + 1, 1.0 / math.sqrt(d), None)
    assert float((out.float().cpu()[0] - v[outside, 0].to(dtype).float().repeat(n_q)).abs().max()) < 1e-3


def test_paged_attention_reports_missing_page():
    from photon_infer_b200.kernels import ops
    n_q, n_kv, d, ps = 2, 1, 16, 8
    kc = torch.zeros(4, n_kv, ps, d, device=DEV)
    table = torch.tensor([[0, -1, 2, -1]], dtype=torch.int32, device=DEV)
    out = torch.empty(1, n_q * d, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.paged_attention(torch.zeros(1, n_q * d, device=DEV), out, kc, kc, table, torch.zeros(1, dtype=torch.int32, device=DEV),
                        torch.tensor([20], dtype=torch.int32, device=DEV), n_q, n_kv, d, None, 0.25, err)
    assert err.cpu().tolist()[0] == 3


def test_paged_attention_refuses_oversized_group():
    from photon_infer_b200.errors import PhotonError
    from photon_infer_b200.kernels import ops
    z = torch.zeros(1, 64 * 128, device=DEV)
    kc = torch.zeros(1, 1, 8, 128, device=DEV)
    i = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(PhotonError):
        ops.paged_attention(z, z.clone(), kc, kc, i.view(1, 1), i, i, 64, 1, 128, None, 1.0, None)


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (1, 300, 77), (65, 64, 16), (130, 257, 1000), (7, 389, 120)])
def test_sgemm_true_fp32(M, N, K):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(8)
    a, w = torch.randn(M, K), torch.randn(N, K)
    out = ops.linear(a.to(DEV), w.to(DEV))
    want = a.double() @ w.double().t()
    assert float((out.cpu().double() - want).abs().max()) <= 1e-6 * math.sqrt(K) * float(want.abs().max() + 1)
    # row results do not depend on the other rows of the batch
    out1 = ops.linear(a[:1].to(DEV), w.to(DEV))
    assert torch.equal(out1.cpu(), out[:1].cpu())
    # a strided input (a section of a wider row)
    wide = torch.randn(M, K + 9).to(DEV)
    out2 = ops.linear(wide[:, 4: 4 + K], w.to(DEV))
    assert torch.equal(out2.cpu(), ops.linear(wide[:, 4: 4 + K].contiguous(), w.to(DEV)).cpu())


def test_sgemm_keeps_what_tf32_would_lose():
    """Inputs with 20 significant bits: a reduced-precision matrix mode would round them to 10."""
    from photon_infer_b200.kernels import ops
    a = torch.tensor([[1.0 + 2.0 ** -18, 1.0]])
    w = torch.tensor([[1.0, -1.0]])
    assert float(ops.linear(a.to(DEV), w.to(DEV)).cpu()[0, 0]) == 2.0 ** -18


@pytest.mark.parametrize("M,N,K", [(1, 389, 120), (40, 512, 256), (3, 100, 72)])
def test_linear_bf16_with_fp32_output(M, N, K):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(9)
    a, w = torch.randn(M, K).bfloat16(), torch.randn(N, K).bfloat16()
    want = a.double() @ w.double().t()
    out = ops.linear(a.to(DEV), w.to(DEV), out_dtype=torch.float32)
    assert out.dtype == torch.float32
    assert float((out.cpu().double() - want).abs().max()) <= 1e-5 * float(want.abs().max())
    _close(ops.linear(a.to(DEV), w.to(DEV)), want, torch.bfloat16)


@pytest.mark.parametrize("V", [5, 389, 1024, 50000, 128256])
def test_sampling(V):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(10)
    rows = 6
    logits = 3 * torch.randn(rows, V)
    logits[1, V // 2] = logits[1, V - 1] = logits[1].max() + 1          # a tie: the earlier index wins
    temps = torch.tensor([0.0, 0.0, 0.8, 0.8, 1.7, 0.3])
    u = torch.tensor([0.0, 0.0, 0.0, 0.37, 0.999, 0.5])
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), temps.to(DEV), u.to(DEV), out)
    got = out.cpu().tolist()
    assert got[0] == int(torch.argmax(logits[0]))
    assert got[1] == V // 2
    for r in range(2, rows):
        p = temperature_probabilities(logits[r], float(temps[r])).double()
        cdf = torch.cumsum(p, 0)
        want = inverse_cdf_sample(p.float(), float(u[r]))
        if got[r] != want:
            # only a value of u within rounding of a step of the CDF may fall to a neighbour
            lo = float(cdf[got[r] - 1]) if got[r] > 0 else 0.0
            assert lo - 1e-5 <= float(u[r]) <= float(cdf[got[r]]) + 1e-5, (r, got[r], want)
    # greedy without temperatures
    out2 = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), None, None, out2)
    assert out2.cpu().tolist() == [int(torch.argmax(logits[r])) if r != 1 else V // 2 for r in range(rows)]


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(64, 64), (389, 120), (2048, 2048), (100, 8200), (16, 8)])
def test_skinny_gemm(M, N, K):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(13)
    x = torch.randn(M, K).bfloat16()
    w = torch.randn(N, K).bfloat16()
    want = x.double() @ w.double().t()
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.skinny_gemm(x.to(DEV), w.to(DEV), out32, "f32")
    assert float((out32.cpu().double() - want).abs().max()) <= 2e-6 * math.sqrt(K) * float(want.abs().max())
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.skinny_gemm(x.to(DEV), w.to(DEV), out, "bf16")
    _close(out, want, torch.bfloat16)
    # a strided x (a section of wider rows)
    wide = torch.randn(M, K + 16).bfloat16().to(DEV)
    out2 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.skinny_gemm(wide[:, 8: 8 + K], w.to(DEV), out2, "f32")
    ref = wide[:, 8: 8 + K].cpu().double() @ w.double().t()
    assert float((out2.cpu().double() - ref).abs().max()) <= 2e-6 * math.sqrt(K) * float(ref.abs().max())


@pytest.mark.parametrize("M", [1, 8, 13, 32])
@pytest.mark.parametrize("I,K", [(48, 64), (200, 96), (8192, 2048), (10, 16)])
def test_skinny_gemm_swiglu(M, I, K):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(14)
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(2 * I, K) / math.sqrt(K)).bfloat16()
    gu = x.double() @ w.double().t()
    want = swiglu(gu[:, :I], gu[:, I:])
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    ops.skinny_gemm(x.to(DEV), w.to(DEV), out, "swiglu")
    _close(out, want, torch.bfloat16)


def test_skinny_gemm_refuses_what_it_cannot_load():
    from photon_infer_b200.errors import PhotonError
    from photon_infer_b200.kernels import ops
    x = torch.randn(4, 20).bfloat16().to(DEV)              # K not a multiple of 8
    w = torch.randn(8, 20).bfloat16().to(DEV)
    assert not ops.skinny_gemm_supported(x, w)
    with pytest.raises(PhotonError):
        ops.skinny_gemm(x, w, torch.empty(4, 8, dtype=torch.bfloat16, device=DEV))
    # the general entry point takes the library path instead and is still right
    got = ops.linear(x, w)
    _close(got, x.cpu().double() @ w.cpu().double().t(), torch.bfloat16)


def _flash_case(n_q, n_kv, d, ps, window, lens, steps, splits, seed=21):
    """Requests of `lens` tokens; `steps[i]` = (first, count) tokens of request i in this step."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(seed)
    dtype = torch.bfloat16
    pages = sum((L + ps - 1) // ps for L in lens) + 3
    kc = torch.full((pages, n_kv, ps, d), float("nan"), dtype=dtype)
    vc = torch.full_like(kc, float("nan"))
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max((L + ps - 1) // ps for L in lens) + 1
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    qs, want, positions, cu = [], [], [], [0]
    for i, L in enumerate(lens):
        q = torch.randn(L, n_q, d).to(dtype)
        k = torch.randn(L, n_kv, d).to(dtype)
        v = torch.randn(L, n_kv, d).to(dtype)
        for lp in range((L + ps - 1) // ps):
            table[i, lp] = perm.pop()
        first, count = steps[i]
        for t in range(first + count):                      # the cache holds what the step can see, nothing later
            kc[table[i, t // ps], :, t % ps] = k[t]
            vc[table[i, t // ps], :, t % ps] = v[t]
        o = causal_attention(q.double(), k.double(), v.double(), window=window)
        qs.append(q[first:first + count]); want.append(o[first:first + count])
        positions += list(range(first, first + count))
        cu.append(cu[-1] + count)
    T = cu[-1]
    q = torch.cat(qs).reshape(T, n_q * d)
    out = torch.full((T, n_q * d), float("nan"), dtype=dtype, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    G = n_q // n_kv
    few = [c * G <= 16 for _, c in steps]
    scratch = torch.full((T * n_q * splits * (d + 2),), float("nan"), device=DEV)
    args = (q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV), torch.tensor(cu, dtype=torch.int32, device=DEV),
            torch.tensor(positions, dtype=torch.int32, device=DEV), len(lens), max(c for _, c in steps),
            n_q, n_kv, d, window, 1.0 / math.sqrt(d), splits, scratch, not all(few), any(few), err)
    ops.flash_attention(*args)
    assert err.cpu().tolist()[0] == 0
    assert not torch.isnan(out.float()).any()
    _close(out, torch.cat(want).reshape(T, n_q * d), dtype)
    # the same with the requests' lengths given: the split-key kernel then does not read the positions
    first = out.clone()
    out.fill_(float("nan"))
    lens_after = torch.tensor([f + c for f, c in steps], dtype=torch.int32, device=DEV)
    ops.flash_attention(*args, lens_after)
    assert err.cpu().tolist()[0] == 0
    assert torch.equal(out, first)
    # and with the keys of a block dealt to groups of warps
    for groups in (2, 4):
        if groups <= ops.flash_attention_max_groups(d):
            out.fill_(float("nan"))
            ops.flash_attention(*args, lens_after, groups)
            assert err.cpu().tolist()[0] == 0
            assert not torch.isnan(out.float()).any()
            _close(out, torch.cat(want).reshape(T, n_q * d), dtype)


@pytest.mark.parametrize("n_q,n_kv,d,ps,window", [
    (4, 1, 64, 16, None), (32, 8, 64, 16, None), (3, 1, 32, 8, None), (6, 2, 48, 16, 24), (8, 1, 128, 16, None),
    (2, 2, 16, 4, 5), (5, 5, 80, 32, None), (6, 2, 64, 16, 70)])
def test_flash_attention_portions_and_single_tokens(n_q, n_kv, d, ps, window):
    """One launch pair: a long portion from the start, a portion in the middle of a request, a single late
    token, the first token of a request, and a two-token portion."""
    lens = [200, 333, 700, 1, 90]
    steps = [(0, 200), (150, 183), (699, 1), (0, 1), (88, 2)]
    for splits in (1, 3):
        _flash_case(n_q, n_kv, d, ps, window, lens, steps, splits)


def test_flash_attention_decode_batch_with_splits():
    lens = [640, 1, 65, 333, 700, 64, 63, 129]
    steps = [(L - 1, 1) for L in lens]
    for splits in (1, 2, 5, 11):
        _flash_case(32, 8, 64, 16, None, lens, steps, splits)
        _flash_case(8, 2, 128, 8, None, lens, steps, splits)


def test_flash_attention_far_key_and_window_edge():
    from photon_infer_b200.kernels import ops
    torch.manual_seed(22)
    n_q, n_kv, d, ps, L = 4, 1, 64, 16, 700
    for far, window, count in ((0, None, 1), (63, None, 1), (64, None, 1), (640, None, 1), (699, None, 1),
                               (699 - 24, 24, 1), (699 - 23, 24, 1), (0, None, 40), (333, None, 40)):
        q = 0.1 * torch.randn(count, n_q, d)
        k = 0.1 * torch.randn(L, n_kv, d)
        v = torch.randn(L, n_kv, d)
        k[far] = 0
        k[far, 0, 0] = 40.0
        q[:, :, 0] = 40.0
        kc, vc, table = _paged(k.bfloat16(), v.bfloat16(), ps, 50, seed=far)
        out = torch.empty(count, n_q * d, dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(count * n_q * 4 * (d + 2), device=DEV)
        G = n_q // n_kv
        ops.flash_attention(q.bfloat16().reshape(count, -1).to(DEV), out, kc.to(DEV), vc.to(DEV),
                            table.to(torch.int32).reshape(1, -1).to(DEV), torch.tensor([0, count], dtype=torch.int32, device=DEV),
                            torch.arange(L - count, L, dtype=torch.int32, device=DEV), 1, count, n_q, n_kv, d, window,
                            1.0 / math.sqrt(d), 4, scratch, count * G > 16, count * G <= 16, None)
        hit = float((out.float().cpu()[-1] - v[far, 0].bfloat16().float().repeat(n_q)).abs().max()) < 1e-3
        visible = window is None or far > L - 1 - window
        assert hit == visible, (far, window, count)


def _decode_attention_case(n_q, n_kv, d, ps, window, lens, counts, chunk, seed=41, spike=None):
    """Requests of `lens` tokens whose last `counts[i]` tokens are this step's; the persistent TMA kernel with work
    items of `chunk` tiles, against float64.  Cache slots the step must not see hold NaN."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(seed)
    dtype = torch.bfloat16
    pages = sum((L + ps - 1) // ps for L in lens) + 3
    kc = torch.full((pages, n_kv, ps, d), float("nan"), dtype=dtype)
    vc = torch.full_like(kc, float("nan"))
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max((L + ps - 1) // ps for L in lens) + 1
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    qs, want, cu = [], [], [0]
    for i, (L, count) in enumerate(zip(lens, counts)):
        q = torch.randn(L, n_q, d)
        k = torch.randn(L, n_kv, d)
        v = torch.randn(L, n_kv, d)
        if spike is not None and i == 0:
            k *= 0.1; q *= 0.1
            k[spike] = 0; k[spike, :, 0] = 40.0; q[:, :, 0] = 40.0
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        for lp in range((L + ps - 1) // ps):
            table[i, lp] = perm.pop()
        for t in range(L):
            kc[table[i, t // ps], :, t % ps] = k[t]
            vc[table[i, t // ps], :, t % ps] = v[t]
        o = causal_attention(q.double(), k.double(), v.double(), window=window)
        qs.append(q[L - count:]); want.append(o[L - count:])
        cu.append(cu[-1] + count)
    T = cu[-1]
    q = torch.cat(qs).reshape(T, n_q * d)
    out = torch.full((T, n_q * d), float("nan"), dtype=dtype, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    keys = max(lens) if window is None else min(window + max(counts), max(lens))
    chunks = len(lens) * (-(-(keys // 64 + 2) // chunk))
    scratch = torch.full((chunks * n_kv * 16 * (d + 2),), float("nan"), device=DEV)
    for _ in range(2):                                      # twice: the tickets and counters must be back at zero
        out.fill_(float("nan"))
        ops.attention_decode(q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV),
                             torch.tensor(cu, dtype=torch.int32, device=DEV),
                             torch.tensor(lens, dtype=torch.int32, device=DEV), len(lens), n_q, n_kv, d, window,
                             1.0 / math.sqrt(d), chunk, scratch, chunks, chunks * n_kv, err)
        assert err.cpu().tolist()[0] == 0
        assert not torch.isnan(out.float()).any()
        _close(out, torch.cat(want).reshape(T, n_q * d), dtype)
    return out.float().cpu(), torch.cat(want).reshape(T, n_q * d)


@pytest.mark.parametrize("n_q,n_kv,d,ps,window", [
    (32, 8, 64, 16, None), (24, 8, 128, 16, None), (3, 1, 64, 8, None), (8, 1, 128, 32, None), (6, 2, 64, 64, None),
    (16, 1, 64, 16, None), (6, 2, 64, 16, 70), (4, 2, 128, 128, 200)])
def test_decode_attention_tma(n_q, n_kv, d, ps, window):
    """Single tokens of requests of very different lengths (one key, a page's edge, a tile's edge, thousands of
    keys), and short portions of up to 16 rows, with items of 1, 4 and 64 tiles: one chunk, many chunks merged."""
    lens = [640, 1, 65, 333, 2100, 64, 63, 129, 1024]
    G = n_q // n_kv
    for chunk in (1, 4, 64):
        _decode_attention_case(n_q, n_kv, d, ps, window, lens, [1] * len(lens), chunk)
    if 16 // G >= 2:
        counts = [min(L, 16 // G) if i % 2 else 1 for i, L in enumerate(lens)]
        _decode_attention_case(n_q, n_kv, d, ps, window, lens, counts, 4)


def test_decode_attention_tma_far_key_and_more_requests_than_blocks():
    """A key far back must carry the result (chunks merged with their true weights), and a step with more work
    items than the GPU has blocks must hand every one of them out."""
    for far in (0, 63, 64, 1000, 2099):
        got, want = _decode_attention_case(4, 1, 64, 16, None, [2100, 300], [1, 1], 4, spike=far)
        assert float((got[0] - want[0].float()).abs().max()) < 2e-2
    lens = [70 + 13 * i for i in range(200)]
    _decode_attention_case(8, 4, 64, 16, None, lens, [1] * len(lens), 1)


@pytest.mark.parametrize("n_q,n_kv,d", [(32, 8, 64), (24, 8, 128)])
def test_decode_attention_tma_cuts_requests_of_one_length_itself(n_q, n_kv, d):
    """Requests of nearly one length with a chunk length from the host that suits them badly (one tile, or more
    tiles than they have): the kernel chooses its own within the room it was given, and the result is the same."""
    lens = [3000, 2900, 3100, 2950]
    for chunk in (1, 2, 64):
        _decode_attention_case(n_q, n_kv, d, 16, None, lens, [1] * len(lens), chunk)
    _decode_attention_case(n_q, n_kv, d, 16, None, [700] * 40, [1] * 40, 1)


def test_decode_attention_tma_refuses_what_it_cannot_take():
    from photon_infer_b200.errors import PhotonError
    from photon_infer_b200.kernels import ops
    assert not ops.attention_decode_supported(torch.bfloat16, 48, 3, 16, 4)
    assert not ops.attention_decode_supported(torch.float32, 64, 4, 16, 4)
    assert not ops.attention_decode_supported(torch.bfloat16, 64, 32, 16, 4)
    assert not ops.attention_decode_supported(torch.bfloat16, 64, 4, 24, 4)
    assert not ops.attention_decode_supported(torch.bfloat16, 64, 4, 16, 600)
    q = torch.zeros(1, 48, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(4, 1, 16, 48, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(PhotonError):
        ops.attention_decode(q, q.clone(), kc, kc.clone(), torch.zeros(1, 8, dtype=torch.int32, device=DEV), z, z, 1, 1, 1,
                             48, None, 1.0, 4, torch.zeros(4096, device=DEV), 1, 1, None)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1, 8, 8), (100, 300, 72), (257, 513, 520), (2048, 3072, 2048),
                                   (333, 389, 120), (4096, 256, 8192)])
def test_gemm_tcgen05(M, N, K):
    """The tensor-memory product against float64, with sizes that leave partial tiles on every side."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(15)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    want = x.double() @ w.double().t()
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tc(x, w, out32, "f32", err)
    assert err.cpu().tolist()[0] == 0
    assert float((out32.double() - want).abs().max()) <= 2e-6 * math.sqrt(K) * float(want.abs().max())
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x, w, out, "bf16", err)
    _close(out, want, torch.bfloat16)
    # a strided input (a section of wider rows), as the attention output projection gets
    wide = torch.randn(M, K + 16, device=DEV).bfloat16()
    out2 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_tc(wide[:, 8: 8 + K], w, out2, "f32", err)
    ref = wide[:, 8: 8 + K].double() @ w.double().t()
    assert float((out2.double() - ref).abs().max()) <= 2e-6 * math.sqrt(K) * float(ref.abs().max())
    assert err.cpu().tolist()[0] == 0


def test_gemm_tcgen05_wait_that_runs_out_is_reported():
    """A build of gemm_tc.cu whose producer loads nothing (``TC_TEST_NO_LOADS``) and whose waits give up after a
    few thousand polls: the consumer's bounded wait on a barrier that nothing completes runs out, the kernel
    records PHOTON_DEV_WAIT_TIMEOUT with the block's index, frees its tensor memory and returns; the stock
    build runs right afterwards in the same context."""
    import ctypes
    from ctypes import c_int, c_long, c_void_p
    from photon_infer_b200.csrc.build import load_module
    from photon_infer_b200.kernels import ops
    torch.manual_seed(16)
    M, N, K = 256, 512, 128
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    lib = load_module("gemm_tc", {"TC_TEST_NO_LOADS": 1, "TC_WAIT_LIMIT": 4096})
    f = lib.photon_gemm_tc
    f.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    f.restype = c_int
    status = f(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K, 0,
               err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert status == 0
    torch.cuda.synchronize()                                   # the kernel came back by itself
    word = err.cpu().tolist()
    assert word[0] == 4 and 0 <= word[1] < 4                   # PHOTON_DEV_WAIT_TIMEOUT, one of the four blocks
    assert float(out.float().abs().max()) == 0.0               # nothing was computed, nothing was written
    err.zero_()
    ops.gemm_tc(x, w, out, "bf16", err)                        # tensor memory and barriers are in order
    _close(out, x.double() @ w.double().t(), torch.bfloat16)
    assert err.cpu().tolist()[0] == 0


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (70, 200, 96), (2048, 8192, 2048), (300, 136, 72)])
def test_gemm_tcgen05_swiglu(M, I, K):
    from photon_infer_b200.kernels import ops
    torch.manual_seed(16)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) / math.sqrt(K)).bfloat16()
    gu = x.double() @ w.double().t()
    want = swiglu(gu[:, :I], gu[:, I:])
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.gemm_tc(x, w, out, "swiglu", err)
    assert err.cpu().tolist()[0] == 0
    _close(out, want, torch.bfloat16)


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("K,N", [(64, 48), (120, 400), (2048, 512)])
@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_delta", [True, False])
def test_skinny_fused_norm_product(M, K, N, w_dtype, with_delta):
    """Residual sum + RMSNorm + product in one kernel, plain and SwiGLU epilogues."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(17)
    res = torch.randn(M, K)
    delta = torch.randn(M, K).bfloat16() if with_delta else None
    nw = (1 + 0.1 * torch.randn(K)).to(w_dtype)
    w = (torch.randn(N, K) / math.sqrt(K)).bfloat16()
    x = res.double() + (delta.double() if with_delta else 0)
    h = rms_norm(x, nw.double(), 1e-5)
    want = h @ w.double().t()
    res_dev = res.to(DEV)
    out, new_res = ops.skinny_fused(res_dev, delta.to(DEV) if with_delta else None, nw.to(DEV), 1e-5, w.to(DEV), "bf16")
    assert torch.equal(res_dev.cpu(), res)                         # the input stream is not written
    assert torch.equal(new_res.cpu(), x.float())
    # the product sees x * w_norm rounded to bfloat16: one more rounding than the output's own
    assert float((out.double().cpu() - want).abs().max()) <= 1.2e-2 * float(want.abs().max())
    act, _ = ops.skinny_fused(res_dev, delta.to(DEV) if with_delta else None, nw.to(DEV), 1e-5, w.to(DEV), "swiglu")
    want_act = swiglu(want[:, : N // 2], want[:, N // 2:])
    assert float((act.double().cpu() - want_act).abs().max()) <= 1.5e-2 * float(want_act.abs().max())


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("n_q,n_kv,d,ps", [(4, 2, 16, 16), (3, 1, 32, 8), (32, 8, 64, 16), (6, 2, 48, 4)])
def test_skinny_fused_qkv_rotation_and_cache_write(M, n_q, n_kv, d, ps):
    """Norm, q/k/v products, rotation of neighbouring pairs and the cache write in one kernel."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(18)
    K = 96 if d < 64 else 2048
    N = (n_q + 2 * n_kv) * d
    res = torch.randn(M, K)
    delta = torch.randn(M, K).bfloat16()
    nw = (1 + 0.1 * torch.randn(K)).bfloat16()
    w = (torch.randn(N, K) / math.sqrt(K)).bfloat16()
    positions = torch.tensor([0, 5, 63, 64, 700, 4095, 1, 17][:M], dtype=torch.int32)
    inv = rope_inverse_frequencies(d, 500000.0, None)
    pages = 12
    slots = torch.randperm(pages * ps)[:M].to(torch.int32)
    kc = torch.zeros(pages, n_kv, ps, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q, new_res = ops.skinny_fused(res.to(DEV), delta.to(DEV), nw.to(DEV), 1e-5, w.to(DEV), "qkv",
                                  rope=dict(positions=positions.to(DEV), inv_freq=inv.to(DEV), slot_mapping=slots.to(DEV),
                                            k_cache=kc, v_cache=vc, n_q=n_q, n_kv=n_kv, head_dim=d))
    x = res.double() + delta.double()
    y = rms_norm(x, nw.double(), 1e-5) @ w.double().t()
    want_q = rope_apply(y[:, : n_q * d].reshape(M, n_q, d), positions, inv, True)
    want_k = rope_apply(y[:, n_q * d: (n_q + n_kv) * d].reshape(M, n_kv, d), positions, inv, True)
    want_v = y[:, (n_q + n_kv) * d:].reshape(M, n_kv, d)
    scale = float(y.abs().max())
    assert float((q.double().cpu().reshape(M, n_q, d) - want_q).abs().max()) <= 1.5e-2 * scale
    got_k = torch.stack([kc.cpu()[int(s) // ps, :, int(s) % ps, :] for s in slots]).double()
    got_v = torch.stack([vc.cpu()[int(s) // ps, :, int(s) % ps, :] for s in slots]).double()
    assert float((got_k - want_k).abs().max()) <= 1.5e-2 * scale
    assert float((got_v - want_v).abs().max()) <= 1.5e-2 * scale
    untouched = torch.ones(pages * ps, dtype=torch.bool)
    untouched[slots.long()] = False
    assert float(kc.cpu().permute(0, 2, 1, 3).reshape(pages * ps, -1)[untouched].abs().max()) == 0.0
    assert torch.equal(new_res.cpu(), x.float())


def _tc_attention_case(n_q, n_kv, d, ps, window, lens, steps, seed=31, spike=None):
    """Like _flash_case, through attention_tc for the portions (and the split-key kernel for requests with
    few rows).  Cache slots that the step cannot see hold NaN."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(seed)
    dtype = torch.bfloat16
    pages = sum((L + ps - 1) // ps for L in lens) + 3
    kc = torch.full((pages, n_kv, ps, d), float("nan"), dtype=dtype)
    vc = torch.full_like(kc, float("nan"))
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max((L + ps - 1) // ps for L in lens) + 1
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    qs, want, positions, cu = [], [], [], [0]
    for i, L in enumerate(lens):
        q = torch.randn(L, n_q, d).to(dtype)
        k = torch.randn(L, n_kv, d).to(dtype)
        v = torch.randn(L, n_kv, d).to(dtype)
        if spike is not None:                                   # one far key that every row must find
            q = (0.1 * torch.randn(L, n_q, d)); k = 0.1 * torch.randn(L, n_kv, d)
            k[spike] = 0; k[spike, :, 0] = 40.0; q[:, :, 0] = 40.0
            q, k = q.to(dtype), k.to(dtype)
        for lp in range((L + ps - 1) // ps):
            table[i, lp] = perm.pop()
        first, count = steps[i]
        for t in range(first + count):
            kc[table[i, t // ps], :, t % ps] = k[t]
            vc[table[i, t // ps], :, t % ps] = v[t]
        o = causal_attention(q.double(), k.double(), v.double(), window=window)
        qs.append(q[first:first + count]); want.append(o[first:first + count])
        positions += list(range(first, first + count))
        cu.append(cu[-1] + count)
    T = cu[-1]
    q = torch.cat(qs).reshape(T, n_q * d)
    out = torch.full((T, n_q * d), float("nan"), dtype=dtype, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    G = n_q // n_kv
    few = [c * G <= 16 for _, c in steps]
    args = (q.to(DEV), out, kc.to(DEV), vc.to(DEV), table.to(DEV), torch.tensor(cu, dtype=torch.int32, device=DEV),
            torch.tensor(positions, dtype=torch.int32, device=DEV), len(lens), max(c for _, c in steps), n_q, n_kv, d,
            window, 1.0 / math.sqrt(d))
    ops.attention_tc(*args, err)
    if any(few):
        ops.flash_attention(*args, 1, None, False, True, err)
    assert err.cpu().tolist()[0] == 0
    assert not torch.isnan(out.float()).any()
    _close(out, torch.cat(want).reshape(T, n_q * d), dtype)
    return out


@pytest.mark.parametrize("n_q,n_kv,d,ps,window", [
    (4, 1, 64, 16, None), (32, 8, 64, 16, None), (8, 1, 128, 16, None), (6, 6, 64, 8, None), (16, 2, 64, 64, None),
    (4, 2, 128, 128, None), (6, 3, 64, 32, 70), (8, 2, 128, 16, 200), (32, 8, 64, 16, 64), (6, 2, 128, 16, None), (5, 1, 64, 16, None),
    (7, 1, 64, 8, 33)])
def test_attention_tcgen05_portions(n_q, n_kv, d, ps, window):
    """Portions from the start, in the middle and at the end of requests, of lengths that leave partial row
    tiles and partial key tiles, beside requests with few rows that the kernel must leave alone."""
    lens = [200, 333, 700, 1, 90, 1100]
    steps = [(0, 200), (150, 183), (699, 1), (0, 1), (60, 30), (513, 587)]
    _tc_attention_case(n_q, n_kv, d, ps, window, lens, steps)


@pytest.mark.parametrize("n_q,n_kv,ps,window", [(32, 8, 16, None), (6, 3, 32, 70), (7, 1, 8, 33), (16, 2, 64, None)])
def test_attention_tcgen05_tiles_of_128_keys(n_q, n_kv, ps, window, monkeypatch):
    """The build with key tiles of 128 (``-DAT_KT=128``, heads of 64: one score buffer in tensor memory, the row's
    scores read twice): kept as an option because it was measured slower, and kept right."""
    from photon_infer_b200.kernels import ops
    real = ops.load_module

    def wide_tiles(module, defines=None):
        if module == "attention_tc" and defines and defines.get("HEAD_DIM") == 64:
            defines = dict(defines, AT_KT=128)
        return real(module, defines)
    monkeypatch.setattr(ops, "load_module", wide_tiles)
    lens = [200, 333, 700, 1, 90, 1100]
    steps = [(0, 200), (150, 183), (699, 1), (0, 1), (60, 30), (513, 587)]
    _tc_attention_case(n_q, n_kv, 64, ps, window, lens, steps)
    for spike in (0, 63, 64, 127, 128, 600):
        _tc_attention_case(4, 1, 64, 16, None, [700], [(640, 60)], seed=40 + spike, spike=spike)


def test_attention_tcgen05_far_key_and_page_edges():
    """A key with a dominant score at a page edge, a tile edge and the far start; every row must land on
    its value row."""
    for spike in (0, 15, 16, 63, 64, 127, 128, 600):
        out = _tc_attention_case(4, 1, 64, 16, None, [700], [(640, 60)], seed=40 + spike, spike=spike)
        assert not torch.isnan(out.float()).any()


def test_attention_tcgen05_refuses_other_sizes():
    from photon_infer_b200.errors import PhotonError
    from photon_infer_b200.kernels import ops
    assert not ops.attention_tc_supported(torch.bfloat16, 80, 4, 16)
    assert not ops.attention_tc_supported(torch.bfloat16, 64, 129, 16)
    assert not ops.attention_tc_supported(torch.bfloat16, 64, 4, 4)
    assert not ops.attention_tc_supported(torch.float32, 64, 4, 16)
    q = torch.zeros(32, 3 * 64, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(4, 1, 4, 64, dtype=torch.bfloat16, device=DEV)            # pages of 4 tokens
    with pytest.raises(PhotonError):
        ops.attention_tc(q, torch.empty_like(q), kc, kc.clone(), torch.zeros(1, 4, dtype=torch.int32, device=DEV),
                         torch.tensor([0, 32], dtype=torch.int32, device=DEV), torch.arange(32, dtype=torch.int32, device=DEV),
                         1, 32, 3, 1, 64, None, 0.125, None)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (1, 8, 8), (100, 300, 72), (257, 513, 520), (2048, 3072, 2048),
                                   (333, 389, 120), (4096, 256, 8192), (129, 129, 136), (2560, 2100, 136)])
def test_gemm_tcgen05_pairs_of_sms(M, N, K):
    """The product on pairs of SMs (cta_group::2) against float64, with partial tiles on every side."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(16)
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    want = x.double() @ w.double().t()
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tc(x, w, out32, "f32", err, pair=True)
    assert err.cpu().tolist()[0] == 0
    assert float((out32.double() - want).abs().max()) <= 2e-6 * math.sqrt(K) * float(want.abs().max())
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x, w, out, "bf16", err, pair=True)
    assert err.cpu().tolist()[0] == 0
    _close(out, want, torch.bfloat16)
    if N % 2 == 0:
        I = N // 2
        act = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_tc(x, w, act, "swiglu", err, pair=True)
        assert err.cpu().tolist()[0] == 0
        g, u = want[:, :I], want[:, I:]
        _close(act, g / (1 + torch.exp(-g)) * u, torch.bfloat16)


@pytest.mark.parametrize("M,n_q,n_kv,d,K,ps,use_table", [(300, 4, 2, 64, 128, 16, True), (513, 6, 2, 32, 72, 8, False),
                                                         (2048, 32, 8, 64, 2048, 16, True), (260, 3, 1, 128, 64, 32, True)])
def test_gemm_tcgen05_qkv_epilogue(M, n_q, n_kv, d, K, ps, use_table):
    """The q/k/v product with rotation and cache write in its epilogue against float64: rotated queries in
    q_out, rotated keys and plain values at their slots of the paged cache, other slots untouched."""
    from photon_infer_b200.kernels import ops
    torch.manual_seed(33)
    N = (n_q + 2 * n_kv) * d
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    inv_freq = (10000.0 ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)).float().to(DEV)
    positions = (torch.arange(M, dtype=torch.int32) + 37).to(DEV)
    pages = (M + ps - 1) // ps + 2
    slots = torch.randperm(pages * ps)[:M].to(torch.int32)
    slots[5] = -1                                               # a token that is not stored
    kc = torch.full((pages, n_kv, ps, d), 7.0, dtype=torch.bfloat16, device=DEV)
    vc = torch.full_like(kc, 7.0)
    q_out = torch.full((M, n_q * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    table = ops.rope_table(inv_freq, 256) if use_table else None     # shorter than the positions: both paths run
    ops.gemm_tc_qkv(x, w, q_out, positions, slots.to(DEV), inv_freq, table, kc, vc, n_q, n_kv, d, err)
    assert err.cpu().tolist()[0] == 0
    y = (x.double() @ w.double().t()).cpu()
    ang = positions.cpu().double()[:, None] * inv_freq.cpu().double()[None, :]
    cs, sn = torch.cos(ang), torch.sin(ang)

    def rotate(t, heads):                                       # neighbouring pairs
        t = t.reshape(M, heads, d // 2, 2)
        a, b = t[..., 0], t[..., 1]
        return torch.stack([a * cs[:, None] - b * sn[:, None], a * sn[:, None] + b * cs[:, None]], dim=-1).reshape(M, heads * d)
    q_want = rotate(y[:, : n_q * d], n_q)
    k_want = rotate(y[:, n_q * d: (n_q + n_kv) * d], n_kv).reshape(M, n_kv, d)
    v_want = y[:, (n_q + n_kv) * d:].reshape(M, n_kv, d)
    _close(q_out, q_want, torch.bfloat16)
    kc_c, vc_c = kc.cpu().double(), vc.cpu().double()
    written = torch.zeros(pages * ps, dtype=torch.bool)
    scale_k, scale_v = float(k_want.abs().max()), float(v_want.abs().max())
    for t in range(M):
        s = int(slots[t])
        if s < 0:
            continue
        written[s] = True
        assert float((kc_c[s // ps, :, s % ps] - k_want[t]).abs().max()) <= 6e-3 * scale_k
        assert float((vc_c[s // ps, :, s % ps] - v_want[t]).abs().max()) <= 6e-3 * scale_v
    untouched = ~written
    assert bool((kc_c.permute(0, 2, 1, 3).reshape(pages * ps, -1)[untouched] == 7.0).all())
    assert bool((vc_c.permute(0, 2, 1, 3).reshape(pages * ps, -1)[untouched] == 7.0).all())
