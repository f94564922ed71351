"""The entry point that allocates nothing, called through its exported C symbol.

Some callers of this library cannot ask the device for memory (another runtime owns the
allocator, or everything was handed out at start-up).  ``photon_skinny_gemm_static`` keeps the
scratch of the few-rows matrix product inside the library image.  Here it is called twice in a
row with different inputs and compared with the regular entry point, which gets its scratch
from the caller; both run the same kernels, so the results must agree to the bit.  This file
sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes
from ctypes import c_int, c_long, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _library():
    from photon_infer_b200.csrc.build import compile_module
    lib = ctypes.CDLL(compile_module("gemm_skinny_static"))
    lib.photon_skinny_gemm_static.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                              c_int, c_int, c_void_p]
    lib.photon_skinny_gemm_static.restype = c_int
    lib.photon_static_error_string.argtypes = [c_int]
    lib.photon_static_error_string.restype = ctypes.c_char_p
    return lib


def _call(lib, x, w, out, epilogue):
    M, K = x.shape
    return lib.photon_skinny_gemm_static(
        c_void_p(x.data_ptr()), x.stride(0), c_void_p(w.data_ptr()), w.stride(0), c_void_p(out.data_ptr()),
        out.stride(0), M, w.shape[0], K, epilogue, c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    from photon_infer_b200.kernels import ops
    lib = _library()
    torch.manual_seed(31)
    # (M, N, K, epilogue): K = 8192 with few rows splits K over blocks (scratch and tickets in use);
    # the second call has other sizes and finds what the first one left in the array
    # the largest N the array has tickets for, and the largest M, are among the cases
    cases = [(8, 2048, 8192, "bf16"), (3, 520, 4104, "f32"), (8, 2048, 8192, "bf16"), (5, 1024, 512, "swiglu"),
             (2, 131072, 64, "f32"), (64, 528, 1024, "bf16")]
    for M, N, K, epi in cases:
        x = torch.randn(M, K, device=DEV).bfloat16()
        w = (torch.randn(N, K, device=DEV) / K ** 0.5).bfloat16()
        cols = N // 2 if epi == "swiglu" else N
        dtype = torch.float32 if epi == "f32" else torch.bfloat16
        want = torch.empty(M, cols, dtype=dtype, device=DEV)
        ops.skinny_gemm(x, w, want, epi)
        got = torch.full((M, cols), float("nan"), dtype=dtype, device=DEV)
        code = _call(lib, x, w, got, {"bf16": 0, "f32": 1, "swiglu": 2}[epi])
        assert code == 0, lib.photon_static_error_string(code).decode()
        torch.cuda.synchronize()
        # The same call once more.  The set-up of the first call on this device is behind us and the driver has
        # loaded this kernel variant's code (it does that at a variant's first launch): now a call must leave
        # the device's free memory and torch's allocator exactly as they were.
        first = got.clone()
        free_before, held_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        code = _call(lib, x, w, got, {"bf16": 0, "f32": 1, "swiglu": 2}[epi])
        assert code == 0, lib.photon_static_error_string(code).decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == held_before
        assert torch.equal(got, first)
        ref = x.double() @ w.double().t()
        if epi == "swiglu":
            ref = ref[:, :cols] / (1 + torch.exp(-ref[:, :cols])) * ref[:, cols:]
        tol = 6e-3 if dtype == torch.bfloat16 else 1e-4
        assert float((got.double() - ref).abs().max()) <= tol * float(ref.abs().max())
        assert torch.equal(got, want), "same kernels, same split of K: the bits must agree"


def test_static_scratch_entry_point_rejects_what_does_not_fit():
    lib = _library()
    x = torch.zeros(65, 64, device=DEV).bfloat16()
    w = torch.zeros(32, 64, device=DEV).bfloat16()
    out = torch.zeros(65, 32, device=DEV).bfloat16()
    code = _call(lib, x, w, out, 0)
    assert code == -4 and b"M <= 64" in lib.photon_static_error_string(code)
    x = torch.zeros(2, 8, device=DEV).bfloat16()
    w = torch.zeros(131072 + 16, 8, device=DEV).bfloat16()
    out = torch.zeros(2, 131072 + 16, device=DEV).bfloat16()
    assert _call(lib, x, w, out, 0) == -4
    # K not a multiple of 8 is refused by the kernel's own check, not run wrongly
    x = torch.zeros(2, 12, device=DEV).bfloat16()
    w = torch.zeros(16, 12, device=DEV).bfloat16()
    out = torch.zeros(2, 16, device=DEV).bfloat16()
    assert _call(lib, x, w, out, 0) == -2
