"""Which kernel a size goes to: the rules of kernels/ops.py, checked without a GPU."""
import torch

from photon_infer_b200.kernels import ops


def test_tcgen05_product_wants_enough_tiles_and_rows():
    assert ops.gemm_tc_tiles(64, 3072) == 0                       # a tile of 128 rows would be mostly padding
    assert ops.gemm_tc_tiles(128, 3072) == 12
    assert ops.gemm_tc_tiles(2048, 3072) == 16 * 12
    assert ops.gemm_tc_tiles(2048, 16384, swiglu=True) == 16 * 64  # a SwiGLU tile covers 128 output columns
    assert ops.gemm_tc_tiles(512, 3072) < ops.TC_MIN_TILES <= ops.gemm_tc_tiles(2048, 2048)
    assert ops.TC_PAIR_MIN_ROWS == 256 and ops.SKINNY_MAX_ROWS == 8


def test_tcgen05_product_refuses_what_tma_cannot_load():
    x = torch.zeros(256, 64, dtype=torch.bfloat16)
    w = torch.zeros(512, 64, dtype=torch.bfloat16)
    assert ops.gemm_tc_supported(x, w)
    assert not ops.gemm_tc_supported(x.float(), w.float())        # bfloat16 only
    assert not ops.gemm_tc_supported(x[:, :60], w[:, :60])        # K not a multiple of 8, rows not contiguous
    assert not ops.gemm_tc_supported(x, w[::2])                   # weight not contiguous
    xs = torch.zeros(256, 72, dtype=torch.bfloat16)[:, :64]       # row stride 72: a multiple of 8, allowed
    assert ops.gemm_tc_supported(xs, w)
    xo = torch.zeros(256 * 64 + 4, dtype=torch.bfloat16)[4:].view(256, 64)   # base 8 bytes off a 16-byte boundary
    assert not ops.gemm_tc_supported(xo, w)


def test_qkv_epilogue_wants_long_portions_and_heads_in_steps_of_32():
    w = torch.zeros(3072, 2048, dtype=torch.bfloat16)
    assert ops.gemm_tc_qkv_supported(torch.zeros(2048, 2048, dtype=torch.bfloat16), w, 64)
    assert ops.gemm_tc_qkv_supported(torch.zeros(2048, 2048, dtype=torch.bfloat16), w, 128)
    assert not ops.gemm_tc_qkv_supported(torch.zeros(2048, 2048, dtype=torch.bfloat16), w, 48)
    assert not ops.gemm_tc_qkv_supported(torch.zeros(128, 2048, dtype=torch.bfloat16), w, 64)    # fewer than 256 rows
    assert not ops.gemm_tc_qkv_supported(torch.zeros(512, 2048, dtype=torch.bfloat16), w, 64)    # too few tiles


def test_tcgen05_attention_sizes():
    bf = torch.bfloat16
    for group in (1, 3, 4, 5, 128):
        assert ops.attention_tc_supported(bf, 64, group, 16)
    for page in (8, 16, 32, 64, 128, 256):
        assert ops.attention_tc_supported(bf, 128, 4, page)
    assert not ops.attention_tc_supported(bf, 64, 129, 16)        # more rows per token than a tile holds
    assert not ops.attention_tc_supported(bf, 96, 4, 16)          # heads of 64 or 128 only
    assert not ops.attention_tc_supported(bf, 64, 4, 4)           # a TMA box needs pages of 8 tokens or more
    assert not ops.attention_tc_supported(bf, 64, 4, 24)          # pages must divide 64 or be a multiple of it
    assert not ops.attention_tc_supported(bf, 64, 4, 96)
    assert not ops.attention_tc_supported(torch.float32, 64, 4, 16)
    assert ops.flash_attention_supported(bf, 48) and not ops.flash_attention_supported(bf, 136)
    assert not ops.flash_attention_supported(torch.float32, 64)   # float32 takes the general kernel


def test_weight_streaming_product_sizes():
    x = torch.zeros(8, 2048, dtype=torch.bfloat16)
    w = torch.zeros(3072, 2048, dtype=torch.bfloat16)
    assert ops.skinny_gemm_supported(x, w)
    assert ops.skinny_gemm_supported(torch.zeros(64, 2048, dtype=torch.bfloat16), w)
    assert not ops.skinny_gemm_supported(torch.zeros(65, 2048, dtype=torch.bfloat16), w)
    assert not ops.skinny_gemm_supported(torch.zeros(33, 2048, dtype=torch.bfloat16), w, swiglu=True)
    assert not ops.skinny_gemm_supported(torch.zeros(8, 2044, dtype=torch.bfloat16), torch.zeros(16, 2044, dtype=torch.bfloat16))
