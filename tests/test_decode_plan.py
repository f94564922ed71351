"""How the persistent decode attention kernel's work is cut (``ops.attention_decode_plan``): pure arithmetic, no GPU."""
import pytest

from photon_infer_b200.kernels import ops


@pytest.fixture(autouse=True)
def slots(monkeypatch):
    monkeypatch.setattr(ops, "attention_decode_slots", lambda head_dim: 296)       # two blocks on each of 148 SMs


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("num_seqs", [1, 3, 8, 16, 64, 200, 512])
@pytest.mark.parametrize("keys", [1, 63, 64, 65, 500, 1200, 4096, 16500, 100000, 250000])
def test_plan_covers_every_key_within_the_kernels_limits(head_dim, num_seqs, keys):
    n_kv = 8
    plan = ops.attention_decode_plan(num_seqs, n_kv, keys, head_dim, 16)
    assert plan is not None
    chunk, chunks, items = plan
    tiles = -(-keys // 64) + 1
    per_seq = -(-tiles // chunk)
    assert 1 <= chunk <= 64                                   # a lane keeps the pages of at most 64 tiles
    assert per_seq <= min(120, head_dim)                      # the merge buffer holds that many chunk weights per row
    assert chunks == num_seqs * per_seq and items == chunks * n_kv
    assert per_seq * chunk >= tiles


def test_plan_refuses_more_keys_than_chunks_hold():
    assert ops.attention_decode_plan(1, 8, 64 * 64 * 64 + 1, 64, 16) is None
    assert ops.attention_decode_plan(1, 8, 64 * 64 * 64 - 64, 64, 16) is not None
    assert ops.attention_decode_plan(1, 8, 120 * 64 * 64 + 1, 128, 16) is None


def test_plan_prefers_one_round_of_items():
    """Measured cases: many short requests run whole; few long ones are cut so that the items fill the blocks
    once or in equal rounds, not once and a bit."""
    assert ops.attention_decode_plan(64, 8, 640, 128, 16)[0] == 11            # 512 pairs: whole requests (10 + 1 tiles)
    chunk, chunks, items = ops.attention_decode_plan(8, 8, 4096, 128, 16)     # 64 pairs x 4 chunks = 256 items, one round
    assert chunk == 17 and items == 256
    chunk, chunks, items = ops.attention_decode_plan(8, 8, 16500, 128, 16)    # not 5 chunks (320 items on 296 blocks)
    assert items % 64 == 0 and (items <= 296 or items >= 2 * 296 - 64)
    chunk, chunks, items = ops.attention_decode_plan(16, 8, 8192, 64, 16)     # not 3 chunks of 43 (384 items)
    assert chunk == 33 and items == 512
