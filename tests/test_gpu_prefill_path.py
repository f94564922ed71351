"""The kernels that long prompt portions and large decode batches run, inside the model, against the plain
implementation: two layers at the width of Llama 3.2 1B (hidden 2,048, 32/8 heads of 64, intermediate
8,192) with a vocabulary of 32,000.  At this width a portion of 2,048 tokens reaches the tcgen05 product on
pairs of SMs with the rotation and the cache write in its epilogue, the tcgen05 attention over the pages
that epilogue just wrote, and the pairs product with the SwiGLU epilogue; a decode step of 64 requests
runs the library products between the package's own norm, rotation and split-key attention kernels.

The weights are drawn wider than usual (0.04) so that attention is far from uniform: a key in the wrong
slot then moves the logits by much more than the tolerance, which the last test shows by breaking the
block table on purpose.
"""
import pytest
import torch

from helpers import TOL, plain_logits, random_ids, rel_err

pytestmark = pytest.mark.gpu

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=8192, num_hidden_layers=2,
           num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=32000,
           max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
           rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                             original_max_position_embeddings=8192),
           tie_word_embeddings=True)
N = 2048
ROWS = [0, 1, 15, 16, 127, 128, 700, 1023, 1024, 1025, 1500, 2046, 2047]
CUT_TOL = 1.5e-2          # two ways of cutting one request, bfloat16: a rounding of the activations


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from photon_infer_b200.weights import write_random_model
    f = str(tmp_path_factory.mktemp("width_1b"))
    write_random_model(f, CFG, seed=21, init_std=0.04, norm_std=0.1)
    return f


@pytest.fixture(scope="module")
def runner(folder):
    from photon_infer_b200 import EngineOptions
    from photon_infer_b200.engine.loading import build_runner
    return build_runner(folder, EngineOptions(dtype="bfloat16", block_size=16, max_cache_tokens=20000,
                                              max_sequences=80, use_cuda_graphs=True))


class Spy:
    """Counts calls of the kernels' Python entries and lets them through."""

    def __init__(self, monkeypatch, names):
        from photon_infer_b200.kernels import ops
        self.calls = {n: [] for n in names}
        for n in names:
            real = getattr(ops, n)

            def wrapped(*a, _real=real, _n=n, **kw):
                self.calls[_n].append((a, kw))
                return _real(*a, **kw)
            monkeypatch.setattr(ops, n, wrapped)


def _step(runner, entries):
    from photon_infer_b200.engine.runner import StepEntry
    return runner.step([StepEntry(*e) for e in entries]).logits.float().cpu()


def test_one_portion_and_two_halves(folder, runner, monkeypatch):
    ids = random_ids(N, CFG["vocab_size"], seed=5)
    want = plain_logits(folder, ids)[ROWS]
    spy = Spy(monkeypatch, ["gemm_tc_qkv", "attention_tc", "gemm_tc"])
    runner.cache.add_request("whole")
    whole = _step(runner, [("whole", ids, ROWS)])
    runner.cache.free_request("whole")
    # per layer: the q/k/v product with its epilogue, the tcgen05 attention, and O, gate/up, down on pairs of SMs
    assert len(spy.calls["gemm_tc_qkv"]) == 2 and len(spy.calls["attention_tc"]) == 2
    assert sum(1 for a, kw in spy.calls["gemm_tc"] if kw.get("pair")) == 6
    runner.cache.add_request("halves")
    first = _step(runner, [("halves", ids[:1024], [r for r in ROWS if r < 1024])])
    second = _step(runner, [("halves", ids[1024:], [r - 1024 for r in ROWS if r >= 1024])])
    runner.cache.free_request("halves")
    assert len(spy.calls["gemm_tc_qkv"]) == 6 and len(spy.calls["attention_tc"]) == 6
    runner.check_device_errors()
    halves = torch.cat([first, second])
    assert rel_err(whole, want) <= TOL["bfloat16"]
    assert rel_err(halves, want) <= TOL["bfloat16"]
    assert rel_err(halves, whole) <= CUT_TOL


def test_portion_beside_decoded_tokens_of_other_requests(folder, runner, monkeypatch):
    """A 1,500-token portion and, in the same step, one token each of eight requests that hold 600 to 700
    tokens: the tcgen05 kernels take the portion, the split-key kernel the eight, from one block table."""
    vocab = CFG["vocab_size"]
    long_ids = random_ids(1500, vocab, seed=6)
    others = [random_ids(600 + 13 * i + 1, vocab, seed=40 + i) for i in range(8)]
    for i, ids in enumerate(others):
        runner.cache.add_request(("o", i))
    # the eight prompts, all but their last token, four requests per step
    for lo in (0, 4):
        _step(runner, [(("o", i), others[i][:-1], []) for i in range(lo, lo + 4)])
    spy = Spy(monkeypatch, ["gemm_tc_qkv", "attention_tc", "flash_attention"])
    runner.cache.add_request("long")
    rows = [0, 16, 777, 1498, 1499]
    got = _step(runner, [("long", long_ids, rows)] + [(("o", i), [others[i][-1]], [0]) for i in range(8)])
    runner.check_device_errors()
    assert len(spy.calls["gemm_tc_qkv"]) == 2 and len(spy.calls["attention_tc"]) == 2
    assert len(spy.calls["flash_attention"]) == 2           # the eight single tokens
    for rid in ["long"] + [("o", i) for i in range(8)]:
        runner.cache.free_request(rid)
    assert rel_err(got[:5], plain_logits(folder, long_ids)[rows]) <= TOL["bfloat16"]
    for i, ids in enumerate(others):
        assert rel_err(got[5 + i: 6 + i], plain_logits(folder, ids)[-1:]) <= TOL["bfloat16"], f"request {i}"


@pytest.mark.parametrize("batch", [64, 50])
def test_decode_step_of_many_requests(folder, runner, monkeypatch, batch):
    """64 requests of 40 to 103 cached tokens decode one token each in one captured step (512 (request,
    key/value head) pairs, more than the GPU has SMs); 50 requests run the graph of 64 with padding rows."""
    from photon_infer_b200.kernels import ops
    vocab = CFG["vocab_size"]
    seqs = [random_ids(41 + i, vocab, seed=200 + i) for i in range(batch)]
    for i in range(batch):
        runner.cache.add_request(("d", i))
    for lo in range(0, batch, 16):
        _step(runner, [(("d", i), seqs[i][:-1], []) for i in range(lo, min(batch, lo + 16))])
    spy = Spy(monkeypatch, ["flash_attention", "skinny_gemm"])
    got = _step(runner, [(("d", i), [seqs[i][-1]], [0]) for i in range(batch)])
    runner.check_device_errors()
    for i in range(batch):
        runner.cache.free_request(("d", i))
    assert got.shape[0] == batch
    if spy.calls["flash_attention"]:                        # the first step of this shape: captured now
        a, kw = spy.calls["flash_attention"][0]
        assert a[7] * CFG["num_key_value_heads"] > ops.sm_count(torch.device("cuda:0")) and not spy.calls["skinny_gemm"]
    for i, ids in enumerate(seqs):
        assert rel_err(got[i: i + 1], plain_logits(folder, ids)[-1:]) <= TOL["bfloat16"], f"request {i}"


def test_a_wrong_block_table_is_seen(folder, runner, monkeypatch):
    """The control: two pages of the request swapped in the table that attention reads.  If this stayed
    within the tolerance, the tests above could not tell a right cache from a wrong one."""
    from photon_infer_b200.kernels import ops
    ids = random_ids(N, CFG["vocab_size"], seed=5)
    want = plain_logits(folder, ids)[ROWS]
    real = ops.attention_tc

    def broken(q, out, k_cache, v_cache, block_table, *rest, **kw):
        table = block_table.clone()
        table[0, 3], table[0, 40] = block_table[0, 40], block_table[0, 3]
        return real(q, out, k_cache, v_cache, table, *rest, **kw)
    monkeypatch.setattr(ops, "attention_tc", broken)
    runner.cache.add_request("broken")
    got = _step(runner, [("broken", ids, ROWS)])
    runner.cache.free_request("broken")
    assert rel_err(got, want) > 4 * TOL["bfloat16"]
