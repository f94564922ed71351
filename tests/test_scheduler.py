"""The scheduler's decisions, driven on the host with a stand-in for the step function."""
import pytest
import torch

from photon_infer_b200.cache import CacheManager
from photon_infer_b200.engine import ContinuousBatchScheduler, RequestState, SamplingParams
from photon_infer_b200.errors import PhotonError
from photon_infer_b200.parts.base import PagedCacheSpec


def _sched(num_pages=64, page_size=8, **kw):
    cache = CacheManager([(PagedCacheSpec(2, 16, None), None)] * 2, [None, None], page_size, num_pages,
                         kw.pop("max_sequences", 8), torch.float32, None)
    args = dict(max_batch_size=8, max_sequences=8, chunk_size=16, max_num_batched_tokens=40, max_model_len=256,
                eos_token_ids=(2,), commits_lengths=True)
    args.update(kw)
    return ContinuousBatchScheduler(cache, **args), cache


def _run(s, next_token=lambda req: 100 + req.num_generated(), limit=10000):
    """Steps until done; returns the batches as [(request id, tokens fed)]."""
    log = []
    for _ in range(limit):
        if not s.has_work():
            return log
        b = s.schedule_next_batch()
        fed = [(it.request.request_id, it.request.next_tokens(it.num_tokens)) for it in b.items]
        log.append((fed, [r.request_id for r in b.preempted], [r.request_id for r in b.failed]))
        s.update_after_step(b, {it.request.request_id: next_token(it.request) for it in b.items if it.samples})
    raise AssertionError("the scheduler did not finish")


def test_prompt_is_cut_into_portions_under_the_budget():
    s, _ = _sched()
    a = s.add_request(list(range(1000, 1037)), SamplingParams(max_new_tokens=3))
    b = s.add_request(list(range(2000, 2030)), SamplingParams(max_new_tokens=2))
    log = _run(s)
    sizes = [[(rid, len(t)) for rid, t in fed] for fed, _, _ in log]
    # step 0: a gets a portion of 16 (chunk), b 16; budget 40 leaves 8 unused only because of the chunk limit
    assert sizes[0] == [(a, 16), (b, 16)]
    assert sizes[1] == [(a, 16), (b, 14)]               # b's prompt ends: it samples
    assert sizes[2] == [(a, 5), (b, 1)]                 # a's last portion beside b's first decoded token
    assert all(sum(n for _, n in step) <= 40 for step in sizes)
    # the logits of the last prompt token give the first generated token: no token is fed twice
    fed_a = [t for fed, _, _ in log for rid, toks in fed if rid == a for t in toks]
    assert fed_a == list(range(1000, 1037)) + [100, 101]
    assert s.get_request(a).generated_tokens == [100, 101, 102]
    assert s.get_request(a).finish_reason == "length" and s.get_request(b).finish_reason == "length"
    st = s.get_stats()
    assert st.num_finished == 2 and st.num_running == 0 and st.prefill_tokens == 67 and st.decode_tokens == 3


def test_budget_smaller_than_a_portion():
    s, _ = _sched(max_num_batched_tokens=10)
    a = s.add_request(list(range(25)), SamplingParams(max_new_tokens=1))
    b = s.add_request(list(range(7)), SamplingParams(max_new_tokens=4))
    log = _run(s)
    sizes = [[(rid, len(t)) for rid, t in fed] for fed, _, _ in log]
    assert sizes[0] == [(a, 10)]                         # nothing left for b: it waits
    assert sizes[1] == [(a, 10)]
    assert sizes[2] == [(a, 5), (b, 5)]                  # running first, then the budget that is left
    assert sizes[3] == [(b, 2)]


def test_running_requests_come_first_and_admission_is_fcfs():
    s, _ = _sched(max_batch_size=2, max_num_batched_tokens=100)
    ids = [s.add_request([1, 2, 3], SamplingParams(max_new_tokens=3)) for _ in range(4)]
    log = _run(s)
    first = [[rid for rid, _ in fed] for fed, _, _ in log]
    assert first[0] == ids[:2] and first[1] == ids[:2] and first[2] == ids[:2]
    assert first[3] == ids[2:]                           # the next two only when the first two are done


def test_max_sequences_limits_live_requests():
    s, cache = _sched(max_sequences=2, max_num_batched_tokens=100)
    for _ in range(5):
        s.add_request([1, 2, 3, 4], SamplingParams(max_new_tokens=5))
    while s.has_work():
        b = s.schedule_next_batch()
        assert s.num_running() <= 2 and len(cache.live_requests()) <= 2
        s.update_after_step(b, {it.request.request_id: 9 for it in b.items if it.samples})
    assert s.get_stats().num_finished == 5


def test_eos_finishes_and_frees():
    s, cache = _sched()
    a = s.add_request([5, 6, 7], SamplingParams(max_new_tokens=50))
    b = s.add_request([5, 6, 7], SamplingParams(max_new_tokens=4, ignore_eos=True))
    _run(s, next_token=lambda req: 2 if req.num_generated() == 2 else 11)
    assert s.get_request(a).generated_tokens == [11, 11, 2] and s.get_request(a).finish_reason == "eos"
    assert s.get_request(b).generated_tokens == [11, 11, 2, 11] and s.get_request(b).finish_reason == "length"
    assert cache.free_pages() == [64] and cache.live_requests() == []


def test_model_len_finishes():
    s, _ = _sched(max_model_len=12)
    a = s.add_request(list(range(10)), SamplingParams(max_new_tokens=50))
    _run(s)
    assert s.get_request(a).finish_reason == "model_len" and s.get_request(a).total_tokens() == 12
    with pytest.raises(PhotonError):
        s.add_request(list(range(12)))
    with pytest.raises(PhotonError):
        s.add_request([])


def test_pages_run_out_last_admitted_is_preempted_and_recomputed():
    # 6 pages of 8 tokens: two requests of 20 tokens (3 pages each) fit, their growth does not
    s, cache = _sched(num_pages=6, max_num_batched_tokens=100, chunk_size=32)
    a = s.add_request(list(range(300, 320)), SamplingParams(max_new_tokens=12))
    b = s.add_request(list(range(400, 420)), SamplingParams(max_new_tokens=12))
    log = _run(s)
    preempted = [p for _, pre, _ in log for p in pre]
    assert preempted and set(preempted) == {b}           # the one admitted last gives way
    assert s.get_request(a).num_preemptions == 0 and s.get_request(b).num_preemptions >= 1
    # both finish with all their tokens, and b was fed its own generated tokens again after coming back
    assert s.get_request(a).generated_tokens == [100 + i for i in range(12)]
    assert s.get_request(b).generated_tokens == [100 + i for i in range(12)]
    refeeds = [toks for fed, _, _ in log for rid, toks in fed if rid == b and toks[:1] == [400]]
    assert len(refeeds) >= 2 and any(t >= 100 and t < 200 for t in refeeds[-1])
    # no request was admitted in a step that preempted one
    for fed, pre, _ in log:
        if pre:
            assert all(rid != b for rid, _ in fed)
    assert cache.free_pages() == [6] and s.get_stats().preemptions == len(preempted)
    cache.check_consistency()


def test_a_request_that_can_never_fit_fails_alone():
    s, cache = _sched(num_pages=2, max_num_batched_tokens=100, chunk_size=64)
    big = s.add_request(list(range(40)), SamplingParams(max_new_tokens=2))          # 5 pages > 2
    small = s.add_request([1, 2, 3], SamplingParams(max_new_tokens=2))
    log = _run(s)
    assert s.get_request(big).finish_reason == "out_of_memory" and s.get_request(big).generated_tokens == []
    assert s.get_request(small).finish_reason == "length"
    assert big in [f for _, _, failed in log for f in failed]
    # one that outgrows the pool while running alone
    s, cache = _sched(num_pages=2, max_num_batched_tokens=100)
    g = s.add_request(list(range(14)), SamplingParams(max_new_tokens=20))
    _run(s)
    assert s.get_request(g).finish_reason == "out_of_memory" and s.get_request(g).num_generated() == 3
    assert cache.free_pages() == [2]


def test_abort():
    s, cache = _sched()
    a = s.add_request(list(range(10)), SamplingParams(max_new_tokens=50))
    b = s.add_request(list(range(10)), SamplingParams(max_new_tokens=50))
    batch = s.schedule_next_batch()
    s.update_after_step(batch, {it.request.request_id: 9 for it in batch.items if it.samples})
    s.abort(a)
    assert s.get_request(a).finish_reason == "aborted" and s.get_request(a).state == RequestState.FINISHED
    assert cache.live_requests() == [b]
    s.abort(b)
    assert not s.has_work() and cache.free_pages() == [64]


def test_key_shares_of_decoded_tokens():
    """Blocks and groups of warps per (request, key/value head): groups while every pair can have an SM,
    blocks on top only for long contexts, one group and about 256 blocks beyond."""
    from photon_infer_b200.parts.attention import choose_key_shares
    assert choose_key_shares(64, 640, 4) == (1, 4)          # batch 8, 8 key/value heads
    assert choose_key_shares(64, 4096, 4) == (2, 4)
    assert choose_key_shares(8, 8192, 4) == (8, 4)          # batch 1
    assert choose_key_shares(128, 640, 4) == (1, 4)
    assert choose_key_shares(512, 640, 4) == (1, 1)         # batch 64
    assert choose_key_shares(160, 4096, 4) == (2, 1)
    assert choose_key_shares(64, 640, 1) == (4, 1)          # a head size with room for one group only
    assert choose_key_shares(1, 30, 4) == (1, 4)
