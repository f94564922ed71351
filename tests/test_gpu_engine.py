"""Generation through the Python entry point and the command line, against the plain
implementation; long decoding; the first tokens of a sequence; preemption."""
import os
import subprocess
import sys

import pytest
import torch

from helpers import ROOT, TINY, TOL, make_model_folder, plain_logits, random_ids, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_model_folder(str(tmp_path_factory.mktemp(name)), name) for name in TINY}


def _options(name, dtype, **kw):
    from photon_infer_b200 import EngineOptions
    args = dict(dtype=dtype, block_size=TINY[name]["block_size"], max_cache_tokens=2048, max_sequences=8,
                chunk_size=16, max_num_batched_tokens=48)
    args.update(kw)
    return EngineOptions(**args)


def _plain_greedy_checked(folder, prompt, got, dtype):
    """``got`` must be the greedy continuation, except that a step whose two best logits lie closer than
    the dtype's tolerance may take either (then the plain side follows the engine's choice)."""
    from plain.llama_plain import PlainLlama
    m = PlainLlama.from_folder(folder)
    ids = list(prompt)
    for step, tok in enumerate(got):
        logits = m.logits(ids)[-1]
        best = int(torch.argmax(logits))
        if tok != best:
            gap = float(logits[best] - logits[tok])
            assert gap <= TOL[dtype] * float(logits.abs().max()), f"token {step}: engine {tok}, plain {best}, gap {gap}"
        ids.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from photon_infer_b200 import ContinuousBatchEngine
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [random_ids(n, vocab, seed=n) for n in (5, 9, 17, 41)]
    engine = ContinuousBatchEngine(folders[name], _options(name, dtype))
    ids = [engine.add_request(p, max_new_tokens=8, ignore_eos=True) for p in prompts]
    out = engine.run_until_complete()
    for rid, p in zip(ids, prompts):
        assert len(out[rid]) == 8 and engine.result(rid).finish_reason == "length"
        _plain_greedy_checked(folders[name], p, out[rid], dtype)
    st = engine.get_stats()
    assert st.num_finished == 4 and st.prefill_tokens == sum(len(p) for p in prompts)
    assert engine.runner.cache.free_pages() == [g.num_pages for g in engine.runner.cache.groups]
    if dtype == "float32":
        from plain.llama_plain import PlainLlama
        assert out[ids[0]] == PlainLlama.from_folder(folders[name]).greedy(prompts[0], 8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """300 tokens decoded one by one from a short prompt, past many page edges and past the window."""
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    name = "tiny_c"
    vocab = TINY[name]["config"]["vocab_size"]
    ids = random_ids(310, vocab, seed=77)
    runner = build_runner(folders[name], _options(name, dtype, max_cache_tokens=320))
    runner.cache.add_request("x")
    got = [runner.step([StepEntry("x", ids[:10], list(range(10)))]).logits.cpu()]
    for t in ids[10:]:
        got.append(runner.step([StepEntry("x", [t], [0])]).logits.cpu())
    runner.check_device_errors()
    got = torch.cat(got)
    want = plain_logits(folders[name], ids)
    assert rel_err(got, want) <= TOL[dtype]
    # the window group kept only a few pages, the full group all of them
    held = [g.pages_held("x") for g in runner.cache.groups]
    assert held[0] <= 24 // 16 + 2 and held[1] == (310 + 15) // 16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_first_tokens_of_a_sequence(folders, name, dtype):
    """Positions 0, 1, 2: a single key, no earlier page, the rotation at angle zero."""
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    vocab = TINY[name]["config"]["vocab_size"]
    ids = random_ids(3, vocab, seed=3)
    runner = build_runner(folders[name], _options(name, dtype))
    want = plain_logits(folders[name], ids)
    for cut in ([1, 1, 1], [3], [1, 2], [2, 1]):
        runner.cache.add_request("f")
        got, p = [], 0
        for n in cut:
            got.append(runner.step([StepEntry("f", ids[p:p + n], list(range(n)))]).logits.cpu())
            p += n
        runner.cache.free_request("f")
        assert rel_err(torch.cat(got), want) <= TOL[dtype], cut
    runner.check_device_errors()


def test_temperature_sampling_is_seeded_and_batch_independent(folders):
    from photon_infer_b200 import ContinuousBatchEngine
    from photon_infer_b200.sampling import uniform
    from plain.llama_plain import PlainLlama, inverse_cdf_sample, temperature_probabilities
    name = "tiny_b"
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [random_ids(n, vocab, seed=50 + n) for n in (3, 12, 31, 70)]

    def run(order):
        engine = ContinuousBatchEngine(folders[name], _options(name, "float32"))
        # request ids follow the order of adding: keep each prompt's id fixed by adding placeholders first
        ids = {}
        for i in order:
            ids[i] = engine.add_request(prompts[i], max_new_tokens=6, temperature=0.8, seed=1234, ignore_eos=True)
        out = engine.run_until_complete()
        return {i: (ids[i], out[ids[i]]) for i in order}

    a = run([0, 1, 2, 3])
    b = run([0, 1, 2, 3])
    assert a == b                                            # same seed, same tokens
    # each token is the inverse-CDF pick of the plain probabilities with the same uniform number
    m = PlainLlama.from_folder(folders[name])
    for i, (rid, toks) in a.items():
        seq = list(prompts[i])
        for k, tok in enumerate(toks):
            p = temperature_probabilities(m.logits(seq)[-1], 0.8)
            u = uniform(1234, rid, k)
            want = inverse_cdf_sample(p, u)
            if tok != want:
                cdf = torch.cumsum(p.double(), 0)
                lo = float(cdf[tok - 1]) if tok > 0 else 0.0
                assert lo - 1e-5 <= u <= float(cdf[tok]) + 1e-5
            seq.append(tok)
    # alone, the first request draws the same tokens as in the batch of four
    alone = run([0])
    assert alone[0] == a[0]
    greedy = ContinuousBatchEngine(folders[name], _options(name, "float32"))
    g = greedy.add_request(prompts[1], max_new_tokens=6, temperature=0.0, ignore_eos=True)
    assert greedy.run_until_complete()[g] == m.greedy(prompts[1], 6)


def test_preemption_on_the_device_changes_no_token(folders):
    """With a pool too small for all requests at once some are preempted and computed again;
    the generated tokens equal those of a run with room for all."""
    from photon_infer_b200 import ContinuousBatchEngine
    name = "tiny_a"
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [random_ids(n, vocab, seed=9 + n) for n in (40, 33, 47, 25)]

    def run(tokens):
        engine = ContinuousBatchEngine(folders[name], _options(name, "float32", max_cache_tokens=tokens))
        ids = [engine.add_request(p, max_new_tokens=40, ignore_eos=True) for p in prompts]
        out = engine.run_until_complete()
        return [out[i] for i in ids], engine.get_stats()

    roomy, st1 = run(4096)
    tight, st2 = run(192)                                     # 12 pages of 16: not enough for four requests of ~80
    assert st1.preemptions == 0 and st2.preemptions > 0
    assert roomy == tight


def test_eos_stops_generation(folders):
    from photon_infer_b200 import ContinuousBatchEngine
    from plain.llama_plain import PlainLlama
    name = "tiny_a"
    m = PlainLlama.from_folder(folders[name])
    prompt = random_ids(12, 256, seed=4)
    free_run = m.greedy(prompt, 10)
    import json
    cfg = json.load(open(os.path.join(folders[name], "config.json")))
    cfg["eos_token_id"] = free_run[4]
    alt = folders[name] + "_eos"
    os.makedirs(alt, exist_ok=True)
    json.dump(cfg, open(os.path.join(alt, "config.json"), "w"))
    if not os.path.exists(os.path.join(alt, "model.safetensors")):
        os.link(os.path.join(folders[name], "model.safetensors"), os.path.join(alt, "model.safetensors"))
    engine = ContinuousBatchEngine(alt, _options(name, "float32"))
    rid = engine.add_request(prompt, max_new_tokens=10)
    out = engine.run_until_complete()[rid]
    stop = free_run.index(free_run[4])
    assert out == free_run[:stop + 1] and engine.result(rid).finish_reason == "eos"


def test_bad_prompt_token_is_refused(folders):
    from photon_infer_b200 import ContinuousBatchEngine, PhotonError
    engine = ContinuousBatchEngine(folders["tiny_a"], _options("tiny_a", "float32"))
    with pytest.raises(PhotonError):
        engine.add_request([1, 256, 3])


def test_command_line(folders):
    name = "tiny_a"
    prompt = random_ids(9, 256, seed=21)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "llama_infer"), folders[name], "cuda", "--dtype", "fp32",
           "--prompt-ids", ",".join(map(str, prompt)), "--prompt-ids", "7 8 9", "--max-new-tokens", "5",
           "--temperature", "0", "--ignore-eos", "--num-blocks", "32", "--no-quantize"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    lines = [l for l in res.stdout.splitlines() if l.startswith("request")]
    from plain.llama_plain import PlainLlama
    m = PlainLlama.from_folder(folders[name])
    assert lines[0].split(": ")[1].split() == [str(t) for t in m.greedy(prompt, 5)]
    assert lines[1].split(": ")[1].split() == [str(t) for t in m.greedy([7, 8, 9], 5)]
    assert "tokens/s" in res.stderr
    bad = subprocess.run(cmd[:3] + ["cpu"] + cmd[4:], capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0 and "CUDA only" in bad.stderr
    bad = subprocess.run(cmd + ["--quantize"], capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0 and "INT8" in bad.stderr


def test_pipelined_decode_equals_step_by_step(folders):
    """Decode steps enqueued one ahead (ids still on the device) give the same tokens and finish reasons as
    steps that wait for their ids, also when one request meets end-of-sequence while the next step is
    already in flight, when another runs out of new tokens, and with temperature sampling."""
    import json
    from photon_infer_b200 import ContinuousBatchEngine
    from plain.llama_plain import PlainLlama
    name = "tiny_a"
    m = PlainLlama.from_folder(folders[name])
    prompts = [random_ids(n, 256, seed=70 + n) for n in (12, 7, 21, 15)]
    free_run = m.greedy(prompts[0], 30)
    eos = free_run[9]                                       # request 0 stops at its first occurrence of this id
    cfg = json.load(open(os.path.join(folders[name], "config.json")))
    cfg["eos_token_id"] = eos
    alt = folders[name] + "_eos2"
    os.makedirs(alt, exist_ok=True)
    json.dump(cfg, open(os.path.join(alt, "config.json"), "w"))
    if not os.path.exists(os.path.join(alt, "model.safetensors")):
        os.link(os.path.join(folders[name], "model.safetensors"), os.path.join(alt, "model.safetensors"))

    def run(async_decode):
        eng = ContinuousBatchEngine(alt, _options(name, "float32", async_decode=async_decode))
        ids = [eng.add_request(prompts[0], max_new_tokens=30),
               eng.add_request(prompts[1], max_new_tokens=5, ignore_eos=True),
               eng.add_request(prompts[2], max_new_tokens=40, temperature=0.9, seed=5, ignore_eos=True),
               eng.add_request(prompts[3], max_new_tokens=33, ignore_eos=True)]
        out = eng.run_until_complete()
        assert eng.runner.cache.free_pages() == [g.num_pages for g in eng.runner.cache.groups]
        return [(out[i], eng.result(i).finish_reason) for i in ids], eng

    a, eng_a = run(True)
    b, _ = run(False)
    assert a == b
    assert a[0][1] == "eos" and a[0][0] == free_run[: free_run.index(eos) + 1]
    assert a[1][1] == "length" and len(a[1][0]) == 5
    assert a[3][0] == m.greedy(prompts[3], 33)
    assert eng_a._inflight is None


def test_captured_decode_steps_keep_their_scratch(tmp_path, monkeypatch):
    """Decode steps replayed as CUDA graphs with the persistent attention kernel (forced here at short contexts,
    chunks of one tile, so that partial results go through its scratch buffer): the buffer a captured step writes
    to must stay owned after the step that captured it is gone.  Tensors allocated after the capture are the
    victims if it does not: they must stay zero, and the replayed steps must agree with the plain implementation."""
    from helpers import TINY, TOL, make_model_folder, plain_logits, random_ids, rel_err
    from photon_infer_b200 import EngineOptions
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    from photon_infer_b200.kernels import ops
    from photon_infer_b200.parts import attention
    folder = make_model_folder(str(tmp_path / "m"), "tiny_d")
    vocab = TINY["tiny_d"]["config"]["vocab_size"]
    monkeypatch.setattr(attention, "DECODE_TMA_MIN_KEYS", {64: 1})
    monkeypatch.setattr(ops, "attention_decode_plan", lambda n, n_kv, keys, d, page: (1, n * (keys // 64 + 2), n * (keys // 64 + 2) * n_kv))
    seen = []
    real = ops.attention_decode

    def spy(*a, **kw):
        seen.append(a[14])                                   # the scratch tensor of this launch
        return real(*a, **kw)
    monkeypatch.setattr(ops, "attention_decode", spy)
    runner = build_runner(folder, EngineOptions(dtype="bfloat16", block_size=32, max_cache_tokens=4096, max_sequences=8,
                                                use_cuda_graphs=True))
    seqs = [random_ids(150 + 37 * i, vocab, seed=70 + i) for i in range(3)]
    for i, ids in enumerate(seqs):
        runner.cache.add_request(i)
        runner.step([StepEntry(i, ids[:-4], [])])
    victims = []
    for k in range(4):                                       # four decode steps: the first captures, the others replay
        got = runner.step([StepEntry(i, [seqs[i][len(seqs[i]) - 4 + k]], [0]) for i in range(3)]).logits.float().cpu()
        for i, ids in enumerate(seqs):
            want = plain_logits(folder, ids[: len(ids) - 3 + k])[-1:]
            assert rel_err(got[i: i + 1], want) <= TOL["bfloat16"], (k, i)
        for v in victims:
            assert float(v.abs().max()) == 0.0               # nobody wrote into memory that has a new owner
        # what the allocator hands out now is what a freed scratch buffer would have left behind
        victims += [torch.zeros(n, dtype=torch.float32, device="cuda:0") for n in (1 << 12, 1 << 14, 1 << 16, 1 << 18, 1 << 20)]
    runner.check_device_errors()
    assert seen and runner.graph_kernel_launches > 0
    owned = {t.data_ptr() for t in ops._decode_scratch[("cuda", 0)]}
    assert all(t.data_ptr() in owned for t in seen)


@pytest.mark.parametrize("name,dtype", [("tiny_a", "float32"), ("tiny_d", "bfloat16")])
def test_graphs_that_come_and_go_change_no_token(folders, name, dtype):
    """Requests that arrive and finish at different times run decode steps of many batch sizes and block-table
    widths; with room for three captured graphs only, graphs are dropped and captured again all the time.  The
    tokens must be those of an engine without graphs (float32: exactly; bfloat16: both are checked against the
    plain implementation under the tie rule, because a graph pads its batch and padding changes no row)."""
    from photon_infer_b200 import ContinuousBatchEngine
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [random_ids(5 + 11 * i, vocab, seed=300 + i) for i in range(7)]
    lengths = [40, 9, 33, 21, 50, 14, 27]

    def run(graphs):
        eng = ContinuousBatchEngine(folders[name], _options(name, dtype, use_cuda_graphs=graphs, max_cache_tokens=4096))
        if graphs:
            eng.runner.max_graphs = 3
        ids = []
        pending = list(zip(prompts, lengths))
        steps = 0
        while pending or eng.has_work():
            if pending and steps % 3 == 0:                   # one arrival every third step
                p, n = pending.pop(0)
                ids.append(eng.add_request(p, max_new_tokens=n, ignore_eos=True))
            eng.step()
            steps += 1
        out = [list(eng.result(i).generated_tokens) for i in ids]
        eng.runner.check_device_errors()
        assert eng.runner.cache.free_pages() == [g.num_pages for g in eng.runner.cache.groups]
        return out, eng
    with_graphs, eng = run(True)
    assert eng.runner.graph_kernel_launches > 0 and len(eng.runner._graphs) <= 3
    without, _ = run(False)
    assert [len(t) for t in with_graphs] == lengths
    if dtype == "float32":
        assert with_graphs == without
    else:
        for p, got in zip(prompts, with_graphs):
            _plain_greedy_checked(folders[name], p, got, dtype)
