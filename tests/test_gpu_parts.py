"""Each part of a layer alone against the plain implementation; a layer run twice and a layer
that reads another's cache; a toy mixer with state of its own, defined here, registered,
built and stepped without a change to the framework's files."""
import math
import os

import pytest
import torch

from helpers import TINY, TOL, make_model_folder, plain_logits, random_ids, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ctx(tokens_per_seq, starts, page_size, n_groups=1, dtype=torch.float32, table=None, num_pages=64):
    """A hand-made StepContext: request i owns pages i*8 .. i*8+7 in order."""
    from photon_infer_b200.parts.base import GroupView, StepContext
    T = sum(tokens_per_seq)
    S = len(tokens_per_seq)
    pos, seq, slots = [], [], []
    for s, (n, st) in enumerate(zip(tokens_per_seq, starts)):
        for p in range(st, st + n):
            pos.append(p); seq.append(s); slots.append((s * 8 + p // page_size) * page_size + p % page_size)
    bt = torch.tensor([[s * 8 + i for i in range(8)] for s in range(S)], dtype=torch.int32, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    g = GroupView(bt, i32(slots), page_size, num_pages, 8)
    cu = [0]
    for n in tokens_per_seq:
        cu.append(cu[-1] + n)
    return StepContext(T, S, dtype, i32([0] * T), i32(pos), i32(seq), i32(cu), i32([a + b for a, b in zip(tokens_per_seq, starts)]),
                       i32(list(range(S))), [g] * n_groups, tokens_per_seq, [a + b for a, b in zip(tokens_per_seq, starts)],
                       starts, max(tokens_per_seq), max(a + b for a, b in zip(tokens_per_seq, starts)),
                       torch.zeros(4, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from photon_infer_b200.parts.registry import create_part
    from plain.llama_plain import rms_norm
    torch.manual_seed(0)
    norm = create_part("norm", "rms_norm", {"size": 200, "eps": 1e-6})
    assert [(t.name, t.shape, t.role) for t in norm.tensor_specs()] == [("weight", (200,), "vector")]
    w = 1 + 0.1 * torch.randn(200)
    norm.load({"weight": w.to(DEV)})
    x = torch.randn(5, 200)
    d = torch.randn(5, 200).to(dtype)
    res = x.to(DEV).clone()
    out = norm.add_forward(d.to(DEV), res, dtype)
    want = rms_norm((x + d.float()).double(), w.double(), 1e-6)
    assert rel_err(out.float().cpu(), want) < (2e-6 if dtype == torch.float32 else 6e-3)
    assert torch.equal(res.cpu(), x + d.float())


@pytest.mark.parametrize("interleaved", [False, True])
def test_position_encoding_part(interleaved):
    from photon_infer_b200.parts.registry import create_part
    from plain.llama_plain import rope_apply, rope_inverse_frequencies
    scaling = TINY["tiny_b"]["config"]["rope_scaling"]
    pe = create_part("position_encoding", "rotary", {"head_dim": 32, "theta": 500000.0, "scaling": scaling,
                                                     "interleaved": interleaved})
    want_inv = rope_inverse_frequencies(32, 500000.0, scaling)
    assert torch.equal(pe.inv_freq_host, want_inv)            # both sides round float64 to float32 once
    pe.to_device(DEV)
    torch.manual_seed(1)
    q, k = torch.randn(9, 3, 32), torch.randn(9, 1, 32)
    positions = torch.tensor([0, 1, 5, 63, 64, 65, 200, 511, 3], dtype=torch.int32)
    qd, kd = q.to(DEV).clone(), k.to(DEV).clone()
    pe.apply(qd, kd, positions.to(DEV))
    assert rel_err(qd.cpu(), rope_apply(q, positions, want_inv, interleaved)) < 3e-6
    assert rel_err(kd.cpu(), rope_apply(k, positions, want_inv, interleaved)) < 3e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from photon_infer_b200.parts.registry import create_part
    from plain.llama_plain import feed_forward
    torch.manual_seed(2)
    ff = create_part("feed_forward", "swiglu", {"hidden_size": 72, "intermediate_size": 136})
    assert sorted(t.name for t in ff.tensor_specs()) == ["down_proj.weight", "gate_proj.weight", "up_proj.weight"]
    w = {"gate_proj.weight": 0.2 * torch.randn(136, 72), "up_proj.weight": 0.2 * torch.randn(136, 72),
         "down_proj.weight": 0.2 * torch.randn(72, 136)}
    w = {k: v.to(dtype) for k, v in w.items()}
    ff.load({k: v.to(DEV) for k, v in w.items()})
    h = torch.randn(7, 72).to(dtype)
    out = ff.forward(h.to(DEV), None)
    want = feed_forward(h.double(), w["gate_proj.weight"].double(), w["up_proj.weight"].double(), w["down_proj.weight"].double())
    assert rel_err(out.float().cpu(), want) < (3e-6 if dtype == torch.float32 else 1.2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 10])
def test_attention_part_two_requests_in_portions(dtype, window):
    """The mixer alone: two requests, each fed in two steps; against dense attention over the whole."""
    from photon_infer_b200.parts.base import LayerCache
    from photon_infer_b200.parts.registry import create_part
    from plain.llama_plain import causal_attention, linear, rope_apply, rope_inverse_frequencies
    torch.manual_seed(3)
    H, nq, nkv, d, ps = 40, 6, 2, 16, 4
    pe = create_part("position_encoding", "rotary", {"head_dim": d, "theta": 10000.0})
    pe.to_device(DEV)
    att = create_part("mixer", "sliding_attention" if window else "full_attention",
                      dict(hidden_size=H, n_q_heads=nq, n_kv_heads=nkv, head_dim=d, position_encoding=pe, window=window))
    spec = att.cache_spec()
    assert (spec.n_kv_heads, spec.head_dim, spec.window) == (nkv, d, window) and att.state_spec() is None
    w = {n: (0.3 * torch.randn(s.shape)).to(dtype) for n, s in ((t.name, t) for t in att.tensor_specs())}
    att.load({k: v.to(DEV) for k, v in w.items()})
    lens = [23, 14]
    hs = [torch.randn(L, H).to(dtype) for L in lens]
    kc = torch.full((64, nkv, ps, d), float("nan"), dtype=dtype, device=DEV)
    cache = LayerCache(group=0, k=kc, v=kc.clone())
    inv = rope_inverse_frequencies(d, 10000.0, None)
    want = []
    for L, h in zip(lens, hs):
        pos = torch.arange(L)
        q = rope_apply(linear(h.double(), w["q_proj.weight"].double()).view(L, nq, d), pos, inv, False)
        k = rope_apply(linear(h.double(), w["k_proj.weight"].double()).view(L, nkv, d), pos, inv, False)
        v = linear(h.double(), w["v_proj.weight"].double()).view(L, nkv, d)
        want.append(linear(causal_attention(q, k, v, window=window).reshape(L, -1), w["o_proj.weight"].double()))
    # step 1: 17 tokens of request 0, 5 of request 1; step 2: the rest
    cuts = [(17, 5), (6, 9)]
    got = [[], []]
    starts = [0, 0]
    for cut in cuts:
        ctx = _ctx(list(cut), list(starts), ps, dtype=dtype)
        h = torch.cat([hs[i][starts[i]:starts[i] + cut[i]] for i in range(2)]).to(DEV)
        out = att.forward(h, ctx, cache).float().cpu()
        got[0].append(out[:cut[0]]); got[1].append(out[cut[0]:])
        starts = [starts[i] + cut[i] for i in range(2)]
        assert ctx.error_flag.cpu().tolist()[0] == 0
    for i in range(2):
        assert rel_err(torch.cat(got[i]), want[i]) < (5e-6 if dtype == torch.float32 else 1.5e-2)


def _register_variant(name, order, kv_from):
    """A test architecture: the Llama parts with another run list."""
    from photon_infer_b200.config import LlamaConfig, register_architecture
    from photon_infer_b200.models.llama import build_llama_spec
    from photon_infer_b200.models.spec import RunEntry

    def build(cfg):
        spec = build_llama_spec(cfg)
        spec.run = [RunEntry(l, kv_from.get(i)) for i, l in enumerate(order)]
        return spec
    register_architecture(name, LlamaConfig, build, replace=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_list_names_a_layer_twice_and_shares_a_cache(tmp_path, dtype):
    """Order [0, 1, 1, 2, 0]: layer 1 runs twice (a cache for each run), the last entry runs layer 0
    again but reads the keys and values that entry 1 wrote."""
    from photon_infer_b200.config import EngineOptions
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    from photon_infer_b200.weights import write_random_model
    order, kv_from = [0, 1, 1, 2, 0], {4: 1}
    _register_variant("LoopedLlamaForTest", order, kv_from)
    t = TINY["tiny_b"]
    cfg = dict(t["config"], architectures=["LoopedLlamaForTest"])
    folder = str(tmp_path)
    write_random_model(folder, cfg, seed=5, init_std=0.05, norm_std=0.1)
    ids = random_ids(50, cfg["vocab_size"], seed=8)
    want = plain_logits(folder, ids, layer_order=order, kv_source=kv_from)
    runner = build_runner(folder, EngineOptions(dtype=dtype, block_size=8, max_cache_tokens=128, max_sequences=2))
    assert len(runner.cache.groups) == 1 and runner.cache.groups[0].entries == [0, 1, 2, 3]
    assert runner.cache.entry_shared == [False, False, False, False, True]
    runner.cache.add_request("a")
    got = []
    for lo, hi in ((0, 19), (19, 21), (21, 49), (49, 50)):
        got.append(runner.step([StepEntry("a", ids[lo:hi], list(range(hi - lo)))]).logits.cpu())
    runner.check_device_errors()
    assert rel_err(torch.cat(got), want) <= TOL[dtype]
    # it is a different function from the plain order
    assert rel_err(plain_logits(folder, ids), want) > 0.05


# --------------------------------------------------------------------------- a toy mixer with state

def _toy_parts():
    """A running-mean mixer: state s (float32 [H]) and a count per request; for each token
    s <- s + x, out = W (s / n).  Defined here with plain torch ops; the framework only sees the
    Mixer interface."""
    from photon_infer_b200.parts.base import Mixer, StateSpec, TensorSpec

    class RunningMeanMixer(Mixer):
        def __init__(self, hidden_size):
            self.h = hidden_size
            self.w = None

        def tensor_specs(self):
            return [TensorSpec("mix.weight", (self.h, self.h))]

        def load(self, tensors):
            self.w = tensors["mix.weight"]

        def cache_spec(self):
            return None

        def state_spec(self):
            return StateSpec((self.h + 1,), torch.float32)       # the sum and the count

        def forward(self, h, ctx, cache):
            out = torch.empty_like(h)
            slots = ctx.state_slots.tolist()
            cu = ctx.cu_tokens.tolist()
            for s, slot in enumerate(slots):
                x = h[cu[s]:cu[s + 1]].float()
                st = cache.state[slot]
                sums = st[: self.h] + torch.cumsum(x, 0)
                counts = st[self.h] + torch.arange(1, x.shape[0] + 1, device=h.device, dtype=torch.float32)
                out[cu[s]:cu[s + 1]] = ((sums / counts[:, None]).to(h.dtype) @ self.w.t())
                st[: self.h] = sums[-1]
                st[self.h] = counts[-1]
            return out

    return RunningMeanMixer


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from photon_infer_b200.config import EngineOptions, LlamaConfig, register_architecture
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    from photon_infer_b200.models.llama import build_llama_spec
    from photon_infer_b200.models.spec import PartSpec
    from photon_infer_b200.parts.registry import register_mixer
    from photon_infer_b200.weights import write_random_model
    from plain.llama_plain import PlainLlama, feed_forward, linear, rms_norm
    from safetensors.torch import load_file

    register_mixer("running_mean_for_test", _toy_parts(), replace=True)

    def build(cfg):
        spec = build_llama_spec(cfg)
        for i, layer in enumerate(spec.layers):
            if cfg.layer_types[i] == "running_mean_for_test":
                layer.mixer = PartSpec("running_mean_for_test", {"hidden_size": cfg.hidden_size}, "toy.")
        return spec
    register_architecture("ToyStateModelForTest", LlamaConfig, build, replace=True)

    cfg = dict(TINY["tiny_a"]["config"], architectures=["ToyStateModelForTest"], num_hidden_layers=3,
               layer_types=["full_attention", "running_mean_for_test", "full_attention"])
    folder = str(tmp_path)
    names = write_random_model(folder, cfg, seed=11, init_std=0.05, norm_std=0.1)
    assert "model.layers.1.toy.mix.weight" in names and "model.layers.1.self_attn.q_proj.weight" not in names
    runner = build_runner(folder, EngineOptions(dtype="float32", block_size=16, max_cache_tokens=256, max_sequences=3))
    assert runner.cache.states.specs.keys() == {1} and len(runner.cache.groups) == 1
    assert runner.cache.groups[0].entries == [0, 2]

    # plain: the same three layers written out
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    base = PlainLlama(dict(cfg, layer_types=None), w)

    def plain(ids):
        x = w["model.embed_tokens.weight"][torch.tensor(ids)]
        pos = torch.arange(len(ids))
        for l in range(3):
            p = f"model.layers.{l}."
            h = rms_norm(x, w[p + "input_layernorm.weight"], base.eps)
            if l == 1:
                mean = torch.cumsum(h, 0) / torch.arange(1, len(ids) + 1)[:, None]
                x = x + linear(mean, w[p + "toy.mix.weight"])
            else:
                x = x + base._attention_part(l, h, pos, None)[0]
            h2 = rms_norm(x, w[p + "post_attention_layernorm.weight"], base.eps)
            x = x + feed_forward(h2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        return linear(rms_norm(x, w["model.norm.weight"], base.eps), w["model.embed_tokens.weight"])

    a, b = random_ids(40, 256, seed=1), random_ids(27, 256, seed=2)
    runner.cache.add_request("a"); runner.cache.add_request("b")
    got_a, got_b = [], []
    r = runner.step([StepEntry("a", a[:25], list(range(25))), StepEntry("b", b[:3], [0, 1, 2])])
    got_a.append(r.logits[:25].cpu()); got_b.append(r.logits[25:].cpu())
    r = runner.step([StepEntry("b", b[3:], list(range(24))), StepEntry("a", a[25:26], [0])])
    got_b.append(r.logits[:24].cpu()); got_a.append(r.logits[24:].cpu())
    r = runner.step([StepEntry("a", a[26:], list(range(14)))])
    got_a.append(r.logits.cpu())
    assert rel_err(torch.cat(got_a), plain(a)) < 2e-5
    assert rel_err(torch.cat(got_b), plain(b)) < 2e-5
    # a slot handed out again starts from zero
    runner.cache.free_request("a")
    runner.cache.add_request("c")
    r = runner.step([StepEntry("c", b, list(range(27)))])
    assert rel_err(r.logits.cpu(), plain(b)) < 2e-5


# --------------------------------------------------------------------------- a toy routed feed-forward and a toy position encoding

def _toy_routed_ff():
    """Top-1 of E small experts: router logits in 32-bit, probability of the chosen expert times
    W2_e relu(W1_e h).  Plain torch ops; the framework only sees the FeedForward interface."""
    from photon_infer_b200.parts.base import FeedForward, TensorSpec

    class Top1Experts(FeedForward):
        def __init__(self, hidden_size, inner_size, experts):
            self.h, self.i, self.e = hidden_size, inner_size, experts
            self.router = self.w1 = self.w2 = None

        def tensor_specs(self):
            return [TensorSpec("router.weight", (self.e, self.h)), TensorSpec("w1.weight", (self.e * self.i, self.h)),
                    TensorSpec("w2.weight", (self.e * self.h, self.i))]

        def load(self, tensors):
            self.router = tensors["router.weight"]
            self.w1 = tensors["w1.weight"].view(self.e, self.i, self.h)
            self.w2 = tensors["w2.weight"].view(self.e, self.h, self.i)

        def forward(self, h, ctx):
            logits = h.float() @ self.router.float().t()                      # 32-bit router
            prob = torch.softmax(logits, dim=-1)
            top = prob.argmax(dim=-1)
            out = torch.zeros_like(h)
            for e in range(self.e):
                rows = (top == e).nonzero().flatten()
                if rows.numel():
                    x = h[rows]
                    y = torch.relu(x @ self.w1[e].t()) @ self.w2[e].t()
                    out[rows] = (y.float() * prob[rows, e][:, None]).to(h.dtype)
            return out

    return Top1Experts


def _toy_position_encoding():
    """Queries and keys shrink with their position: x <- x / (1 + rate * pos).  No tensors."""
    from photon_infer_b200.parts.base import PositionEncoding

    class DecayEncoding(PositionEncoding):
        def __init__(self, rate):
            self.rate = float(rate)

        def apply(self, q, k, positions):
            s = 1.0 / (1.0 + self.rate * positions.float())
            q.mul_(s[:, None, None].to(q.dtype))
            if k is not None:
                k.mul_(s[:, None, None].to(k.dtype))

    return DecayEncoding


def test_toy_routed_feed_forward_and_position_encoding_without_touching_the_framework(tmp_path):
    """An architecture whose layers use the framework's paged attention with a position encoding defined
    here, and a routed feed-forward defined here: registered, given random weights, loaded and stepped in
    portions beside another request, against the same model written out with the plain functions."""
    from photon_infer_b200.config import EngineOptions, LlamaConfig, register_architecture
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    from photon_infer_b200.models.llama import build_llama_spec
    from photon_infer_b200.models.spec import PartSpec
    from photon_infer_b200.parts.registry import register_feed_forward, register_position_encoding
    from photon_infer_b200.weights import write_random_model
    from plain.llama_plain import causal_attention, feed_forward, linear, rms_norm
    from safetensors.torch import load_file

    E, INNER, RATE = 3, 40, 0.03
    register_feed_forward("top1_experts_for_test", _toy_routed_ff(), replace=True)
    register_position_encoding("decay_for_test", _toy_position_encoding(), replace=True)

    def build(cfg):
        spec = build_llama_spec(cfg)
        spec.position_encodings = {"decay": PartSpec("decay_for_test", {"rate": RATE})}
        for i, layer in enumerate(spec.layers):
            layer.mixer.params["position_encoding"] = "decay"
            if i == 1:                                                         # the middle layer routes
                layer.feed_forward = PartSpec("top1_experts_for_test",
                                              {"hidden_size": cfg.hidden_size, "inner_size": INNER, "experts": E}, "moe.")
        return spec
    register_architecture("ToyRoutedModelForTest", LlamaConfig, build, replace=True)

    cfg = dict(TINY["tiny_b"]["config"], architectures=["ToyRoutedModelForTest"], num_hidden_layers=3)
    folder = str(tmp_path)
    names = write_random_model(folder, cfg, seed=12, init_std=0.08, norm_std=0.1)
    assert "model.layers.1.moe.router.weight" in names and "model.layers.1.mlp.gate_proj.weight" not in names
    assert "model.layers.0.mlp.gate_proj.weight" in names
    runner = build_runner(folder, EngineOptions(dtype="float32", block_size=8, max_cache_tokens=256, max_sequences=3))

    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    c = LlamaConfig.from_dict(cfg)
    n_q, n_kv, d = c.num_attention_heads, c.num_key_value_heads, c.head_dim

    def plain(ids):
        T = len(ids)
        x = w["model.embed_tokens.weight"][torch.tensor(ids)]
        s = (1.0 / (1.0 + RATE * torch.arange(T).float()))[:, None, None]
        for l in range(3):
            p = f"model.layers.{l}."
            h = rms_norm(x, w[p + "input_layernorm.weight"], c.rms_norm_eps)
            q = linear(h, w[p + "self_attn.q_proj.weight"]).view(T, n_q, d) * s
            k = linear(h, w[p + "self_attn.k_proj.weight"]).view(T, n_kv, d) * s
            v = linear(h, w[p + "self_attn.v_proj.weight"]).view(T, n_kv, d)
            x = x + linear(causal_attention(q, k, v).reshape(T, -1), w[p + "self_attn.o_proj.weight"])
            h2 = rms_norm(x, w[p + "post_attention_layernorm.weight"], c.rms_norm_eps)
            if l == 1:
                prob = torch.softmax(h2 @ w[p + "moe.router.weight"].t(), dim=-1)
                top = prob.argmax(dim=-1)
                w1 = w[p + "moe.w1.weight"].view(E, INNER, -1)
                w2 = w[p + "moe.w2.weight"].view(E, -1, INNER)
                y = torch.stack([torch.relu(h2[t] @ w1[top[t]].t()) @ w2[top[t]].t() * prob[t, top[t]] for t in range(T)])
                x = x + y
            else:
                x = x + feed_forward(h2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        return linear(rms_norm(x, w["model.norm.weight"], c.rms_norm_eps), w["lm_head.weight"])

    vocab = cfg["vocab_size"]
    a, b = random_ids(37, vocab, seed=3), random_ids(21, vocab, seed=4)
    runner.cache.add_request("a"); runner.cache.add_request("b")
    got_a, got_b = [], []
    r = runner.step([StepEntry("a", a[:20], list(range(20))), StepEntry("b", b[:2], [0, 1])])
    got_a.append(r.logits[:20].cpu()); got_b.append(r.logits[20:].cpu())
    r = runner.step([StepEntry("b", b[2:], list(range(19))), StepEntry("a", a[20:21], [0])])
    got_b.append(r.logits[:19].cpu()); got_a.append(r.logits[19:].cpu())
    r = runner.step([StepEntry("a", a[21:], list(range(16)))])
    got_a.append(r.logits.cpu())
    assert rel_err(torch.cat(got_a), plain(a)) < 2e-5
    assert rel_err(torch.cat(got_b), plain(b)) < 2e-5
