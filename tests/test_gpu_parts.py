"""Each part alone against its plain counterpart, and the framework's openness: a toy mixer
with state of its own, a toy architecture whose layers differ, whose schedule names a
layer twice and lets an entry read another entry's cache - all defined here, registered
and stepped without touching the package."""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import cpp_minilamma_b200 as ml
import plain_llama as pl
from cpp_minilamma_b200 import StepEntry
from cpp_minilamma_b200.cache import SequenceCache
from cpp_minilamma_b200.config.base import ModelConfig, take_int
from cpp_minilamma_b200.engine.step import make_step_state
from cpp_minilamma_b200.parts import (BuildContext, CacheNeed, LayerSpec, Mixer, ModelSpec, PartSpec, ScheduleEntry,
                                      StateNeed, WeightSpec, WeightStore, build_part, register_part)
from cpp_minilamma_b200.parts.rope import inverse_frequencies
from helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def close(got, ref, dtype, what=""):
    """float32: element-wise 2e-5 / 2e-6.  bfloat16: the rule of helpers.assert_close (largest
    error <= 2%, mean error <= 0.4% of the largest |reference|), fixed before the first run."""
    if dtype == torch.float32:
        np.testing.assert_allclose(got, ref, rtol=2e-5, atol=2e-6, err_msg=what)
    else:
        assert_close(got, ref, "bfloat16", what)


def as64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def make_state(slots, starts, lens, tokens=None, parts=()):
    """A StepState for sequences in `slots` that bring `lens` tokens from positions `starts`, with the index
    arrays that `parts` prepare for themselves."""
    return make_step_state(DEV, slots, starts, lens, tokens=tokens, parts=parts)


def ctx_for(dtype, hidden, max_positions=512):
    return BuildContext(hidden, dtype, DEV, max_positions)


def bind(part, dtype, seed):
    tensors = {}
    for i, spec in enumerate(part.weight_specs()):
        t = rnd(spec.shape, seed + i, 0.05)
        if spec.init == "norm":
            t = 1 + t
        tensors[spec.name] = t.to(torch.float32 if spec.kind == "vector" else dtype).to(DEV)
    host = {k: as64(v) for k, v in tensors.items()}
    part.bind(WeightStore(tensors))
    return host


# ------------------------------------------------------------------------------------ #
def test_rotary_tables_match_the_plain_frequencies():
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 32}
    for head_dim, theta, sc in [(16, 10000.0, None), (32, 500000.0, scaling), (128, 500000.0,
                                {**scaling, "original_max_position_embeddings": 8192})]:
        ours = inverse_frequencies(head_dim, theta, sc)
        plain = pl.rope_inverse_frequencies(head_dim, theta, sc)
        np.testing.assert_allclose(ours, plain, rtol=1e-14)
        if sc:  # the three regimes are all present for the small original length
            ratio = plain / pl.rope_inverse_frequencies(head_dim, theta, None)
            assert ratio.max() == 1.0 and np.isclose(ratio.min(), 1 / 8)
        part = build_part("position_encoding", PartSpec("rotary", {"head_dim": head_dim, "theta": theta,
                                                                    "scaling": sc, "interleaved": False}),
                          ctx_for(torch.float32, 64, 300))
        cos, sin = part.tables()
        ang = np.arange(300)[:, None] * plain[None, :]
        np.testing.assert_allclose(cos.cpu().numpy(), np.cos(ang), atol=1e-7)
        np.testing.assert_allclose(sin.cpu().numpy(), np.sin(ang), atol=1e-7)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    part = build_part("norm", PartSpec("rms_norm", {"width": 100, "eps": 3e-4, "name": "n.weight"}), ctx_for(dtype, 100))
    host = bind(part, dtype, 1)
    x = rnd((9, 100), 2).to(DEV)
    delta = rnd((9, 100), 3).to(dtype).to(DEV)
    expect_x = as64(x) + as64(delta)
    out = part.forward(make_state([0], [0], [9]), x, delta)
    close(as64(out), pl.rms_norm(expect_x, host["n.weight"], 3e-4), dtype)
    np.testing.assert_allclose(as64(x), expect_x, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [250, 176])
def test_feed_forward_part(dtype, inter):
    names = {p: f"mlp.{p}_proj" for p in ("gate", "up", "down")}
    part = build_part("feed_forward", PartSpec("swiglu", {"intermediate": inter, "names": names}), ctx_for(dtype, 100))
    host = bind(part, dtype, 10)
    assert part.block == (8 if inter % 8 == 0 else 0)
    h = rnd((13, 100), 4).to(dtype).to(DEV)
    out = part.forward(make_state([0], [0], [13]), h)
    round_ = pl.round_bf16 if dtype == torch.bfloat16 else (lambda v: v)
    ref = pl.feed_forward(as64(h), host["mlp.gate_proj.weight"], host["mlp.up_proj.weight"],
                          host["mlp.down_proj.weight"], round_)
    close(as64(out), ref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    ctx = ctx_for(dtype, 100)
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab": 333, "name": "e.weight"}), ctx)
    head = build_part("lm_head", PartSpec("linear_head", {"vocab": 333, "name": "h.weight", "tied_to": "e.weight"}), ctx)
    assert head.weight_specs() == []
    table = rnd((333, 100), 5, 0.05).to(dtype).to(DEV)
    store = WeightStore({"e.weight": table})
    emb.bind(store)
    head.bind(store)
    state = make_state([0], [0], [4], tokens=[332, 0, 7, 7])
    x = emb.forward(state, state.tokens)
    np.testing.assert_array_equal(x.cpu().numpy(), table.float().cpu().numpy()[[332, 0, 7, 7]])
    h = rnd((4, 100), 6).to(dtype).to(DEV)
    logits = head.forward(state, h)
    assert logits.dtype == torch.float32
    np.testing.assert_allclose(as64(logits), as64(h) @ as64(table).T, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 40])
def test_attention_part_prefill_then_decode(dtype, window):
    hidden, hq, hk, d = 100, 6, 2, 32
    position = PartSpec("rotary", {"head_dim": d, "theta": 1000.0, "scaling": None, "interleaved": True})
    names = {p: f"a.{p}_proj" for p in "qkvo"}
    ctx = ctx_for(dtype, hidden)
    part = build_part("mixer", PartSpec("attention", {
        "n_heads": hq, "n_kv_heads": hk, "head_dim": d, "window": window, "position": position,
        "qkv_bias": True, "o_bias": True, "names": names}), ctx)
    host = bind(part, dtype, 20)
    cache = SequenceCache([(0, None, part.cache_need())], 64 * 8, 4, 512, dtype, DEV)
    slots = cache.acquire(2)
    lens = [70, 5]
    h = rnd((sum(lens) + 2, hidden), 7).to(dtype)
    # prompts of 70 and 5 tokens in one step, then one token each
    cache.reserve(list(zip(slots, lens)))
    cache.flush()
    out1 = part.forward(make_state(slots, [0, 0], lens, parts=[part]), h[:75].to(DEV), cache.view(0)).clone()
    cache.reserve([(s, 1) for s in slots])
    cache.flush()
    out2 = part.forward(make_state(slots, lens, [1, 1], parts=[part]), h[75:].to(DEV), cache.view(0)).clone()
    cfg = {"num_attention_heads": hq, "num_key_value_heads": hk, "head_dim": d, "hidden_size": hidden,
           "rope_interleaved": True, "sliding_window": window or None}
    weights = {f"self_attn.{p}_proj.{kind}": host[f"a.{p}_proj.{kind}"] for p in "qkvo" for kind in ("weight", "bias")}
    inv = pl.rope_inverse_frequencies(d, 1000.0)
    round_ = pl.round_bf16 if dtype == torch.bfloat16 else (lambda v: v)
    seq0 = np.concatenate([as64(h[:70]), as64(h[75:76])])
    seq1 = np.concatenate([as64(h[70:75]), as64(h[76:77])])
    ref0 = pl.attention_block(seq0, np.arange(71), weights, "", cfg, inv, round_)
    ref1 = pl.attention_block(seq1, np.arange(6), weights, "", cfg, inv, round_)
    close(as64(out1[:70]), ref0[:70], dtype)
    close(as64(out1[70:]), ref1[:5], dtype)
    close(as64(out2[0]), ref0[70], dtype)
    close(as64(out2[1]), ref1[5], dtype)
    # what the cache holds is the rotated key and the value of every position
    k, v = cache.read_kv(0, slots[1])
    x = round_(seq1 @ weights["self_attn.k_proj.weight"].T) + weights["self_attn.k_proj.bias"]
    k_ref = pl.apply_rope(x.reshape(6, hk, d), np.arange(6), inv, True)
    close(as64(k), k_ref, dtype)


# ------------------------------------------------------------------------------------ #
# a toy mixer with state of its own and a toy architecture, defined here                #
# ------------------------------------------------------------------------------------ #
class RunningMeanMixer(Mixer):
    """out_t = W . mean(h_0 .. h_t): keeps (sum, count) per sequence as fixed-size state."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.name = params["name"]
        self.weight = None

    def weight_specs(self):
        D = self.ctx.hidden_size
        return [WeightSpec(self.name, (D, D))]

    def bind(self, store):
        self.weight = store.take(self.name)

    def cache_need(self):
        D = self.ctx.hidden_size
        return CacheNeed(state=StateNeed((("sum", (D,)), ("count", (1,)))))

    def forward(self, step, h, cache):
        out = step.ws.buffer("toy.out", tuple(h.shape), h.dtype)
        at = 0
        for slot, n in zip(step.shape.slots, step.shape.lens):  # tokens of a sequence in order
            rows = h[at:at + n].float()
            sums = cache.state["sum"][slot] + torch.cumsum(rows, dim=0)
            counts = cache.state["count"][slot] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)[:, None]
            mean = (sums / counts).to(self.weight.dtype)
            out[at:at + n] = (mean @ self.weight.t()).to(h.dtype)
            cache.state["sum"][slot] = sums[-1]
            cache.state["count"][slot] = counts[-1]
            at += n
        return out


@dataclass
class ToyConfig(ModelConfig):
    vocab_size: int = 0
    hidden_size: int = 0
    torch_dtype: str = "float32"

    @classmethod
    def from_dict(cls, raw):
        return cls(vocab_size=take_int(raw, "vocab_size"), hidden_size=take_int(raw, "hidden_size"),
                   torch_dtype=raw.get("torch_dtype", "float32"))

    def validate(self):
        pass

    def to_dict(self):
        return {"architectures": ["ToyStateLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "torch_dtype": self.torch_dtype}


HQ, HK, HD, INTER = 4, 2, 16, 72


def toy_builder(cfg):
    D = cfg.hidden_size

    def norm(name):
        return PartSpec("rms_norm", {"width": D, "eps": 1e-5, "name": name})

    def ffn(i):
        return PartSpec("swiglu", {"intermediate": INTER, "names": {p: f"l{i}.{p}" for p in ("gate", "up", "down")}})

    def attention(i, reads_only=False):
        return PartSpec("attention", {
            "n_heads": HQ, "n_kv_heads": HK, "head_dim": HD, "window": 0, "reads_cache_only": reads_only,
            "position": PartSpec("rotary", {"head_dim": HD, "theta": 100.0, "scaling": None, "interleaved": False}),
            "names": {p: f"l{i}.{p}" for p in "qkvo"}})

    def layer(i, mixer):
        return LayerSpec(PartSpec("pre_norm"), mixer, ffn(i), {"input": norm(f"l{i}.n1"), "post_mixer": norm(f"l{i}.n2")})

    layers = [layer(0, attention(0)), layer(1, PartSpec("running_mean", {"name": "l1.mix"})),
              layer(2, attention(2, reads_only=True))]
    # layer 0, the state mixer, layer 0 again (a cache of its own), then a layer that reads entry 0's cache,
    # then the state mixer again (a state of its own)
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2, cache_of=0), ScheduleEntry(1)]
    return ModelSpec(hidden_size=D, vocab_size=cfg.vocab_size, max_positions=256,
                     embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "name": "emb"}),
                     layers=layers, schedule=schedule, final_norm=norm("final"),
                     lm_head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "name": "head", "tied_to": None}))


def toy_plain(weights, tokens, D):
    """Whole-sequence forward of the toy model in NumPy, float64."""
    T = len(tokens)
    pos = np.arange(T)
    inv = pl.rope_inverse_frequencies(HD, 100.0)
    x = pl.embedding(weights["emb"], tokens)
    kv = {}

    def attention(i, h, entry, source=None):
        q = pl.apply_rope(pl.linear(h, weights[f"l{i}.q.weight"]).reshape(T, HQ, HD), pos, inv, False)
        if source is None:
            k = pl.apply_rope(pl.linear(h, weights[f"l{i}.k.weight"]).reshape(T, HK, HD), pos, inv, False)
            v = pl.linear(h, weights[f"l{i}.v.weight"]).reshape(T, HK, HD)
            kv[entry] = (k, v)
        else:
            k, v = kv[source]
        return pl.linear(pl.causal_attention(q, k, v).reshape(T, HQ * HD), weights[f"l{i}.o.weight"])

    def running_mean(h):
        mean = np.cumsum(h, axis=0) / np.arange(1, T + 1)[:, None]
        return pl.linear(mean, weights["l1.mix"])

    for entry, (i, source) in enumerate([(0, None), (1, None), (0, None), (2, 0), (1, None)]):
        h = pl.rms_norm(x, weights[f"l{i}.n1"], 1e-5)
        x = x + (running_mean(h) if i == 1 else attention(i, h, entry, source))
        h = pl.rms_norm(x, weights[f"l{i}.n2"], 1e-5)
        x = x + pl.feed_forward(h, weights[f"l{i}.gate.weight"], weights[f"l{i}.up.weight"], weights[f"l{i}.down.weight"])
    return pl.linear(pl.rms_norm(x, weights["final"], 1e-5), weights["head"])


def test_toy_architecture_with_a_state_mixer(tmp_path):
    register_part("mixer", "running_mean", RunningMeanMixer)
    ml.register_architecture("ToyStateLM", ToyConfig, toy_builder)
    cfg = ml.config_from_dict({"architectures": ["ToyStateLM"], "vocab_size": 97, "hidden_size": 40})
    folder = ml.write_random_model(cfg, tmp_path, seed=5)
    _, weights = pl.read_model_folder(folder)
    llm = ml.load(folder, dtype="float32", max_tokens=64 * 12, max_seqs=3)
    assert len(llm.engine.cache.groups) == 1 and llm.engine.cache.groups[0].entries == [0, 2]
    assert sorted(llm.engine.cache.state) == [1, 4]
    rng = np.random.RandomState(0)
    requests = [[int(t) for t in rng.randint(0, 97, size=n)] for n in (70, 3, 20, 9)]
    refs = [toy_plain(weights, r, 40) for r in requests]
    # whole
    for r, ref in zip(requests, refs):
        slot, = llm.engine.acquire(1)
        got = llm.engine.step([StepEntry(slot, r, list(range(len(r))))])
        llm.engine.release(slot)
        assert_close(got.cpu().numpy(), ref, "float32", "toy whole")
    # batches of unequal lengths, prompts then one token each, slots reused by the second batch
    for group in ([0, 1, 2], [3, 1]):
        slots = dict(zip(group, llm.engine.acquire(len(group))))
        fed = {g: max(1, len(requests[g]) // 2) for g in group}
        out = llm.engine.step([StepEntry(slots[g], requests[g][:fed[g]], [fed[g] - 1]) for g in group])
        for j, g in enumerate(group):
            assert_close(out[j].cpu().numpy(), refs[g][fed[g] - 1], "float32", "toy prompt")
        live = list(group)
        while live:
            live = [g for g in live if fed[g] < len(requests[g])]
            if not live:
                break
            out = llm.engine.step([StepEntry(slots[g], [requests[g][fed[g]]], [0]) for g in live])
            for j, g in enumerate(live):
                assert_close(out[j].cpu().numpy(), refs[g][fed[g]], "float32", f"toy decode request {g}")
                fed[g] += 1
        for g in group:
            llm.engine.release(slots[g])
    llm.engine.cache.check()
    # greedy generation runs through the same loop
    assert len(llm.generate([requests[1]], max_new_tokens=5)[0]) == 5


# ------------------------------------------------------------------------------------ #
# a second toy architecture: windowed attention without position encoding next to full  #
# attention with rotary encoding, a feed-forward with routing, another position encoding #
# ------------------------------------------------------------------------------------ #
from cpp_minilamma_b200.parts import FeedForward, PositionEncoding  # noqa: E402


class Top1Experts(FeedForward):
    """Routed feed-forward: router logits in float32, the best expert's SwiGLU output scaled by
    its softmax weight.  Written with torch ops: the interface is what is under test."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.n, self.inter, self.prefix = params["experts"], params["intermediate"], params["prefix"]

    def weight_specs(self):
        D = self.ctx.hidden_size
        specs = [WeightSpec(self.prefix + "router", (self.n, D))]
        for e in range(self.n):
            specs += [WeightSpec(f"{self.prefix}e{e}.gate", (self.inter, D)), WeightSpec(f"{self.prefix}e{e}.up", (self.inter, D)),
                      WeightSpec(f"{self.prefix}e{e}.down", (D, self.inter))]
        return specs

    def bind(self, store):
        self.router = store.take(self.prefix + "router").float()
        self.experts = [(store.take(f"{self.prefix}e{e}.gate").float(), store.take(f"{self.prefix}e{e}.up").float(),
                         store.take(f"{self.prefix}e{e}.down").float()) for e in range(self.n)]

    def forward(self, step, h):
        x = h.float()
        probs = torch.softmax(x @ self.router.t(), dim=-1)
        best = probs.argmax(dim=-1)
        out = torch.zeros_like(x)
        for e, (g, u, d) in enumerate(self.experts):
            y = (torch.nn.functional.silu(x @ g.t()) * (x @ u.t())) @ d.t()
            out += torch.where((best == e)[:, None], y * probs[:, e:e + 1], torch.zeros_like(y))
        return out.to(h.dtype)


class HalfSpeedRotary(PositionEncoding):
    """Another position encoding: rotary tables whose angles advance half a step per position."""

    interleaved = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        freqs = pl.rope_inverse_frequencies(params["head_dim"], params["theta"]) * 0.5
        ang = np.arange(ctx.max_positions)[:, None] * freqs[None, :]
        self.cos = torch.tensor(np.cos(ang), dtype=torch.float32, device=ctx.device)
        self.sin = torch.tensor(np.sin(ang), dtype=torch.float32, device=ctx.device)

    def tables(self):
        return self.cos, self.sin


@dataclass
class MixConfig(ToyConfig):
    def to_dict(self):
        return {**super().to_dict(), "architectures": ["ToyMixLM"]}


WINDOW = 70


def mix_builder(cfg):
    D = cfg.hidden_size

    def norm(name):
        return PartSpec("rms_norm", {"width": D, "eps": 1e-6, "name": name})

    def attention(i, window, position):
        return PartSpec("attention", {"n_heads": HQ, "n_kv_heads": HK, "head_dim": HD, "window": window,
                                      "position": position, "names": {p: f"l{i}.{p}" for p in "qkvo"}})

    layers = [
        LayerSpec(PartSpec("pre_norm"), attention(0, 0, PartSpec("half_speed_rotary", {"head_dim": HD, "theta": 50.0})),
                  PartSpec("top1_experts", {"experts": 3, "intermediate": 24, "prefix": "l0.moe."}),
                  {"input": norm("l0.n1"), "post_mixer": norm("l0.n2")}),
        LayerSpec(PartSpec("pre_norm"), attention(1, WINDOW, PartSpec("none")),
                  PartSpec("swiglu", {"intermediate": INTER, "names": {p: f"l1.{p}" for p in ("gate", "up", "down")}}),
                  {"input": norm("l1.n1"), "post_mixer": norm("l1.n2")}),
    ]
    return ModelSpec(hidden_size=D, vocab_size=cfg.vocab_size, max_positions=512,
                     embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "name": "emb"}),
                     layers=layers, schedule=[ScheduleEntry(0), ScheduleEntry(1)], final_norm=norm("final"),
                     lm_head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "name": "head", "tied_to": "emb"}))


def mix_plain(weights, tokens):
    T = len(tokens)
    pos = np.arange(T)
    x = pl.embedding(weights["emb"], tokens)
    # layer 0: full attention, half-speed interleaved rotary, routed feed-forward
    h = pl.rms_norm(x, weights["l0.n1"], 1e-6)
    inv = pl.rope_inverse_frequencies(HD, 50.0) * 0.5
    q = pl.apply_rope(pl.linear(h, weights["l0.q.weight"]).reshape(T, HQ, HD), pos, inv, True)
    k = pl.apply_rope(pl.linear(h, weights["l0.k.weight"]).reshape(T, HK, HD), pos, inv, True)
    v = pl.linear(h, weights["l0.v.weight"]).reshape(T, HK, HD)
    x = x + pl.linear(pl.causal_attention(q, k, v).reshape(T, HQ * HD), weights["l0.o.weight"])
    h = pl.rms_norm(x, weights["l0.n2"], 1e-6)
    logits = pl.linear(h, weights["l0.moe.router"])
    probs = np.exp(logits - logits.max(axis=-1, keepdims=True))
    probs /= probs.sum(axis=-1, keepdims=True)
    best = probs.argmax(axis=-1)
    moe = np.zeros_like(x)
    for t in range(T):
        e = int(best[t])
        moe[t] = probs[t, e] * pl.feed_forward(h[t:t + 1], weights[f"l0.moe.e{e}.gate"], weights[f"l0.moe.e{e}.up"],
                                               weights[f"l0.moe.e{e}.down"])[0]
    x = x + moe
    # layer 1: the last WINDOW keys only, no position encoding, dense feed-forward
    h = pl.rms_norm(x, weights["l1.n1"], 1e-6)
    q = pl.linear(h, weights["l1.q.weight"]).reshape(T, HQ, HD)
    k = pl.linear(h, weights["l1.k.weight"]).reshape(T, HK, HD)
    v = pl.linear(h, weights["l1.v.weight"]).reshape(T, HK, HD)
    x = x + pl.linear(pl.causal_attention(q, k, v, window=WINDOW).reshape(T, HQ * HD), weights["l1.o.weight"])
    h = pl.rms_norm(x, weights["l1.n2"], 1e-6)
    x = x + pl.feed_forward(h, weights["l1.gate.weight"], weights["l1.up.weight"], weights["l1.down.weight"])
    return pl.linear(pl.rms_norm(x, weights["final"], 1e-6), weights["emb"])


def test_toy_architecture_with_window_group_routing_and_other_encoding(tmp_path):
    register_part("feed_forward", "top1_experts", Top1Experts)
    register_part("position_encoding", "half_speed_rotary", HalfSpeedRotary)
    ml.register_architecture("ToyMixLM", MixConfig, mix_builder)
    cfg = ml.config_from_dict({"architectures": ["ToyMixLM"], "vocab_size": 61, "hidden_size": 48})
    folder = ml.write_random_model(cfg, tmp_path, seed=9, matrix_std=0.08)
    _, weights = pl.read_model_folder(folder)
    llm = ml.load(folder, dtype="float32", max_tokens=64 * 10, max_seqs=2)
    cache = llm.engine.cache
    # the two attention layers differ in their need: storage and block table of their own
    assert len(cache.groups) == 2 and {g.need.window for g in cache.groups} == {0, WINDOW}
    rng = np.random.RandomState(1)
    tokens = [int(t) for t in rng.randint(0, 61, size=300)]
    ref = mix_plain(weights, tokens)
    slot, = llm.engine.acquire(1)
    rows = [llm.engine.step([StepEntry(slot, tokens[:150], list(range(150)))]).cpu().numpy()]
    for t in range(150, 300):   # decoding far beyond the window: the windowed group gives pages back
        rows.append(llm.engine.step([StepEntry(slot, [tokens[t]], [0])]).cpu().numpy())
    assert_close(np.concatenate(rows), ref, "float32", "toy mix: prompt then decode")
    full, windowed = sorted(cache.groups, key=lambda g: g.need.window)
    assert sum(p is not None for p in full.pages[slot]) == 5           # 300 tokens: 5 pages
    assert sum(p is not None for p in windowed.pages[slot]) <= 3       # about WINDOW tokens stay
    cache.check()
    llm.engine.release(slot)
    # whole, in one step, next to a second sequence
    a, b = llm.engine.acquire(2)
    out = llm.engine.step([StepEntry(a, tokens, list(range(300))), StepEntry(b, tokens[:7], [6])]).cpu().numpy()
    assert_close(out[:300], ref, "float32", "toy mix: whole")
    assert_close(out[300], mix_plain(weights, tokens[:7])[6], "float32", "toy mix: short neighbour")
    llm.engine.release(a)
    llm.engine.release(b)
    # the same prompt cut into chunks of 64 tokens inside the engine: the window's edge (70 keys back) falls
    # inside every portion but the first, and the windowed group hands pages back between the portions
    chunked = ml.load(folder, dtype="float32", max_tokens=64 * 10, max_seqs=2, max_step_tokens=64)
    slot, = chunked.engine.acquire(1)
    out = chunked.engine.step([StepEntry(slot, tokens, list(range(300)))]).cpu().numpy()
    assert_close(out, ref, "float32", "toy mix: whole, in chunks of 64")
    chunked.engine.cache.check()


# ------------------------------------------------------------------------------------ #
# a third toy architecture: a mixer whose kernels want an index array of their own      #
# ------------------------------------------------------------------------------------ #
class BucketGainMixer(Mixer):
    """out_t = gain[min(pos_t // 16, 3)] * (W . h_t): the bucket of every token is an index array that the part
    prepares on the host for each step and finds on the device in `step.meta`.  `forward` enqueues device work
    at fixed addresses only, so decode steps are captured and replayed, and the array is refreshed inside the
    captured step's buffer.  It also asks for a launch parameter that is fixed at capture."""

    capturable = True
    KEY = ("toy.bucket", 16)
    prepared = 0

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.name = params["name"]
        self.weight = self.gain = None

    def weight_specs(self):
        D = self.ctx.hidden_size
        return [WeightSpec(self.name + ".w", (D, D)), WeightSpec(self.name + ".gain", (4,), kind="vector", init="norm")]

    def bind(self, store):
        self.weight = store.take(self.name + ".w")
        self.gain = store.take(self.name + ".gain")

    def step_metadata_key(self):
        return self.KEY

    def prepare_step(self, shape):
        BucketGainMixer.prepared += 1
        return {"bucket": [min(pos // 16, 3) for start, n in zip(shape.starts, shape.lens) for pos in range(start, start + n)]}

    def capture_parameters(self, batch, max_positions):
        return {"batch_at_capture": batch}

    def forward(self, step, h, cache):
        fixed = step.fixed.get(self)
        assert fixed is None or fixed["batch_at_capture"] == step.n_seqs
        bucket = step.meta[self.KEY]["bucket"]
        assert bucket.shape[0] == h.shape[0] and bucket.dtype == torch.int32
        gain = torch.index_select(self.gain, 0, bucket.long())[:, None]
        return ((h.float() @ self.weight.float().t()) * gain).to(h.dtype)


@dataclass
class BucketConfig(ToyConfig):
    def to_dict(self):
        return {**super().to_dict(), "architectures": ["ToyBucketLM"]}


def bucket_builder(cfg):
    D = cfg.hidden_size

    def norm(name):
        return PartSpec("rms_norm", {"width": D, "eps": 1e-5, "name": name})

    def ffn(i):
        return PartSpec("swiglu", {"intermediate": INTER, "names": {p: f"l{i}.{p}" for p in ("gate", "up", "down")}})

    attention = PartSpec("attention", {
        "n_heads": HQ, "n_kv_heads": HK, "head_dim": HD, "window": 0,
        "position": PartSpec("rotary", {"head_dim": HD, "theta": 100.0, "scaling": None, "interleaved": False}),
        "names": {p: f"l0.{p}" for p in "qkvo"}})
    layers = [LayerSpec(PartSpec("pre_norm"), attention, ffn(0), {"input": norm("l0.n1"), "post_mixer": norm("l0.n2")}),
              LayerSpec(PartSpec("pre_norm"), PartSpec("bucket_gain", {"name": "l1.mix"}), ffn(1),
                        {"input": norm("l1.n1"), "post_mixer": norm("l1.n2")})]
    return ModelSpec(hidden_size=D, vocab_size=cfg.vocab_size, max_positions=256,
                     embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "name": "emb"}),
                     layers=layers, schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1)], final_norm=norm("final"),
                     lm_head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "name": "head", "tied_to": None}))


def bucket_plain(weights, tokens):
    T = len(tokens)
    pos = np.arange(T)
    inv = pl.rope_inverse_frequencies(HD, 100.0)
    x = pl.embedding(weights["emb"], tokens)
    for i in (0, 1, 1):
        h = pl.rms_norm(x, weights[f"l{i}.n1"], 1e-5)
        if i == 0:
            q = pl.apply_rope(pl.linear(h, weights["l0.q.weight"]).reshape(T, HQ, HD), pos, inv, False)
            k = pl.apply_rope(pl.linear(h, weights["l0.k.weight"]).reshape(T, HK, HD), pos, inv, False)
            v = pl.linear(h, weights["l0.v.weight"]).reshape(T, HK, HD)
            x = x + pl.linear(pl.causal_attention(q, k, v).reshape(T, HQ * HD), weights["l0.o.weight"])
        else:
            gain = weights["l1.mix.gain"].astype(np.float64)[np.minimum(pos // 16, 3)][:, None]
            x = x + pl.linear(h, weights["l1.mix.w"]) * gain
        h = pl.rms_norm(x, weights[f"l{i}.n2"], 1e-5)
        x = x + pl.feed_forward(h, weights[f"l{i}.gate.weight"], weights[f"l{i}.up.weight"], weights[f"l{i}.down.weight"])
    return pl.linear(pl.rms_norm(x, weights["final"], 1e-5), weights["head"])


def test_toy_mixer_with_index_arrays_of_its_own_under_graph_replay(tmp_path):
    from cpp_minilamma_b200 import EngineBackend, SamplingParams
    from cpp_minilamma_b200.engine.generate import generate
    register_part("mixer", "bucket_gain", BucketGainMixer)
    ml.register_architecture("ToyBucketLM", BucketConfig, bucket_builder)
    cfg = ml.config_from_dict({"architectures": ["ToyBucketLM"], "vocab_size": 89, "hidden_size": 40})
    folder = ml.write_random_model(cfg, tmp_path, seed=9)
    _, weights = pl.read_model_folder(folder)
    llm = ml.load(folder, dtype="float32", max_tokens=64 * 12, max_seqs=3)
    assert llm.model.capturable()
    assert set(llm.engine.providers) == {BucketGainMixer.KEY, llm.model.layers[0].mixer.step_metadata_key()}
    rng = np.random.RandomState(3)
    requests = [[int(t) for t in rng.randint(0, 89, size=n)] for n in (70, 5, 20)]
    # whole requests, and a batch of prompts followed by single tokens, against the plain implementation
    for r in requests:
        slot, = llm.engine.acquire(1)
        BucketGainMixer.prepared = 0
        got = llm.engine.step([StepEntry(slot, r, list(range(len(r))))])
        assert BucketGainMixer.prepared == 1   # two schedule entries, one preparation
        llm.engine.release(slot)
        assert_close(got.cpu().numpy(), bucket_plain(weights, r), "float32", "bucket whole")
    slots = llm.engine.acquire(3)
    heads = [len(r) - 4 for r in requests]
    llm.engine.step([StepEntry(s, r[:h], []) for s, r, h in zip(slots, requests, heads)])
    for k in range(4):
        out = llm.engine.step([StepEntry(s, [r[h + k]], [0]) for s, r, h in zip(slots, requests, heads)]).cpu().numpy()
        for i, r in enumerate(requests):
            assert_close(out[i], bucket_plain(weights, r)[heads[i] + k], "float32", f"bucket decode {i}")
    for s in slots:
        llm.engine.release(s)
    # generation: 40 new tokens from prompts of 5 and 20 tokens, so that positions pass through every bucket while the
    # decode steps replay a captured graph one step ahead of the host; same tokens as eager step-by-step launches
    prompts = [requests[1], requests[2]]
    eager = generate(EngineBackend(llm.engine, SamplingParams(), use_graphs=False), prompts, 40)
    backend = EngineBackend(llm.engine, SamplingParams())
    replayed = generate(backend, prompts, 40)
    assert backend.graphs.replays > 30
    assert [c.tokens for c in replayed] == [c.tokens for c in eager]
    for prompt, completion in zip(prompts, replayed):
        ref = bucket_plain(weights, list(prompt) + completion.tokens)
        for i, token in enumerate(completion.tokens):
            row = ref[len(prompt) - 1 + i]
            assert token == int(np.argmax(row)) or row.max() - row[token] <= 2e-4
    llm.engine.cache.check()
