"""Each part alone against its plain function, and the generality of the assembly: a toy mixer
with state of its own, a layer run twice, a layer reading another layer's cache."""
import math

import numpy as np
import pytest
import torch

from plain import model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def f64(t):
    return t.detach().double().cpu().numpy()


def rel(got, want):
    return float(np.abs(f64(got) - want).max() / np.abs(want).max())


def context_for(cache, token_lists, dtype):
    from xeno_rt_b200.engine import StepEntry, build_context
    slots = [cache.open_slot() for _ in token_lists]
    ctx, _ = build_context([StepEntry(s, t) for s, t in zip(slots, token_lists)], cache, 10 ** 6, dtype, DEV)
    cache.flush_tables()
    return ctx, slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.parts import part_class
    w = 1 + 0.1 * torch.randn(100, device=DEV)
    part = part_class("norm", "rmsnorm")({"width": 100, "eps": 2e-6}, {"weight": w}, parse_dtype(dtype), DEV)
    x = torch.randn(6, 100, device=DEV)
    out = part.forward(x)
    assert out.dtype == DT[dtype] and rel(out, pm.rmsnorm(f64(x), f64(w), 2e-6)) < TOL[dtype]
    rows = torch.tensor([5, 2], dtype=torch.int32, device=DEV)
    assert torch.equal(part.forward(x, rows), out[[5, 2]])


def test_rotary_part_and_no_position():
    from xeno_rt_b200.cache import Cache, KVNeed
    from xeno_rt_b200.core import DType
    from xeno_rt_b200.parts import part_class
    cache = Cache([KVNeed(1, 16)], 256, 4096, DType.F32, DEV)
    ctx, _ = context_for(cache, [[1] * 70, [2] * 3], DType.F32)
    part = part_class("position", "rotary")({"rope_dim": 48, "base": 50000.0, "scale": 1.0}, {}, DType.F32, DEV)
    table = part.tables(ctx)
    assert part.tables(ctx) is table  # once a step
    pos = ctx.tok_pos.cpu().numpy().astype(np.float32)
    angle = (pos[:, None] / pm.rope_frequencies(48, 50000.0)[None]).astype(np.float32).astype(np.float64)
    assert np.abs(f64(table[..., 0]) - np.cos(angle)).max() < 2e-7
    assert part_class("position", "none")({}, {}, DType.F32, DEV).tables(ctx) is None


def _attention_setup(dtype, nh, nkv, hd, d, qk_norm, token_lists):
    from xeno_rt_b200.cache import Cache
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.parts import part_class
    dt = parse_dtype(dtype)
    g = torch.Generator(device="cpu").manual_seed(hd + nh)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.15).to(DEV).to(DT[dtype])
    weights = {"q": mk(nh * hd, d), "k": mk(nkv * hd, d), "v": mk(nkv * hd, d), "o": mk(d, nh * hd)}
    if qk_norm:
        weights["q_norm"] = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV)
        weights["k_norm"] = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV)
    params = {"width": d, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "qk_norm": qk_norm, "eps": 1e-6,
              "window": None, "position": {"kind": "rotary", "params": {"rope_dim": hd, "base": 10000.0, "scale": 1.0}}}
    part = part_class("mixer", "attention")(params, weights, dt, DEV)
    cache = Cache([part.cache_need()], 64 * 8, 1024, dt, DEV)
    return part, cache, weights, dt


def _plain_attention(h, weights, nh, nkv, hd, qk_norm):
    q, k, v = pm.linear(h, f64(weights["q"])), pm.linear(h, f64(weights["k"])), pm.linear(h, f64(weights["v"]))
    if qk_norm:
        q = pm.head_rmsnorm(q, f64(weights["q_norm"]), nh, hd, 1e-6)
        k = pm.head_rmsnorm(k, f64(weights["k_norm"]), nkv, hd, 1e-6)
    pos = np.arange(h.shape[0])
    q, k = pm.rope(q, pos, nh, hd, hd, 10000.0, 1.0), pm.rope(k, pos, nkv, hd, hd, 10000.0, 1.0)
    return pm.linear(pm.causal_gqa_attention(q, k, v, nh, nkv, hd), f64(weights["o"]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,d,qk_norm", [(5, 1, 48, 100, True), (4, 4, 32, 72, False)])
def test_attention_part_prompt_then_single_tokens(dtype, nh, nkv, hd, d, qk_norm):
    from xeno_rt_b200.engine import StepEntry, build_context
    lens = [75, 9]
    part, cache, weights, dt = _attention_setup(dtype, nh, nkv, hd, d, qk_norm, lens)
    hs = [torch.randn(n, d, device=DEV).to(DT[dtype]) for n in lens]
    wants = [_plain_attention(f64(h), weights, nh, nkv, hd, qk_norm) for h in hs]
    slots = [cache.open_slot() for _ in lens]
    heads = [n - 4 for n in lens]
    # the prompts' heads in one step
    ctx, _ = build_context([StepEntry(s, [0] * k) for s, k in zip(slots, heads)], cache, 10, dt, DEV)
    cache.flush_tables()
    residual = torch.zeros(sum(heads), d, device=DEV)
    part.forward(torch.cat([h[:k] for h, k in zip(hs, heads)]), residual, ctx, cache.store(0))
    for s, k in zip(slots, heads):
        cache.advance(s, k)
    got = [[residual[:heads[0]]], [residual[heads[0]:]]]
    for t in range(4):
        ctx, _ = build_context([StepEntry(s, [0]) for s in slots], cache, 10, dt, DEV)
        cache.flush_tables()
        residual = torch.zeros(2, d, device=DEV)
        part.forward(torch.cat([h[k + t:k + t + 1] for h, k in zip(hs, heads)]), residual, ctx, cache.store(0))
        for i, s in enumerate(slots):
            cache.advance(s, 1)
            got[i].append(residual[i:i + 1])
    for i in range(2):
        assert rel(torch.cat(got[i]), wants[i]) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_embedding_and_head_parts(dtype):
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.parts import part_class
    dt = parse_dtype(dtype)
    mk = lambda *s: (torch.randn(*s, device=DEV) * 0.2).to(DT[dtype])
    w = {"gate": mk(136, 100), "up": mk(136, 100), "down": mk(100, 136)}
    ffn = part_class("feed_forward", "swiglu")({"width": 100, "inner": 136}, w, dt, DEV)
    h = torch.randn(7, 100, device=DEV).to(DT[dtype])
    residual = torch.randn(7, 100, device=DEV)
    want = f64(residual) + pm.linear(pm.swiglu(pm.linear(f64(h), f64(w["gate"])), pm.linear(f64(h), f64(w["up"]))),
                                     f64(w["down"]))
    ffn.forward(h, residual, None)
    assert rel(residual, want) < TOL[dtype]
    table = mk(203, 100)
    emb = part_class("embedding", "token")({"vocab_size": 203, "width": 100}, {"weight": table}, dt, DEV)
    ids = torch.tensor([5, 202, 0], dtype=torch.int32, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids, flag), table[ids.long()].float())
    head = part_class("lm_head", "linear")({"vocab_size": 203, "width": 100}, {"weight": table}, dt, DEV)
    logits = head.forward(h)
    assert logits.dtype == torch.float32 and rel(logits, pm.linear(f64(h), f64(table))) < TOL[dtype]


class RunningMeanMixer:
    """A toy mixer with a state of its own: y_t = W . mean(h_0 .. h_t) of its sequence.  The state
    kept for each sequence is the sum of its inputs so far (its length comes with the step)."""

    @classmethod
    def weight_shapes(cls, params):
        return {"w": ((params["width"], params["width"]), "matrix")}

    def __init__(self, params, weights, dtype, device):
        self.width = params["width"]
        self.w = weights["w"]

    def cache_need(self):
        from xeno_rt_b200.cache import StateNeed
        return StateNeed((self.width,), "float32")

    def forward(self, h, residual, ctx, store, owns_cache=True):
        cu = ctx.cu_seqlens.tolist()
        for i, slot in enumerate(ctx.seq_slot.tolist()):
            seg = h[cu[i]:cu[i + 1]].float()
            sums = store.state[slot] + torch.cumsum(seg, dim=0)
            counts = torch.arange(1, seg.shape[0] + 1, device=h.device).float() + ctx.starts[i]
            residual[cu[i]:cu[i + 1]] += (sums / counts[:, None]) @ self.w.float().T
            store.state[slot] = sums[-1]


def _toy_spec(schedule=None, share=False):
    from xeno_rt_b200.parts import ModelSpec, PartSpec, SchedulePlace, prenorm_layer
    d, vocab = 40, 50
    norm = lambda name: PartSpec("rmsnorm", {"width": d, "eps": 1e-5}, {"weight": name})
    attn = PartSpec("attention", {"width": d, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16, "qk_norm": False,
                                  "eps": 1e-5, "window": None,
                                  "position": {"kind": "rotary", "params": {"rope_dim": 16, "base": 100.0, "scale": 1.0}}},
                    {"q": "l0.q", "k": "l0.k", "v": "l0.v", "o": "l0.o"})
    ffn = lambda i: PartSpec("swiglu", {"width": d, "inner": 24}, {"gate": f"l{i}.g", "up": f"l{i}.u", "down": f"l{i}.d"})
    layers = [prenorm_layer(norm("l0.n1"), attn, norm("l0.n2"), ffn(0)),
              prenorm_layer(norm("l1.n1"), PartSpec("test_running_mean", {"width": d}, {"w": "l1.w"}), norm("l1.n2"), ffn(1))]
    schedule = schedule or [SchedulePlace(0), SchedulePlace(1)]
    return ModelSpec(vocab_size=vocab, hidden_size=d, max_positions=256,
                     embedding=PartSpec("token", {"vocab_size": vocab, "width": d}, {"weight": "emb"}),
                     layers=layers, schedule=schedule, final_norm=norm("fn"),
                     lm_head=PartSpec("linear", {"vocab_size": vocab, "width": d}, {"weight": "emb"}))


def _toy_model(spec, dtype="float32"):
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.engine import Model
    from xeno_rt_b200.weights import random_tensors
    dt = parse_dtype(dtype)
    tensors = {k: v.to(DEV) for k, v in random_tensors(spec.expected_tensors(), 4, dt).items()}
    for k in tensors:
        if k.endswith((".q", ".k", ".w")):
            tensors[k] = tensors[k] * 8
    return Model(spec, tensors, dt, DEV), tensors


def _plain_toy(tensors, schedule, tokens):
    """The toy model restated on whole sequences with the plain functions."""
    w = {k: f64(v) for k, v in tensors.items()}
    x = pm.embedding(w["emb"], tokens)
    pos = np.arange(len(tokens))
    kv_of_place = {}
    for i, (layer, cache_from) in enumerate(schedule):
        h = pm.rmsnorm(x, w[f"l{layer}.n1"], 1e-5)
        if layer == 0:
            q = pm.rope(pm.linear(h, w["l0.q"]), pos, 2, 16, 16, 100.0, 1.0)
            if cache_from is None:
                k = pm.rope(pm.linear(h, w["l0.k"]), pos, 1, 16, 16, 100.0, 1.0)
                kv_of_place[i] = (k, pm.linear(h, w["l0.v"]))
            k, v = kv_of_place[i if cache_from is None else cache_from]
            x = x + pm.linear(pm.causal_gqa_attention(q, k, v, 2, 1, 16), w["l0.o"])
        else:
            means = np.cumsum(h, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
            x = x + pm.linear(means, w["l1.w"])
        h = pm.rmsnorm(x, w[f"l{layer}.n2"], 1e-5)
        x = x + pm.linear(pm.swiglu(pm.linear(h, w[f"l{layer}.g"]), pm.linear(h, w[f"l{layer}.u"])), w[f"l{layer}.d"])
    return pm.linear(pm.rmsnorm(x, w["fn"], 1e-5), w["emb"])


def _run_cut(engine, tokens, cuts):
    from xeno_rt_b200.engine import StepEntry
    slot = engine.open_slot()
    parts, at = [], 0
    for size in cuts:
        parts.append(engine.step([StepEntry(slot, tokens[at:at + size], list(range(size)))]).cpu().numpy())
        at += size
    engine.close_slot(slot)
    return np.concatenate(parts)


def test_a_toy_mixer_with_state_is_registered_built_and_stepped():
    from xeno_rt_b200.engine import Engine
    from xeno_rt_b200.parts import register_part
    register_part("mixer", "test_running_mean", RunningMeanMixer, replace=True)
    spec = _toy_spec()
    model, tensors = _toy_model(spec)
    engine = Engine(model, 64 * 4)
    assert len(engine.cache.kv_groups) == 1 and len(engine.cache.state_groups) == 1
    tokens = np.random.default_rng(0).integers(0, 50, size=70).tolist()
    want = _plain_toy(tensors, [(0, None), (1, None)], tokens)
    assert np.abs(_run_cut(engine, tokens, [70]) - want).max() / np.abs(want).max() < 2e-5
    assert np.abs(_run_cut(engine, tokens, [40] + [1] * 30) - want).max() / np.abs(want).max() < 2e-5
    # the slot is used again: its state must start from zero
    assert np.abs(_run_cut(engine, tokens, [3, 67]) - want).max() / np.abs(want).max() < 2e-5


def test_a_layer_named_twice_and_a_layer_reading_anothers_cache():
    from xeno_rt_b200.engine import Engine
    from xeno_rt_b200.parts import SchedulePlace, register_part
    register_part("mixer", "test_running_mean", RunningMeanMixer, replace=True)
    tokens = np.random.default_rng(1).integers(0, 50, size=80).tolist()
    # layer 0 runs twice with a cache of its own each time, then once more reading the first place's cache
    schedule = [SchedulePlace(0), SchedulePlace(1), SchedulePlace(0), SchedulePlace(0, cache_from=0)]
    spec = _toy_spec(schedule)
    model, tensors = _toy_model(spec)
    engine = Engine(model, 64 * 4)
    assert engine.cache.kv_groups[0].k.shape[0] == 2  # two places own keys and values, the fourth owns none
    want = _plain_toy(tensors, [(0, None), (1, None), (0, None), (0, 0)], tokens)
    assert np.abs(_run_cut(engine, tokens, [80]) - want).max() / np.abs(want).max() < 2e-5
    assert np.abs(_run_cut(engine, tokens, [50] + [1] * 30) - want).max() / np.abs(want).max() < 2e-5


def _windowed_spec():
    """Three attention layers of one shape: keys of the last 70 positions, every key, and the last 150
    positions read from the first layer's storage (which must then keep 150)."""
    from xeno_rt_b200.parts import ModelSpec, PartSpec, SchedulePlace, prenorm_layer
    d, vocab = 40, 50
    norm = lambda name: PartSpec("rmsnorm", {"width": d, "eps": 1e-5}, {"weight": name})
    attn = lambda i, window: PartSpec(
        "attention", {"width": d, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16, "qk_norm": False, "eps": 1e-5,
                      "window": window,
                      "position": {"kind": "rotary", "params": {"rope_dim": 16, "base": 100.0, "scale": 1.0}}},
        {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"})
    ffn = lambda i: PartSpec("swiglu", {"width": d, "inner": 24}, {"gate": f"l{i}.g", "up": f"l{i}.u", "down": f"l{i}.d"})
    layer = lambda i, window: prenorm_layer(norm(f"l{i}.n1"), attn(i, window), norm(f"l{i}.n2"), ffn(i))
    return ModelSpec(vocab_size=vocab, hidden_size=d, max_positions=512,
                     embedding=PartSpec("token", {"vocab_size": vocab, "width": d}, {"weight": "emb"}),
                     layers=[layer(0, 70), layer(1, None), layer(2, 150)],
                     schedule=[SchedulePlace(0), SchedulePlace(1), SchedulePlace(0)],
                     final_norm=norm("fn"),
                     lm_head=PartSpec("linear", {"vocab_size": vocab, "width": d}, {"weight": "emb"}))


def _plain_windowed(tensors, schedule, tokens):
    """schedule: (layer, window, place whose keys it reads or None) for each place."""
    w = {k: f64(v) for k, v in tensors.items()}
    x = pm.embedding(w["emb"], tokens)
    pos = np.arange(len(tokens))
    kv_of_place = {}
    for i, (layer, window, cache_from) in enumerate(schedule):
        h = pm.rmsnorm(x, w[f"l{layer}.n1"], 1e-5)
        q = pm.rope(pm.linear(h, w[f"l{layer}.q"]), pos, 2, 16, 16, 100.0, 1.0)
        if cache_from is None:
            kv_of_place[i] = (pm.rope(pm.linear(h, w[f"l{layer}.k"]), pos, 1, 16, 16, 100.0, 1.0),
                              pm.linear(h, w[f"l{layer}.v"]))
        k, v = kv_of_place[i if cache_from is None else cache_from]
        x = x + pm.linear(pm.causal_gqa_attention(q, k, v, 2, 1, 16, window=window), w[f"l{layer}.o"])
        h = pm.rmsnorm(x, w[f"l{layer}.n2"], 1e-5)
        x = x + pm.linear(pm.swiglu(pm.linear(h, w[f"l{layer}.g"]), pm.linear(h, w[f"l{layer}.u"])), w[f"l{layer}.d"])
    return pm.linear(pm.rmsnorm(x, w["fn"], 1e-5), w["emb"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_and_full_layers_in_one_model_release_their_blocks(dtype):
    """Layers that see a window of keys have a storage group of their own that gives blocks back while
    the sequence runs; the results must be those of plain windowed attention at every position,
    however the tokens are cut, and with a second sequence taking the blocks that the first gave back."""
    from xeno_rt_b200.engine import Engine, StepEntry
    from xeno_rt_b200.parts import SchedulePlace
    tol = {"float32": 2e-5, "bfloat16": 3e-2}[dtype]
    spec = _windowed_spec()
    model, tensors = _toy_model(spec, dtype)
    engine = Engine(model, 64 * 12)
    groups = {g.need.window: g for g in engine.cache.kv_groups}
    assert set(groups) == {70, None}
    tokens = np.random.default_rng(5).integers(0, 50, size=330).tolist()
    want = _plain_windowed(tensors, [(0, 70, None), (1, None, None), (0, 70, None)], tokens)
    scale = np.abs(want).max()
    assert np.abs(want - _plain_windowed(tensors, [(0, None, None), (1, None, None), (0, None, None)], tokens)).max() \
        > 0.05 * scale  # the window matters for these weights
    assert np.abs(_run_cut(engine, tokens, [330]) - want).max() / scale < tol
    assert np.abs(_run_cut(engine, tokens, [100, 130] + [1] * 100) - want).max() / scale < tol

    # two sequences of unequal lengths; the longer one gives blocks back that the next batch's sequences take
    other = np.random.default_rng(6).integers(0, 50, size=200).tolist()
    want_other = _plain_windowed(tensors, [(0, 70, None), (1, None, None), (0, 70, None)], other)
    for _ in range(2):
        a, b = engine.open_slot(), engine.open_slot()
        got_a = [engine.step([StepEntry(a, tokens[:150], list(range(150))), StepEntry(b, other[:90], list(range(90)))])]
        got_b = [got_a[0][150:]]
        got_a[0] = got_a[0][:150]
        for i in range(110):
            out = engine.step([StepEntry(a, [tokens[150 + i]], [0]), StepEntry(b, [other[90 + i]], [0])])
            got_a.append(out[:1]); got_b.append(out[1:])
            engine.cache.check()
        engine.close_slot(b)
        for i in range(70):
            got_a.append(engine.step([StepEntry(a, [tokens[260 + i]], [0])]))
        # length 330: positions up to 330 - 70 are behind the window: blocks 0 .. 3 of six are given back
        # (a block number stands for that block of every place of the group)
        assert groups[70].allocator.held == 2 and groups[None].allocator.held == 6
        engine.close_slot(a)
        assert np.abs(torch.cat(got_a).cpu().numpy() - want).max() / scale < tol
        assert np.abs(torch.cat(got_b).cpu().numpy() - want_other).max() / np.abs(want_other).max() < tol
    assert engine.cache.blocks_free() == engine.cache.n_blocks

    # a layer that sees 150 keys reads the storage of the layer that sees 70: the storage keeps 150
    spec = _windowed_spec()
    spec.schedule = [SchedulePlace(0), SchedulePlace(1), SchedulePlace(2, cache_from=0)]
    model = type(model)(spec, tensors, model.dtype, DEV)
    engine = Engine(model, 64 * 12)
    assert {g.need.window for g in engine.cache.kv_groups} == {150, None}
    want = _plain_windowed(tensors, [(0, 70, None), (1, None, None), (2, 150, 0)], tokens)
    assert np.abs(_run_cut(engine, tokens, [200] + [1] * 130) - want).max() / np.abs(want).max() < tol


class RoutedFeedForward:
    """A toy feed-forward with routing: a 32-bit softmax router over E experts picks one expert a
    token; y = p_e * W2_e . relu(W1_e . h).  Defined here, never in the framework."""

    @classmethod
    def weight_shapes(cls, params):
        d, f, e = params["width"], params["inner"], params["experts"]
        return {"router": ((e, d), "matrix"), "w1": ((e * f, d), "matrix"), "w2": ((e * d, f), "matrix")}

    def __init__(self, params, weights, dtype, device):
        self.d, self.f, self.e = params["width"], params["inner"], params["experts"]
        self.router = weights["router"].float()
        self.w1 = weights["w1"].float().view(self.e, self.f, self.d)
        self.w2 = weights["w2"].float().view(self.e, self.d, self.f)

    def forward(self, h, residual, ctx):
        h = h.float()
        probs = torch.softmax(h @ self.router.T, dim=-1)
        top = probs.argmax(dim=-1)
        for e in range(self.e):
            rows = (top == e).nonzero().flatten()
            if rows.numel():
                y = torch.relu(h[rows] @ self.w1[e].T) @ self.w2[e].T
                residual[rows] += probs[rows, e, None] * y


class LinearAngles:
    """A toy position encoding: pair i of a head is turned by pos * (i + 1) * step radians (not a
    power law).  It fits the rotation interface by handing the attention kernel another table."""

    @classmethod
    def weight_shapes(cls, params):
        return {}

    def __init__(self, params, weights, dtype, device):
        self.half = params["rope_dim"] // 2
        self.step = float(params["step"])

    def tables(self, ctx):
        key = ("test_linear_angles", self.half, self.step)
        if key not in ctx.shared:
            i = torch.arange(1, self.half + 1, device=ctx.tok_pos.device, dtype=torch.float32)
            angle = ctx.tok_pos.float()[:, None] * (i * self.step)[None]
            ctx.shared[key] = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).contiguous()
        return ctx.shared[key]


def test_toy_feed_forward_with_routing_and_another_position_encoding():
    """Both toy parts are registered from here, chosen by the spec for one layer of two, built and
    stepped (whole, cut into steps, and in a batch of two) without a change to the framework."""
    from xeno_rt_b200.engine import Engine, StepEntry
    from xeno_rt_b200.parts import ModelSpec, PartSpec, SchedulePlace, prenorm_layer, register_part
    register_part("feed_forward", "test_routed", RoutedFeedForward, replace=True)
    register_part("position", "test_linear_angles", LinearAngles, replace=True)
    d, vocab, hd, nh, nkv, experts, inner = 40, 50, 16, 3, 1, 3, 24
    norm = lambda name: PartSpec("rmsnorm", {"width": d, "eps": 1e-5}, {"weight": name})

    def attn(i, position):
        return PartSpec("attention", {"width": d, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "qk_norm": False,
                                      "eps": 1e-5, "window": None, "position": position},
                        {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"})
    layers = [
        prenorm_layer(norm("l0.n1"), attn(0, {"kind": "test_linear_angles", "params": {"rope_dim": 12, "step": 0.05}}),
                  norm("l0.n2"), PartSpec("test_routed", {"width": d, "inner": inner, "experts": experts},
                                          {"router": "l0.r", "w1": "l0.w1", "w2": "l0.w2"})),
        prenorm_layer(norm("l1.n1"), attn(1, {"kind": "rotary", "params": {"rope_dim": 16, "base": 100.0, "scale": 1.0}}),
                  norm("l1.n2"), PartSpec("swiglu", {"width": d, "inner": inner}, {"gate": "l1.g", "up": "l1.u", "down": "l1.d"})),
    ]
    spec = ModelSpec(vocab_size=vocab, hidden_size=d, max_positions=256,
                     embedding=PartSpec("token", {"vocab_size": vocab, "width": d}, {"weight": "emb"}),
                     layers=layers, schedule=[SchedulePlace(0), SchedulePlace(1)], final_norm=norm("fn"),
                     lm_head=PartSpec("linear", {"vocab_size": vocab, "width": d}, {"weight": "emb"}))
    model, tensors = _toy_model(spec)
    for k in tensors:
        if k.endswith(".r"):
            tensors[k] = tensors[k] * 40  # a clear winner among the experts, so that rounding cannot flip the choice
    from xeno_rt_b200.engine import Model
    model = Model(spec, tensors, model.dtype, DEV)
    assert not model.graph_safe  # the toy parts do not promise what graph replay needs: steps run kernel by kernel

    def plain(tokens):
        w = {k: f64(v) for k, v in tensors.items()}
        x = pm.embedding(w["emb"], tokens)
        pos = np.arange(len(tokens))
        for i in (0, 1):
            h = pm.rmsnorm(x, w[f"l{i}.n1"], 1e-5)
            q, k, v = pm.linear(h, w[f"l{i}.q"]), pm.linear(h, w[f"l{i}.k"]), pm.linear(h, w[f"l{i}.v"])
            if i == 0:
                def turn(t, heads):
                    t = t.reshape(len(tokens), heads, hd).copy()
                    angle = pos[:, None] * (np.arange(1, 7) * 0.05)[None]
                    c, s_ = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
                    a, b = t[..., :6].copy(), t[..., 6:12].copy()  # pairs (j, j + half) of the first 12 dims
                    t[..., :6], t[..., 6:12] = a * c - b * s_, a * s_ + b * c
                    return t.reshape(len(tokens), heads * hd)
                q, k = turn(q, nh), turn(k, nkv)
            else:
                q = pm.rope(q, pos, nh, hd, 16, 100.0, 1.0)
                k = pm.rope(k, pos, nkv, hd, 16, 100.0, 1.0)
            x = x + pm.linear(pm.causal_gqa_attention(q, k, v, nh, nkv, hd), w[f"l{i}.o"])
            h = pm.rmsnorm(x, w[f"l{i}.n2"], 1e-5)
            if i == 0:
                logits = pm.linear(h, w["l0.r"])
                probs = np.exp(logits - logits.max(-1, keepdims=True))
                probs /= probs.sum(-1, keepdims=True)
                y = np.zeros_like(x)
                for t in range(len(tokens)):
                    e = int(probs[t].argmax())
                    w1 = w["l0.w1"].reshape(experts, inner, d)[e]
                    w2 = w["l0.w2"].reshape(experts, d, inner)[e]
                    y[t] = probs[t, e] * (w2 @ np.maximum(w1 @ h[t], 0))
                x = x + y
            else:
                x = x + pm.linear(pm.swiglu(pm.linear(h, w["l1.g"]), pm.linear(h, w["l1.u"])), w["l1.d"])
        return pm.linear(pm.rmsnorm(x, w["fn"], 1e-5), w["emb"])

    rng = np.random.default_rng(3)
    a, b = rng.integers(0, vocab, size=70).tolist(), rng.integers(0, vocab, size=33).tolist()
    want_a, want_b = plain(a), plain(b)
    engine = Engine(model, 64 * 4)
    close = lambda got, want: np.abs(got - want).max() / np.abs(want).max() < 2e-5
    assert close(_run_cut(engine, a, [70]), want_a)
    assert close(_run_cut(engine, a, [38] + [1] * 32), want_a)
    # a batch of two of unequal lengths, prompts in one step and then one token each; the shorter ends earlier
    sa, sb = engine.open_slot(), engine.open_slot()
    first = engine.step([StepEntry(sa, a[:60], list(range(60))), StepEntry(sb, b[:30], list(range(30)))]).cpu().numpy()
    got_a, got_b = [first[:60]], [first[60:]]
    for t in range(10):
        entries = [StepEntry(sa, [a[60 + t]], [0])] + ([StepEntry(sb, [b[30 + t]], [0])] if t < 3 else [])
        out = engine.step(entries).cpu().numpy()
        got_a.append(out[:1])
        if t < 3:
            got_b.append(out[1:2])
        if t == 2:
            engine.close_slot(sb)
    engine.close_slot(sa)
    assert close(np.concatenate(got_a), want_a) and close(np.concatenate(got_b), want_b)


class InterleavedAngles:
    """A toy position encoding that turns NEIGHBOURING dims (2i, 2i + 1) of a head by pos * (i + 1) *
    step radians: it says so with ``pairing`` and hands the attention mixer its table."""
    pairing = "interleaved"

    @classmethod
    def weight_shapes(cls, params):
        return {}

    def __init__(self, params, weights, dtype, device):
        self.rope_dim = params["rope_dim"]
        self.half = self.rope_dim // 2
        self.step = float(params["step"])

    def tables(self, ctx):
        key = ("test_interleaved_angles", self.half, self.step)
        if key not in ctx.shared:
            i = torch.arange(1, self.half + 1, device=ctx.tok_pos.device, dtype=torch.float32)
            angle = ctx.tok_pos.float()[:, None] * (i * self.step)[None]
            ctx.shared[key] = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).contiguous()
        return ctx.shared[key]


def sandwich_residual(parts, x, ctx, stores, owns_cache):
    """A toy arrangement with a norm before AND after each of mixer and feed-forward:
    x += post(mixer(pre(x))); x += post(ffn(pre(x))).  It uses six named parts of the layer."""
    branch = torch.zeros_like(x)
    parts.mixer.forward(parts.pre_mixer.forward(x), branch, ctx, stores.get("mixer"), owns_cache)
    x += parts.post_mixer.forward(branch).float()
    branch = torch.zeros_like(x)
    parts.ffn.forward(parts.pre_ffn.forward(x), branch, ctx)
    x += parts.post_ffn.forward(branch).float()


def _keys_and_memory_mixer():
    from xeno_rt_b200.cache import StateNeed
    from xeno_rt_b200.parts.attention import GroupedQueryAttention

    class KeysAndMemoryMixer(GroupedQueryAttention):
        """A toy mixer that keeps keys AND a fixed-size state: attention plus 0.5 * the running mean
        of its inputs.  It asks the cache for both with a list and is handed a list of storages."""

        def cache_need(self):
            return [super().cache_need(), StateNeed((self.width,), "float32")]

        def forward(self, h, residual, ctx, store, owns_cache=True):
            keys, memory = store
            super().forward(h, residual, ctx, keys, owns_cache)
            cu = ctx.cu_seqlens.tolist()
            for i, slot in enumerate(ctx.seq_slot.tolist()):
                seg = h[cu[i]:cu[i + 1]].float()
                sums = memory.state[slot] + torch.cumsum(seg, dim=0)
                counts = torch.arange(1, seg.shape[0] + 1, device=h.device).float() + ctx.starts[i]
                residual[cu[i]:cu[i + 1]] += 0.5 * sums / counts[:, None]
                if owns_cache:
                    memory.state[slot] = sums[-1]

    KeysAndMemoryMixer.graph_safe = False
    return KeysAndMemoryMixer


def test_a_layer_of_six_parts_an_interleaved_encoding_and_a_mixer_with_keys_and_state():
    """Defined here alone and run through the unmodified engine: an arrangement over six named parts
    (norms before and after mixer and feed-forward), a position encoding that pairs neighbouring
    dims over part of the head, and a mixer whose ``cache_need`` is a list (keys and a state)."""
    from xeno_rt_b200.engine import Engine, Model, StepEntry
    from xeno_rt_b200.parts import LayerSpec, ModelSpec, PartSpec, SchedulePlace, prenorm_layer, register_part
    register_part("position", "test_interleaved_angles", InterleavedAngles, replace=True)
    register_part("arrangement", "test_sandwich", sandwich_residual, replace=True)
    register_part("mixer", "test_keys_and_memory", _keys_and_memory_mixer(), replace=True)
    d, vocab, hd, nh, nkv, inner, rd, step = 40, 50, 16, 3, 1, 24, 10, 0.07
    norm = lambda name: PartSpec("rmsnorm", {"width": d, "eps": 1e-5}, {"weight": name})
    attn = lambda i, kind: PartSpec(kind, {"width": d, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "qk_norm": False,
                                           "eps": 1e-5, "window": None,
                                           "position": {"kind": "test_interleaved_angles",
                                                        "params": {"rope_dim": rd, "step": step}}},
                                    {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"})
    ffn = lambda i: PartSpec("swiglu", {"width": d, "inner": inner}, {"gate": f"l{i}.g", "up": f"l{i}.u", "down": f"l{i}.d"})
    sandwich = LayerSpec({"pre_mixer": ("norm", norm("l0.n1")), "mixer": ("mixer", attn(0, "attention")),
                          "post_mixer": ("norm", norm("l0.n2")), "pre_ffn": ("norm", norm("l0.n3")),
                          "ffn": ("feed_forward", ffn(0)), "post_ffn": ("norm", norm("l0.n4"))}, "test_sandwich")
    layers = [sandwich, prenorm_layer(norm("l1.n1"), attn(1, "test_keys_and_memory"), norm("l1.n2"), ffn(1))]
    spec = ModelSpec(vocab_size=vocab, hidden_size=d, max_positions=256,
                     embedding=PartSpec("token", {"vocab_size": vocab, "width": d}, {"weight": "emb"}),
                     layers=layers, schedule=[SchedulePlace(0), SchedulePlace(1)], final_norm=norm("fn"),
                     lm_head=PartSpec("linear", {"vocab_size": vocab, "width": d}, {"weight": "emb"}))
    model, tensors = _toy_model(spec)
    assert {e.name for e in spec.expected_tensors()} >= {"l0.n3", "l0.n4"}
    needs = model.cache_needs()
    assert set(needs[0]) == {"mixer"} and isinstance(needs[1]["mixer"], list) and len(needs[1]["mixer"]) == 2
    engine = Engine(model, 64 * 4)
    assert len(engine.cache.kv_groups) == 1 and len(engine.cache.state_groups) == 1

    def turn(t, heads, n):
        t = t.reshape(n, heads, hd).copy()
        angle = np.arange(n)[:, None] * (np.arange(1, rd // 2 + 1) * step)[None]
        c, s_ = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
        a, b = t[..., 0:rd:2].copy(), t[..., 1:rd:2].copy()  # pairs (2j, 2j + 1) of the first rd dims
        t[..., 0:rd:2], t[..., 1:rd:2] = a * c - b * s_, a * s_ + b * c
        return t.reshape(n, heads * hd)

    def plain(tokens):
        w = {k: f64(v) for k, v in tensors.items()}
        n = len(tokens)
        x = pm.embedding(w["emb"], tokens)

        def attention(i, h):
            q, k, v = pm.linear(h, w[f"l{i}.q"]), pm.linear(h, w[f"l{i}.k"]), pm.linear(h, w[f"l{i}.v"])
            return pm.linear(pm.causal_gqa_attention(turn(q, nh, n), turn(k, nkv, n), v, nh, nkv, hd), w[f"l{i}.o"])

        def mlp(i, h):
            return pm.linear(pm.swiglu(pm.linear(h, w[f"l{i}.g"]), pm.linear(h, w[f"l{i}.u"])), w[f"l{i}.d"])
        x = x + pm.rmsnorm(attention(0, pm.rmsnorm(x, w["l0.n1"], 1e-5)), w["l0.n2"], 1e-5)
        x = x + pm.rmsnorm(mlp(0, pm.rmsnorm(x, w["l0.n3"], 1e-5)), w["l0.n4"], 1e-5)
        h = pm.rmsnorm(x, w["l1.n1"], 1e-5)
        x = x + attention(1, h) + 0.5 * np.cumsum(h, axis=0) / np.arange(1, n + 1)[:, None]
        x = x + mlp(1, pm.rmsnorm(x, w["l1.n2"], 1e-5))
        return pm.linear(pm.rmsnorm(x, w["fn"], 1e-5), w["emb"])

    rng = np.random.default_rng(5)
    a, b = rng.integers(0, vocab, size=75).tolist(), rng.integers(0, vocab, size=20).tolist()
    want_a, want_b = plain(a), plain(b)
    close = lambda got, want: np.abs(got - want).max() / np.abs(want).max() < 2e-5
    assert close(_run_cut(engine, a, [75]), want_a)
    assert close(_run_cut(engine, a, [40] + [1] * 35), want_a)   # the slot is used again: the state starts at zero
    sa, sb = engine.open_slot(), engine.open_slot()
    first = engine.step([StepEntry(sb, b[:18], list(range(18))), StepEntry(sa, a[:70], list(range(70)))]).cpu().numpy()
    got_b, got_a = [first[:18]], [first[18:]]
    for t in range(5):
        entries = ([StepEntry(sb, [b[18 + t]], [0])] if t < 2 else []) + [StepEntry(sa, [a[70 + t]], [0])]
        out = engine.step(entries).cpu().numpy()
        if t < 2:
            got_b.append(out[:1])
        got_a.append(out[-1:])
        if t == 1:
            engine.close_slot(sb)
    engine.close_slot(sa)
    assert close(np.concatenate(got_a), want_a) and close(np.concatenate(got_b), want_b)
    engine.cache.check()


def test_spec_errors():
    from xeno_rt_b200.core import ConfigError
    from xeno_rt_b200.parts import SchedulePlace, part_class
    with pytest.raises(ConfigError, match="no mixer part named"):
        part_class("mixer", "nonexistent")
    spec = _toy_spec([SchedulePlace(0), SchedulePlace(0, cache_from=1)])
    with pytest.raises(ConfigError, match="does not come before"):
        spec.validate()
    spec = _toy_spec([SchedulePlace(5)])
    with pytest.raises(ConfigError, match="names layer 5"):
        spec.validate()
