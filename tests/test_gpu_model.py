"""The engine against the plain implementation, in 32-bit and in bfloat16: each request alone and
whole; with the last 32 tokens one by one; in batches of unequal lengths whose shorter requests
end earlier, one batch after another so that slots and blocks are used again; long decoding; the
first tokens of a sequence; padding."""
import numpy as np
import pytest
import torch

from helpers import CONFIGS, TOL, make_folder, random_prompts, scaled_error

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"tiny-llama": [5, 9, 13, 70, 128], "tiny-qwen3": [1, 7, 16, 31, 97, 200], "tiny-odd": [3, 65, 130],
           "tiny-wide": [40, 129, 330]}


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    """For each tiny configuration: folder (sharpened weights), prompts, plain logits."""
    from plain.files import read_model_folder
    from plain.model import forward_logits
    out = {}
    root = tmp_path_factory.mktemp("models")
    for name in CONFIGS:
        folder = make_folder(root, name, sharpen=6.0)
        cfg, weights = read_model_folder(folder)
        prompts = random_prompts(cfg["vocab_size"], LENGTHS[name], seed=len(name))
        out[name] = (folder, prompts, [forward_logits(cfg, weights, p) for p in prompts])
    return out


@pytest.fixture(scope="module")
def engines(setups):
    from xeno_rt_b200.engine import Engine, Model
    made = {}

    def get(name, dtype, max_tokens=64 * 12):
        key = (name, dtype, max_tokens)
        if key not in made:
            made[key] = Engine(Model.load(setups[name][0], dtype=dtype), max_tokens=max_tokens)
        return made[key]
    return get


def _whole(engine, prompt):
    from xeno_rt_b200.engine import StepEntry
    slot = engine.open_slot()
    logits = engine.step([StepEntry(slot, prompt, list(range(len(prompt))))]).cpu().numpy()
    engine.close_slot(slot)
    return logits


def _tail_one_by_one(engine, prompt, tail=32):
    from xeno_rt_b200.engine import StepEntry
    slot = engine.open_slot()
    head = max(1, len(prompt) - tail)
    parts = [engine.step([StepEntry(slot, prompt[:head], list(range(head)))]).cpu().numpy()]
    for t in range(head, len(prompt)):
        parts.append(engine.step([StepEntry(slot, [prompt[t]], [0])]).cpu().numpy())
    engine.close_slot(slot)
    return np.concatenate(parts)


def _batch(engine, prompts, decode=8, pad_to=None):
    """The prompts minus their last ``decode`` tokens in one step, then one token each; a request
    leaves (and its slot is closed) when its tokens run out.  Returns logits for each request."""
    from xeno_rt_b200.engine import StepEntry
    slots = [engine.open_slot() for _ in prompts]
    heads = [max(1, len(p) - decode) for p in prompts]
    logits = engine.step([StepEntry(s, p[:h], list(range(h))) for s, p, h in zip(slots, prompts, heads)]).cpu().numpy()
    outs, offset = [[] for _ in prompts], 0
    for i, h in enumerate(heads):
        outs[i].append(logits[offset:offset + h])
        offset += h
    live = list(range(len(prompts)))
    step = 0
    while True:
        for i in [i for i in live if heads[i] + step >= len(prompts[i])]:
            engine.close_slot(slots[i])
            live.remove(i)
        if not live:
            break
        entries = [StepEntry(slots[i], [prompts[i][heads[i] + step]], [0]) for i in live]
        logits = engine.step(entries, pad_to=pad_to).cpu().numpy()
        for row, i in enumerate(live):
            outs[i].append(logits[row:row + 1])
        step += 1
    return [np.concatenate(o) for o in outs]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_each_request_alone_and_whole(setups, engines, name, dtype):
    _, prompts, refs = setups[name]
    engine = engines(name, dtype)
    for p, r in zip(prompts, refs):
        assert scaled_error(_whole(engine, p), r) < TOL[dtype], (name, dtype, len(p))
    engine.cache.check()
    assert engine.cache.blocks_free() == engine.cache.n_blocks


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_last_32_tokens_one_by_one(setups, engines, name, dtype):
    _, prompts, refs = setups[name]
    engine = engines(name, dtype)
    for p, r in zip(prompts, refs):
        got = _tail_one_by_one(engine, p)
        assert scaled_error(got, r) < TOL[dtype], (name, dtype, len(p))
        # cutting the tokens into steps changes the result by rounding only
        assert scaled_error(got, _whole(engine, p).astype(np.float64)) < (1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batches_one_after_another(setups, engines, name, dtype):
    folder, prompts, refs = setups[name]
    # a cache that holds one batch but not two: the second batch must reuse blocks and slots
    need = sum((len(p) + 63) // 64 * 64 for p in prompts)
    engine = engines(name, dtype, max_tokens=need)
    for round_ in range(3):
        order = list(range(len(prompts)))
        if round_ == 1:
            order.reverse()
        if round_ == 2:
            order = order[1:] + order[:1]
        got = _batch(engine, [prompts[i] for i in order], decode=8)
        for i, g in zip(order, got):
            assert scaled_error(g, refs[i]) < TOL[dtype], (name, dtype, round_, len(prompts[i]))
        engine.cache.check()
        assert engine.cache.blocks_free() == engine.cache.n_blocks


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_changes_no_result(setups, engines, dtype):
    _, prompts, refs = setups["tiny-qwen3"]
    engine = engines("tiny-qwen3", dtype)
    plain_run = _batch(engine, prompts[:4], decode=6)
    padded_run = _batch(engine, prompts[:4], decode=6, pad_to=16)
    for a, b in zip(plain_run, padded_run):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny-odd", "tiny-wide"])
def test_long_decoding(setups, engines, tmp_path, name, dtype):
    """300 tokens one by one from the first token on: positions cross four block edges.  At head size
    128 every step's attention kernel also norms, rotates and writes the step's own key and value."""
    from plain.files import read_model_folder
    from plain.model import forward_logits
    from xeno_rt_b200.engine import StepEntry
    folder, _, _ = setups[name]
    engine = None
    if name == "tiny-wide":
        # at head size 128 the sharpening of the other tests (x 6 on q and k) makes every softmax a near one-hot
        # choice, and bfloat16's rounding of q and k alone then moves single rows by 3 % of the logit scale; x 3
        # keeps far keys visible without that
        from xeno_rt_b200.engine import Engine, Model
        folder = make_folder(tmp_path, name, sharpen=3.0)
        engine = Engine(Model.load(folder, dtype=dtype), max_tokens=64 * 12)
    cfg, weights = read_model_folder(folder)
    (prompt,) = random_prompts(cfg["vocab_size"], [300], seed=9)
    ref = forward_logits(cfg, weights, prompt)
    engine = engine or engines(name, dtype)
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in prompt]
    engine.close_slot(slot)
    got = np.concatenate(rows)
    assert scaled_error(got[:4], ref[:4]) < TOL[dtype]  # the first tokens of a sequence
    assert scaled_error(got, ref) < TOL[dtype]
    worst = int(np.abs(got - ref).max(axis=1).argmax())
    assert scaled_error(got[worst:worst + 1], ref[worst:worst + 1]) < TOL[dtype], worst


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["tiny-odd", "tiny-wide"])
def test_decode_steps_of_very_unequal_lengths(setups, tmp_path, name, graphs):
    """Sequences of 3, 70, 300 and 900 tokens decode together: attention cuts its keys by the longest and
    by the mean length (finer than for four sequences of 900), so most splits of the short sequences hold
    no key at all, and the batch crosses a power of two of the mean on the way.  Every row against the
    plain implementation."""
    from plain.files import read_model_folder
    from plain.model import forward_logits
    from xeno_rt_b200.engine import Engine, Model
    folder = make_folder(tmp_path, name, sharpen=3.0)
    cfg, weights = read_model_folder(folder)
    prompts = random_prompts(cfg["vocab_size"], [3 + 12, 70 + 12, 300 + 12, 900 + 12], seed=21)
    engine = Engine(Model.load(folder, dtype="bfloat16"), max_tokens=64 * 24, use_graphs=graphs)
    got = _batch(engine, prompts, decode=12)
    for p, g in zip(prompts, got):
        assert scaled_error(g, forward_logits(cfg, weights, p)) < TOL["bfloat16"], len(p)
    if graphs:
        assert len({key[2] for key in engine._graphs}) >= 1 and all(key[2] <= key[1] for key in engine._graphs)


@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_of_several_tokens_continue_a_sequence(setups, engines, dtype):
    """Chunks of unequal size (not only prompts and single tokens) continue where the slot stands."""
    from xeno_rt_b200.engine import StepEntry
    _, prompts, refs = setups["tiny-qwen3"]
    p, r = prompts[-1], refs[-1]  # 200 tokens
    engine = engines("tiny-qwen3", dtype)
    slot = engine.open_slot()
    parts, at = [], 0
    for size in (63, 1, 2, 64, 70):
        parts.append(engine.step([StepEntry(slot, p[at:at + size], list(range(size)))]).cpu().numpy())
        at += size
    engine.close_slot(slot)
    assert at == 200 and scaled_error(np.concatenate(parts), r) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny-qwen3", "tiny-wide"])
def test_a_step_that_mixes_a_prompt_with_single_tokens_of_running_sequences(setups, engines, name, dtype):
    """Two sequences are under way (their prompts ran in an earlier step); the next step brings one
    token of each of them together with the whole prompt of a third, and the step after that one token
    of all three.  Every row against the plain implementation."""
    from xeno_rt_b200.engine import StepEntry
    _, prompts, refs = setups[name]
    a, b, c = prompts[-1], prompts[-2], prompts[-3]
    ra, rb, rc = refs[-1], refs[-2], refs[-3]
    engine = engines(name, dtype)
    sa, sb, sc = engine.open_slot(), engine.open_slot(), engine.open_slot()
    ha, hb, hc = len(a) - 2, len(b) - 2, len(c) - 1
    first = engine.step([StepEntry(sa, a[:ha], [ha - 1]), StepEntry(sb, b[:hb], list(range(hb)))]).cpu().numpy()
    assert scaled_error(first[:1], ra[ha - 1:ha]) < TOL[dtype] and scaled_error(first[1:], rb[:hb]) < TOL[dtype]
    mixed = engine.step([StepEntry(sa, [a[ha]], [0]), StepEntry(sc, c[:hc], list(range(hc))),
                         StepEntry(sb, [b[hb]], [0])]).cpu().numpy()
    assert scaled_error(mixed[:1], ra[ha:ha + 1]) < TOL[dtype]
    assert scaled_error(mixed[1:1 + hc], rc[:hc]) < TOL[dtype]
    assert scaled_error(mixed[1 + hc:], rb[hb:hb + 1]) < TOL[dtype]
    last = engine.step([StepEntry(sc, [c[hc]], [0]), StepEntry(sb, [b[hb + 1]], [0]),
                        StepEntry(sa, [a[ha + 1]], [0])]).cpu().numpy()
    for row, (ref, at) in enumerate(((rc, hc), (rb, hb + 1), (ra, ha + 1))):
        assert scaled_error(last[row:row + 1], ref[at:at + 1]) < TOL[dtype], row
    for s in (sa, sb, sc):
        engine.close_slot(s)
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_fed_with_ids_on_the_device_gives_the_logits_of_the_same_ids_from_the_host(setups, dtype):
    """``step_sampled`` takes the next ids from a device tensor (as the sampler leaves them) without
    a visit to the host; its logits are those of ``step`` on the same ids, bit for bit, graphs on or off."""
    from xeno_rt_b200.engine import Engine, Model, StepEntry
    folder, prompts, refs = setups["tiny-wide"]
    model = Model.load(folder, dtype=dtype)
    for graphs in (True, False):
        one, two = Engine(model, 64 * 12, use_graphs=graphs), Engine(model, 64 * 12, use_graphs=graphs)
        slots = []
        for engine in (one, two):
            slots.append([engine.open_slot() for _ in prompts])
            engine.step([StepEntry(s, p[:-3], []) for s, p in zip(slots[-1], prompts)])
        for k in (3, 2, 1):
            ids = [p[-k] for p in prompts]
            a = one.step([StepEntry(s, [t], [0]) for s, t in zip(slots[0], ids)])
            b = two.step_sampled(slots[1], torch.tensor(ids, dtype=torch.int32, device=model.device))
            assert torch.equal(a, b[:len(ids)])
            for row, (p, r) in enumerate(zip(prompts, refs)):
                assert scaled_error(b[row:row + 1].cpu().numpy(), r[len(p) - k:len(p) - k + 1]) < TOL[dtype]
        one.check_errors()
        two.check_errors()


VARIANTS = [{"decode_gemm": "stream"}, {"decode_gemm": "tcgen05"}, {"decode_gemm": "tcgen05", "decode_gemm_clusters": False},
            {"decode_attention": "nocluster"}, {"decode_attention": "cp"}, {"decode_attention": "rows"},
            {"prefill_attention": "mma"}, {"gemm_tile_rows": 128}, {"gemm_tile_rows": 256}, {"pdl": False},
            {"pending_norm": "force"}, {"pending_norm": "off"}, {"decode_cluster_pairs": 0}]


@pytest.mark.parametrize("variant", VARIANTS, ids=lambda v: ",".join(f"{k}={x}" for k, x in v.items()))
def test_every_kernel_variant_as_a_model_against_the_plain_implementation(setups, variant):
    """The library chooses among several kernels for one operation by size; each choice can be forced
    (``ops.Tuning``).  Here every forced variant runs the head-size-128 model in bfloat16 through the
    one-by-one and the unequal-batch schedules against the plain implementation, so that no variant is
    tested at kernel level only."""
    from xeno_rt_b200.csrc import ops
    from xeno_rt_b200.engine import Engine, Model
    folder, prompts, refs = setups["tiny-wide"]
    with ops.tuned(**variant):
        engine = Engine(Model.load(folder, dtype="bfloat16"), 64 * 12)
        for p, r in zip(prompts, refs):
            assert scaled_error(_tail_one_by_one(engine, p, tail=6), r) < TOL["bfloat16"], len(p)
        for g, r in zip(_batch(engine, prompts, decode=5), refs):
            assert scaled_error(g, r) < TOL["bfloat16"]
        engine.check_errors()
        engine.cache.check()
    assert ops.tuning() == ops.Tuning()


def test_step_errors(setups, engines):
    from xeno_rt_b200.core import CacheError, RuntimeFault
    from xeno_rt_b200.engine import StepEntry
    engine = engines("tiny-llama", "float32")
    slot = engine.open_slot()
    with pytest.raises(RuntimeFault, match="outside the vocabulary"):
        engine.step([StepEntry(slot, [256], [0])])
    with pytest.raises(RuntimeFault, match="at least one token"):
        engine.step([StepEntry(slot, [], [])])
    with pytest.raises(RuntimeFault, match="wanted place"):
        engine.step([StepEntry(slot, [1, 2], [2])])
    with pytest.raises(RuntimeFault, match="twice"):
        engine.step([StepEntry(slot, [1], [0]), StepEntry(slot, [2], [0])])
    with pytest.raises(CacheError, match="positions"):
        engine.step([StepEntry(slot, [1] * 129, [0])])
    assert engine.step([StepEntry(slot, [1, 2], [])]) is None
    engine.close_slot(slot)
    with pytest.raises(CacheError, match="not open"):
        engine.step([StepEntry(slot, [1], [0])])
    engine.cache.check()


def test_random_model_on_the_device_matches_the_written_folder(tmp_path):
    """Model.random draws on the GPU what write_random_model draws on the host."""
    from xeno_rt_b200.engine import Engine, Model, StepEntry
    from helpers import TINY_QWEN3
    from xeno_rt_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "m"), TINY_QWEN3, seed=5, dtype="bfloat16")
    a = Engine(Model.load(folder, dtype="bfloat16"), 128)
    b = Engine(Model.random(TINY_QWEN3, seed=5, dtype="bfloat16"), 128)
    prompt = list(range(40))
    la = a.step([StepEntry(a.open_slot(), prompt, [39])])
    lb = b.step([StepEntry(b.open_slot(), prompt, [39])])
    # the device draws what the host draws up to the last bit of a logarithm or cosine here and there
    assert scaled_error(lb.cpu().numpy(), la.cpu().numpy().astype(np.float64)) < 2e-3


@pytest.mark.parametrize("dtype", DTYPES)
def test_graph_replay_equals_eager_steps(setups, dtype):
    """Decode steps replayed from a CUDA graph give what the same steps give launched one by one,
    also when the batch shrinks and when a slot is used again."""
    from xeno_rt_b200.engine import Engine, Model
    folder, prompts, refs = setups["tiny-qwen3"]
    model = Model.load(folder, dtype=dtype)
    eager = Engine(model, 64 * 12, use_graphs=False)
    graphed = Engine(model, 64 * 12, use_graphs=True)
    for _ in range(2):
        a = _batch(eager, prompts[:5], decode=8)
        b = _batch(graphed, prompts[:5], decode=8)
        for x, y, r in zip(a, b, refs):
            assert np.array_equal(x, y)
            assert scaled_error(y, r) < TOL[dtype]
    assert graphed._graphs and not eager._graphs


def test_full_width_layers_agree_between_the_32_bit_and_the_bfloat16_path():
    """Two layers at the widths of the 8B models (hidden 4096, 32 heads over 8 kv heads of 128, feed-forward
    14336): the products, attention and fused kernels run at the sizes they are tuned for (the tiled tcgen05 product
    for the prompts, both decode products for 3 and 20 rows).  The 32-bit path, which the other tests tie to the
    plain implementation, is the oracle here; whole prompts and one-by-one decoding must agree too."""
    from xeno_rt_b200.engine import Engine, Model, StepEntry
    cfg = {"architectures": ["Qwen3ForCausalLM"], "vocab_size": 5000, "max_position_embeddings": 1024,
           "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 2, "num_attention_heads": 32,
           "num_key_value_heads": 8, "head_dim": 128, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
           "tie_word_embeddings": False}
    lengths = [300, 70, 129] + [40] * 17
    prompts = random_prompts(5000, lengths, seed=11)
    results = {}
    for dtype in ("float32", "bfloat16"):
        model = Model.random(cfg, seed=3, dtype=dtype)
        engine = Engine(model, 64 * 40)
        results[dtype] = {}
        for n_seq in (3, 20):
            got = _batch(engine, prompts[:n_seq], decode=4)
            results[dtype][n_seq] = got
            engine.cache.check()
        whole = _whole(engine, prompts[0])
        assert scaled_error(results[dtype][3][0], whole.astype(np.float64)) < (1e-5 if dtype == "float32" else 2e-2)
        del engine, model
        torch.cuda.empty_cache()
    for n_seq in (3, 20):
        for a, b in zip(results["bfloat16"][n_seq], results["float32"][n_seq]):
            assert scaled_error(a, b.astype(np.float64)) < TOL["bfloat16"]
    # the 32-bit result does not depend on the batch at all
    for a, b in zip(results["float32"][3], results["float32"][20][:3]):
        assert np.array_equal(a, b)
