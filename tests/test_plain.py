"""The plain implementation against closed forms, some of them the reference's own test cases
(tests/kernels_test.rs of the reference), and against itself (no GPU)."""
import math

import numpy as np

from plain import model as pm
from plain import sampler as ps


def test_rmsnorm_closed_form():
    # the reference's case (tests/kernels_test.rs:75-91): hand formula
    x = np.array([1.0, 2.0, 3.0, 4.0])
    w = np.array([1.0, 0.5, 2.0, 1.5])
    inv = 1.0 / math.sqrt((1 + 4 + 9 + 16) / 4 + 1e-5)
    assert np.allclose(pm.rmsnorm(x, w, 1e-5), x * inv * w, atol=1e-12)


def test_rope_manual_angles():
    # the reference's case (tests/kernels_test.rs:94-108): head_dim 4, position 2, base 1e4
    x = np.array([[1.0, 2.0, 3.0, 4.0]])
    out = pm.rope(x, [2], 1, 4, 4, 10000.0, 1.0)[0]
    a0, a1 = 2.0, 2.0 / 100.0
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            1 * math.sin(a0) + 3 * math.cos(a0), 2 * math.sin(a1) + 4 * math.cos(a1)]
    assert np.allclose(out, want, atol=1e-6)
    # position 0 rotates nothing; a partial rope_dim leaves the tail alone
    assert np.allclose(pm.rope(x, [0], 1, 4, 4, 10000.0, 1.0), x)
    assert np.allclose(pm.rope(x, [5], 1, 4, 2, 10000.0, 1.0)[0, 2:], x[0, 2:])


def test_softmax_and_swiglu():
    s = pm.softmax(np.array([1.0, 2.0, 3.0]))
    assert abs(s.sum() - 1) < 1e-12 and np.allclose(s, np.exp([1, 2, 3]) / np.exp([1, 2, 3]).sum())
    assert np.allclose(pm.swiglu(np.array([0.0, 1.0, -2.0]), np.array([3.0, 2.0, 1.0])),
                       [0.0, 2.0 / (1 + math.exp(-1)), -2.0 / (1 + math.exp(2))])


def test_attention_is_causal_and_grouped():
    rng = np.random.default_rng(0)
    t, nh, nkv, hd = 6, 4, 2, 8
    q, k, v = rng.normal(size=(t, nh * hd)), rng.normal(size=(t, nkv * hd)), rng.normal(size=(t, nkv * hd))
    full = pm.causal_gqa_attention(q, k, v, nh, nkv, hd)
    k2, v2 = k.copy(), v.copy()
    k2[4:], v2[4:] = 99.0, -99.0  # later keys must not reach earlier queries
    assert np.allclose(pm.causal_gqa_attention(q, k2, v2, nh, nkv, hd)[:4], full[:4])
    assert np.allclose(full[0].reshape(nh, hd)[1], v[0].reshape(nkv, hd)[0])  # head 1 reads kv head 0
    assert np.allclose(full[0].reshape(nh, hd)[2], v[0].reshape(nkv, hd)[1])  # head 2 reads kv head 1
    windowed = pm.causal_gqa_attention(q, k, v, nh, nkv, hd, window=1)
    assert np.allclose(windowed.reshape(t, nh, hd)[:, 0], v.reshape(t, nkv, hd)[:, 0])


def test_prefix_logits_do_not_depend_on_what_follows(tmp_path):
    from helpers import make_folder, random_prompts
    from plain.files import read_model_folder
    cfg, w = read_model_folder(make_folder(tmp_path, "tiny-qwen3", sharpen=6.0))
    (p,) = random_prompts(cfg["vocab_size"], [12])
    whole = pm.forward_logits(cfg, w, p)
    assert np.allclose(pm.forward_logits(cfg, w, p[:7]), whole[:7], atol=1e-12)
    assert whole.shape == (12, cfg["vocab_size"]) and np.isfinite(whole).all()
    gen = pm.greedy_generate(cfg, w, p, 3)
    assert gen[0] == int(np.argmax(whole[-1])) and len(gen) == 3


def test_plain_sampler_follows_the_reference_rules():
    logits = np.array([1.0, 3.0, 2.0, 3.0, -1.0])
    assert ps.greedy(logits) == 1  # first maximum
    assert ps.greedy(logits, history=[1, 3], repetition_penalty=2.0) == 2  # 3/2 < 2
    assert ps.penalised(np.array([-1.0, 2.0]), [0, 1, 1], 2.0).tolist() == [-2.0, 1.0]
    ids, probs = ps.candidate_distribution(logits, (), 1.0, 3, 1.0, 1.0)
    assert ids.tolist() == [1, 3, 2] and abs(probs.sum() - 1) < 1e-12
    ids, probs = ps.candidate_distribution(logits, (), 1.0, 0, 0.5, 1.0)
    assert ids.tolist() == [1, 3]  # 0.39 < 0.5 <= 0.78
    assert ps.sample(logits, 0.0, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0) == 1
    assert ps.sample(logits, 0.999999, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0) == 4
    cold = [ps.sample(logits, r, temperature=0.05, top_k=0, top_p=1.0, repetition_penalty=1.0)
            for r in np.linspace(0, 0.999, 50)]
    assert set(cold) <= {1, 3}  # a low temperature sharpens
