"""The sampling kernel against the plain restatement of the reference's sampler."""
import numpy as np
import pytest
import torch

from plain import sampler as ps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_sampler(logits_row, n_draws, temperature, top_k, top_p, penalty, history=(), seed=0):
    """Draws ``n_draws`` tokens from one row of logits, each from a slot with a stream of its own."""
    from xeno_rt_b200.csrc import ops
    from xeno_rt_b200.sampling import sequence_key
    vocab = len(logits_row)
    logits = torch.tensor(np.asarray(logits_row, dtype=np.float32), device=DEV).repeat(n_draws, 1).contiguous()
    slots = torch.arange(n_draws, dtype=torch.int32, device=DEV)
    keys = np.array([sequence_key(seed * 100003 + i) for i in range(n_draws)], dtype=np.uint64).view(np.int64)
    rng_key = torch.from_numpy(keys).to(DEV)
    counter = torch.zeros(n_draws, dtype=torch.int32, device=DEV)
    words = (vocab + 31) // 32
    seen = torch.zeros(n_draws, words, dtype=torch.int32, device=DEV)
    if len(history):
        ids = torch.tensor(list(history) * n_draws, dtype=torch.int32, device=DEV)
        sl = slots.repeat_interleave(len(history)).contiguous()
        ops.mark_seen(seen, sl, ids, vocab)
    full = lambda v, dt: torch.full((n_draws,), v, dtype=dt, device=DEV)
    out = torch.empty(n_draws, dtype=torch.int32, device=DEV)
    ops.sample(out, logits, slots, full(temperature, torch.float32), full(top_k, torch.int32),
               full(top_p, torch.float32), full(penalty, torch.float32), seen, rng_key, counter)
    assert counter.eq(1).all()
    return out.cpu().numpy()


def test_greedy_is_argmax_first_maximum():
    logits = np.random.default_rng(0).normal(size=5000).astype(np.float32)
    logits[[77, 4000]] = 9.0
    assert run_sampler(logits, 3, 0.0, 40, 0.95, 1.0).tolist() == [77] * 3
    assert run_sampler(logits, 2, 1e-5, 0, 1.0, 1.0).tolist() == [77] * 2


def test_repetition_penalty_flips_greedy():
    logits = np.zeros(300, dtype=np.float32)
    logits[10], logits[20], logits[30] = 4.0, 3.0, -1.0
    assert run_sampler(logits, 1, 0.0, 0, 1.0, 2.0, history=[10, 10, 30])[0] == 20  # 4/2 < 3
    assert run_sampler(logits, 1, 0.0, 0, 1.0, 1.0, history=[10])[0] == 10  # penalty 1 = none
    assert run_sampler(logits, 1, 0.0, 0, 1.0, 2.0)[0] == 10  # empty history


@pytest.mark.parametrize("temperature,top_k,top_p,penalty,history", [
    (0.8, 40, 0.95, 1.1, (3, 5, 700)),      # the reference's defaults
    (1.0, 0, 1.0, 1.0, ()),                 # plain temperature sampling over everything
    (1.5, 5, 1.0, 1.0, ()),                 # top-k alone
    (0.7, 0, 0.6, 1.0, ()),                 # top-p alone
    (1.0, 3, 0.5, 1.3, (0, 1, 2)),
])
def test_support_and_frequencies_match_the_plain_sampler(temperature, top_k, top_p, penalty, history):
    rng = np.random.default_rng(42)
    vocab = 1000
    logits = (rng.normal(size=vocab) * 2.0).astype(np.float32)
    ids, probs = ps.candidate_distribution(logits, history, temperature, top_k, top_p, penalty)
    n = 20000
    got = run_sampler(logits, n, temperature, top_k, top_p, penalty, history)
    assert set(got.tolist()) <= set(ids.tolist()), "a token outside the kept set was drawn"
    expect = dict(zip(ids.tolist(), probs.tolist()))
    counts = np.bincount(got, minlength=vocab)
    for tok, p in expect.items():
        if p > 0.02:
            assert abs(counts[tok] / n - p) < 4 * np.sqrt(p * (1 - p) / n) + 1e-3, (tok, p, counts[tok] / n)
    big = [t for t, p in expect.items() if p > 0.02]
    assert all(counts[t] > 0 for t in big)


def test_top_k_keeps_the_earlier_of_equal_values():
    logits = np.full(200, -5.0, dtype=np.float32)
    logits[[50, 60, 70, 80]] = 2.0  # four equal maxima, top_k = 2 keeps ids 50 and 60
    got = run_sampler(logits, 4000, 1.0, 2, 1.0, 1.0)
    assert set(got.tolist()) == {50, 60}
    assert abs((got == 50).mean() - 0.5) < 0.05
    got = run_sampler(logits, 2000, 1.0, 0, 0.5, 1.0)  # mass 0.5 of 4 equal tokens (plus dust): 50, 60 (and 70 at most)
    assert 50 in got and 60 in got and 80 not in got


def test_a_seed_gives_the_same_tokens_and_another_seed_others():
    logits = np.random.default_rng(1).normal(size=4000).astype(np.float32)
    a = run_sampler(logits, 64, 1.0, 0, 1.0, 1.0, seed=7)
    b = run_sampler(logits, 64, 1.0, 0, 1.0, 1.0, seed=7)
    c = run_sampler(logits, 64, 1.0, 0, 1.0, 1.0, seed=8)
    assert np.array_equal(a, b) and not np.array_equal(a, c)


def test_big_vocabulary_and_padding_rows():
    from xeno_rt_b200.csrc import ops
    vocab = 151936
    logits = torch.randn(3, vocab, device=DEV)
    logits[0, 150000] = 50.0
    slots = torch.tensor([0, -1, 1], dtype=torch.int32, device=DEV)
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    f = lambda v, dt: torch.full((3,), v, dtype=dt, device=DEV)
    ops.sample(out, logits, slots, f(0.8, torch.float32), f(40, torch.int32), f(0.95, torch.float32),
               f(1.0, torch.float32), None, torch.zeros(2, dtype=torch.int64, device=DEV),
               torch.zeros(2, dtype=torch.int32, device=DEV))
    got = out.tolist()
    assert got[0] == 150000 and got[1] == -1 and 0 <= got[2] < vocab
    top40 = set(torch.topk(logits[2], 40).indices.tolist())
    assert got[2] in top40


def test_small_top_k_over_a_big_vocabulary_gathered_or_not():
    """A small top_k gathers its candidates into shared memory first (everything in the bin of the
    k-th largest logit or above, at most 4,096); when more than that share the bin the kernel walks
    the vocabulary instead.  Both ways keep the same set: equal values at the cut in index order."""
    vocab = 70001
    rng = np.random.default_rng(5)
    # (1) gathered: ties at the cut.  300 equal logits share the 40th place; ids in rising order win
    logits = (rng.normal(size=vocab) * 0.5).astype(np.float32)
    high = rng.choice(vocab, size=30, replace=False)
    logits[high] = 6.0 + rng.random(30).astype(np.float32)
    tied = np.setdiff1d(rng.choice(vocab, size=320, replace=False), high)[:300]
    logits[tied] = 4.25
    got = run_sampler(logits, 3000, 1.0, 40, 1.0, 1.0)
    kept = set(high.tolist()) | set(np.sort(tied)[:10].tolist())
    assert set(got.tolist()) <= kept
    ids, probs = ps.candidate_distribution(logits, (), 1.0, 40, 1.0, 1.0)
    assert set(ids.tolist()) == kept
    # (2) not gathered: every logit equal, 70,001 elements in one bin; top_k 40 keeps ids 0 .. 39
    flat = np.full(vocab, 1.5, dtype=np.float32)
    got = run_sampler(flat, 2000, 1.0, 40, 1.0, 1.0)
    assert set(got.tolist()) <= set(range(40)) and len(set(got.tolist())) > 30
    # (3) the reference's defaults on the gathered path against the plain sampler's kept set
    logits = (rng.normal(size=vocab) * 3.0).astype(np.float32)
    ids, probs = ps.candidate_distribution(logits, (7, 8), 0.8, 40, 0.95, 1.1)
    got = run_sampler(logits, 4000, 0.8, 40, 0.95, 1.1, history=(7, 8))
    assert set(got.tolist()) <= set(ids.tolist())
    top = int(ids[np.argmax(probs)])
    assert abs((got == top).mean() - probs.max()) < 4 * np.sqrt(probs.max() * (1 - probs.max()) / 4000) + 1e-3
