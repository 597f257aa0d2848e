"""The generation loop's decisions with a scripted backend (no GPU)."""
import pytest

import xeno_rt_b200  # noqa: F401
from xeno_rt_b200.core import ConfigError, RuntimeFault
from xeno_rt_b200.engine import (GenerateRequest, SequenceProgress, generate, plan_batches, tokens_held)


class ScriptedBackend:
    """Each sequence 'samples' from a script keyed by its first prompt token: script[first][n] is
    its n-th sampled token.  Records every call so that tests can check what was run."""

    def __init__(self, scripts, n_slots=8):
        self.scripts = scripts
        self.free = list(range(n_slots))
        self.open = {}
        self.calls = []
        self.closed = []

    def open_slot(self):
        slot = self.free.pop(0)
        self.open[slot] = {"first": None, "fed": 0, "sampled": 0}
        return slot

    def close_slot(self, slot):
        assert slot in self.open, "slot closed twice"
        del self.open[slot]
        self.free.insert(0, slot)
        self.closed.append(slot)

    def begin(self, slots, requests):
        for s, r in zip(slots, requests):
            self.open[s]["first"] = r.prompt_ids[0]

    def forward(self, slots, token_lists):
        self.calls.append(("forward", list(slots), [list(t) for t in token_lists]))
        for s, t in zip(slots, token_lists):
            self.open[s]["fed"] += len(t)
        return list(slots)

    def sample(self, logits, slots, requests):
        assert logits == list(slots)
        out = []
        for s in slots:
            st = self.open[s]
            out.append(self.scripts[st["first"]][st["sampled"]])
            st["sampled"] += 1
        return out


def req(first, n_prompt, **kw):
    return GenerateRequest(prompt_ids=[first] + [50] * (n_prompt - 1), **kw)


def test_sequence_progress_order_of_decisions():
    p = SequenceProgress(GenerateRequest([1, 2, 3], max_tokens=2), stop_ids=(9,), context_length=10)
    assert p.accept(4) is True and p.generated == [4]
    assert p.accept(5) is False and p.finish_reason == "length" and p.generated == [4, 5]
    with pytest.raises(RuntimeFault):
        p.accept(6)
    p = SequenceProgress(GenerateRequest([1, 2, 3], max_tokens=5), stop_ids=(9,), context_length=10)
    assert p.accept(9) is False and p.finish_reason == "stop" and p.generated == []  # stop id not kept
    p = SequenceProgress(GenerateRequest([1] * 9, max_tokens=5), stop_ids=(), context_length=10)
    assert p.accept(4) is True  # holds 10 now
    assert p.accept(5) is False and p.finish_reason == "context" and p.generated == [4]
    p = SequenceProgress(GenerateRequest([1], max_tokens=0), stop_ids=(), context_length=10)
    assert p.finished and p.finish_reason == "length"


def test_unequal_batch_early_finishers_and_no_trailing_forward():
    scripts = {1: [10, 11, 99], 2: [20, 99], 3: [30, 31, 32, 33, 34]}
    backend = ScriptedBackend(scripts)
    requests = [req(1, 5, max_tokens=8), req(2, 9, max_tokens=8), req(3, 13, max_tokens=4)]
    results, stats = generate(backend, requests, vocab_size=100, context_length=64, default_stop_ids=(99,))
    assert [r.tokens for r in results] == [[10, 11], [20], [30, 31, 32, 33]]
    assert [r.finish_reason for r in results] == ["stop", "stop", "length"]
    forwards = [c for c in backend.calls if c[0] == "forward"]
    # the prompts in one step, then one token each for those still running
    assert [len(t) for t in forwards[0][2]] == [5, 9, 13]
    assert forwards[1][2] == [[10], [20], [30]]
    assert forwards[2][2] == [[11], [31]]
    assert forwards[3][2] == [[32]]
    assert len(forwards) == 4  # no forward after the last token
    assert stats.tokens == 7 and stats.decode_steps == 3 and stats.batches == 1
    assert not backend.open and sorted(backend.closed) == [0, 1, 2]


def test_batches_one_after_another_reuse_slots():
    scripts = {i: [60 + i] * 10 for i in range(1, 7)}
    backend = ScriptedBackend(scripts, n_slots=2)
    requests = [req(i, 3 + i, max_tokens=2) for i in range(1, 7)]
    results, stats = generate(backend, requests, 100, 64, max_batch=2)
    assert stats.batches == 3 and [r.tokens for r in results] == [[60 + i] * 2 for i in range(1, 7)]
    assert sorted(backend.closed) == [0, 0, 0, 1, 1, 1] and not backend.open


def test_plan_batches_by_tokens_and_count():
    reqs = [GenerateRequest([1] * 10, max_tokens=20), GenerateRequest([1] * 100, max_tokens=100),
            GenerateRequest([1] * 60, max_tokens=10), GenerateRequest([1] * 5, max_tokens=5)]
    assert [tokens_held(r, 4096) for r in reqs] == [64, 256, 128, 64]
    assert tokens_held(reqs[1], 128) == 128  # capped by the context
    assert plan_batches(reqs, 4096, 320, 8) == [[0, 1], [2, 3]]
    assert plan_batches(reqs, 4096, 10 ** 6, 3) == [[0, 1, 2], [3]]
    with pytest.raises(RuntimeFault, match="may hold"):
        plan_batches(reqs, 4096, 128, 8)


def test_request_errors():
    backend = ScriptedBackend({})
    with pytest.raises(RuntimeFault, match="empty prompt"):
        generate(backend, [GenerateRequest([])], 100, 64)
    with pytest.raises(RuntimeFault, match="exceeds model context length"):
        generate(backend, [GenerateRequest([1] * 65)], 100, 64)
    with pytest.raises(RuntimeFault, match="outside the vocabulary"):
        generate(backend, [GenerateRequest([100])], 100, 64)
    with pytest.raises(ConfigError, match="temperature"):
        generate(backend, [GenerateRequest([1], temperature=-1.0)], 100, 64)


def test_slots_are_closed_when_the_backend_fails():
    class Failing(ScriptedBackend):
        def sample(self, logits, slots, requests):
            raise RuntimeError("boom")
    backend = Failing({1: [5]})
    with pytest.raises(RuntimeError):
        generate(backend, [req(1, 3)], 100, 64)
    assert not backend.open


def test_on_token_and_request_defaults():
    r = GenerateRequest([1])
    assert (r.max_tokens, r.temperature, r.top_k, r.top_p, r.repetition_penalty, r.seed) == (128, 0.8, 40, 0.95, 1.1, None)
    seen = []
    backend = ScriptedBackend({1: [5, 6, 7]})
    generate(backend, [req(1, 2, max_tokens=3)], 100, 64, on_token=lambda i, t: seen.append((i, t)))
    assert seen == [(0, 5), (0, 6), (0, 7)]


class PipelinedBackend(ScriptedBackend):
    """The same scripts through the calls of a backend that starts the next step before the ids
    reach the host.  'Device ids' are a list the host side of the test never looks at before
    ``sample_end``; a step fed by them records which rows it ran."""

    def sample_begin(self, logits, slots, requests):
        return {"ids": ScriptedBackend.sample(self, logits, slots, requests), "slots": list(slots)}

    def sample_end(self, pending):
        return list(pending["ids"])

    def forward_sampled(self, slots, pending):
        assert list(slots) == pending["slots"]  # the rows line up with the sampler's rows
        self.calls.append(("forward_sampled", list(slots), [[t] for t in pending["ids"]]))
        for s in slots:
            self.open[s]["fed"] += 1
        return list(slots)

    def rows(self, logits, rows):
        self.calls.append(("rows", list(rows)))
        return [logits[r] for r in rows]


@pytest.mark.parametrize("scripts,limits", [
    ({1: [10, 11, 99], 2: [20, 99], 3: [30, 31, 32, 33, 34]}, (8, 8, 4)),
    ({1: [10, 11, 12, 13], 2: [20, 21, 22, 23], 3: [30, 31, 32, 33]}, (3, 3, 3)),
    ({1: [99], 2: [20, 21, 99], 3: [30, 99]}, (5, 5, 5)),
])
def test_pipelined_backend_same_results(scripts, limits):
    """Starting the next step early changes no result and no finish reason; a sequence that ends on
    a stop token has run one step too many, and its row is dropped from that step's logits."""
    def run(backend):
        requests = [req(f, 4 + f, max_tokens=m) for f, m in zip((1, 2, 3), limits)]
        results, stats = generate(backend, requests, vocab_size=100, context_length=64, default_stop_ids=(99,))
        assert not backend.open  # every slot given back
        assert sorted(backend.closed) == sorted(set(backend.closed))
        return [(r.tokens, r.finish_reason) for r in results], stats
    plain, plain_stats = run(ScriptedBackend(scripts))
    piped_backend = PipelinedBackend(scripts)
    piped, piped_stats = run(piped_backend)
    assert piped == plain
    assert piped_stats.tokens == plain_stats.tokens and piped_stats.decode_steps == plain_stats.decode_steps
    kinds = [c[0] for c in piped_backend.calls]
    assert kinds[0] == "forward"
    if limits == (3, 3, 3):  # nobody stops: every decode step was started early except none at the token limit
        assert kinds.count("forward") == 1 and kinds.count("forward_sampled") == 2 and "rows" not in kinds
