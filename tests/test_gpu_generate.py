"""Generation through the Python entry point and the command line, and trace replay as a user
runs it, against the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import (CONFIGS, TOL, check_greedy_tokens, make_folder, random_prompts, replay_logits,
                     scaled_error)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    return {name: make_folder(root, name, sharpen=6.0) for name in ("tiny-llama", "tiny-qwen3")}


def _plain_greedy(folder, prompt, n, stop_ids=()):
    from plain.files import read_model_folder
    from plain.model import greedy_generate
    cfg, weights = read_model_folder(folder)
    return greedy_generate(cfg, weights, prompt, n, stop_ids)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_the_plain_implementation(folders, dtype):
    """configs[0]'s workload: prompts of 5, 9 and 13 tokens, 8 greedy steps."""
    from xeno_rt_b200 import GenerateRequest, Runtime
    folder = folders["tiny-llama"]
    prompts = random_prompts(256, [5, 9, 13], seed=3)
    session = Runtime.load(folder, dtype=dtype).new_session()
    requests = [GenerateRequest(p, max_tokens=8, temperature=0.0, repetition_penalty=1.0, stop_ids=()) for p in prompts]
    results, stats = session.generate_batch(requests)
    from plain.files import read_model_folder
    cfg, weights = read_model_folder(folder)
    for p, r in zip(prompts, results):
        if dtype == "float32":
            assert r.tokens == _plain_greedy(folder, p, 8)
        # every token is the plain model's best at its place unless the plain model's two best logits
        # lie within the precision's tolerance there; and the logits along the way are the plain ones
        want = check_greedy_tokens(cfg, weights, p, r.tokens, TOL[dtype])
        got = replay_logits(session.backend.engine, p, r.tokens[:-1])
        assert scaled_error(got, want[:len(got)]) < TOL[dtype]
        assert r.finish_reason == "length" and r.prompt_tokens == len(p)
    assert stats.tokens == 24 and stats.decode_steps == 7
    # one request through the single-request calls gives the same tokens as inside the batch
    assert session.generate(requests[1]) == results[1].tokens
    streamed = []
    session.generate_stream(requests[2], streamed.append)
    assert streamed == results[2].tokens


def test_stop_ids_context_limit_and_batches_in_a_row(folders):
    from xeno_rt_b200 import GenerateRequest, Runtime
    folder = folders["tiny-llama"]
    runtime = Runtime.load(folder, dtype="float32", cache_tokens=64 * 3, max_batch=2)
    session = runtime.new_session()
    prompts = random_prompts(256, [5, 9, 13, 4, 120], seed=5)
    free_run = [_plain_greedy(folder, p, 12) for p in prompts[:4]]
    stop = free_run[0][3]  # the fourth token of the first request ends it
    requests = [GenerateRequest(p, max_tokens=12, temperature=0.0, repetition_penalty=1.0, stop_ids=(stop,)) for p in prompts]
    results, stats = session.generate_batch(requests)
    assert stats.batches >= 3  # two sequences a batch at most
    for p, r, free in zip(prompts[:4], results, free_run):
        want = free[:free.index(stop)] if stop in free else free
        assert r.tokens == want
        assert r.finish_reason == ("stop" if stop in free else "length")
    # 120 prompt tokens of 128 positions: 8 tokens fit, then the context is full
    last = results[4]
    assert len(last.tokens) <= 8 and (last.finish_reason in ("context", "stop"))
    if last.finish_reason == "context":
        assert len(last.tokens) == 8
    session.backend.engine.cache.check()
    assert session.backend.engine.cache.blocks_free() == session.backend.engine.cache.n_blocks


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(folders):
    """configs[1]'s workload: prompts of 1, 7, 16 and 31 tokens, 12 steps at temperature 0.8."""
    from xeno_rt_b200 import GenerateRequest, Runtime
    session = Runtime.load(folders["tiny-qwen3"], dtype="float32").new_session()
    prompts = random_prompts(320, [1, 7, 16, 31], seed=8)
    mk = lambda: [GenerateRequest(p, max_tokens=12, temperature=0.8, seed=100 + i, stop_ids=()) for i, p in enumerate(prompts)]
    a, _ = session.generate_batch(mk())
    b, _ = session.generate_batch(mk())
    assert [r.tokens for r in a] == [r.tokens for r in b]
    alone = [session.generate(r) for r in mk()]
    assert alone == [r.tokens for r in a]  # a sequence's draws depend on its own seed only
    other, _ = session.generate_batch([GenerateRequest(p, max_tokens=12, temperature=0.8, seed=7 + i, stop_ids=())
                                       for i, p in enumerate(prompts)])
    assert [r.tokens for r in other] != [r.tokens for r in a]
    assert all(len(r.tokens) == 12 and all(0 <= t < 320 for t in r.tokens) for r in a)


def test_command_line(folders):
    folder = folders["tiny-llama"]
    prompts = random_prompts(256, [5, 9], seed=3)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "xrt"), "generate", "--model", folder, "--dtype", "float32",
           "--max-tokens", "6", "--temperature", "0", "--repetition-penalty", "1.0", "--stop-ids", "",
           "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids", ",".join(map(str, prompts[1]))]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    lines = [l for l in proc.stdout.strip().splitlines() if l]
    assert [list(map(int, l.split(","))) for l in lines] == [_plain_greedy(folder, p, 6) for p in prompts]
    assert "tokens in" in proc.stderr and "tok/s" in proc.stderr
    bad = subprocess.run(cmd[:4] + ["/nonexistent", "--prompt-ids", "1"], capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "no such file" in bad.stderr


def test_command_line_with_a_configuration_and_a_seed_as_the_model(tmp_path):
    """``--random-config cfg.json --seed-weights N`` draws on the device the weights that
    ``write_random_model`` writes for that seed: the command gives the tokens of ``--model`` on the
    written folder (stored as shards here, with stop ids in generation_config.json)."""
    from helpers import TINY_QWEN3
    from xeno_rt_b200.weights import write_random_model
    raw = dict(TINY_QWEN3, tie_word_embeddings=False)
    del raw["eos_token_id"]
    folder = write_random_model(str(tmp_path / "m"), raw, seed=21, dtype="bfloat16", shards=3)
    config_file = str(tmp_path / "cfg.json")
    json.dump(raw, open(config_file, "w"))
    prompts = random_prompts(320, [6, 11], seed=4)
    common = ["--dtype", "float32", "--max-tokens", "7", "--temperature", "0", "--repetition-penalty", "1.0",
              "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids", ",".join(map(str, prompts[1]))]
    xrt = [sys.executable, os.path.join(ROOT, "bin", "xrt"), "generate"]
    a = subprocess.run(xrt + ["--model", folder] + common, capture_output=True, text=True, timeout=600)
    b = subprocess.run(xrt + ["--random-config", config_file, "--seed-weights", "21"] + common,
                       capture_output=True, text=True, timeout=600)
    assert a.returncode == 0 and b.returncode == 0, a.stderr + b.stderr
    tokens = [list(map(int, l.split(","))) for l in a.stdout.strip().splitlines() if l]
    assert len(tokens) == 2 and all(len(t) == 7 for t in tokens) and a.stdout == b.stdout
    other = subprocess.run(xrt + ["--random-config", config_file, "--seed-weights", "22"] + common,
                           capture_output=True, text=True, timeout=600)
    assert other.returncode == 0 and other.stdout != a.stdout
    # the stop id of generation_config.json ends the first sequence where it would emit that id
    stop = tokens[0][3]
    json.dump({"eos_token_id": [stop]}, open(os.path.join(folder, "generation_config.json"), "w"))
    c = subprocess.run(xrt + ["--model", folder] + common, capture_output=True, text=True, timeout=600)
    assert c.returncode == 0 and c.stdout.splitlines()[0] == ",".join(map(str, tokens[0][:tokens[0].index(stop)]))
    # the two sources exclude each other, and one of them is needed
    both = subprocess.run(xrt + ["--model", folder, "--random-config", config_file] + common, capture_output=True, text=True)
    none = subprocess.run(xrt + common, capture_output=True, text=True)
    assert both.returncode == 2 and none.returncode == 2
    bad = subprocess.run(xrt + ["--random-config", str(tmp_path / "nope.json")] + common, capture_output=True, text=True)
    assert bad.returncode == 1 and "no such file" in bad.stderr


def _trace_steps(prompts, schedule):
    """Builds step records.  schedule 'whole': each request alone in one step; 'tail': whole minus
    32, then one by one; 'batch': all start together, then one token each, shorter ones end first."""
    steps, n = [], 0
    if schedule in ("whole", "tail"):
        for i, p in enumerate(prompts):
            head = len(p) if schedule == "whole" else max(1, len(p) - 32)
            cuts = [head] + [1] * (len(p) - head)
            at = 0
            for j, size in enumerate(cuts):
                last = j == len(cuts) - 1
                steps.append({"step": n, "entries": [{"id": f"r{i}", "tokens": p[at:at + size],
                                                      "want": list(range(size))}], "end": [f"r{i}"] if last else []})
                at += size
                n += 1
    else:
        heads = [max(1, len(p) - 8) for p in prompts]
        live = list(range(len(prompts)))
        ends = [i for i in live if heads[i] == len(prompts[i])]
        steps.append({"step": n, "entries": [{"id": f"r{i}", "tokens": prompts[i][:heads[i]],
                                              "want": list(range(heads[i]))} for i in live], "end": [f"r{i}" for i in ends]})
        n += 1
        live = [i for i in live if i not in ends]
        t = 0
        while live:
            ends = [i for i in live if heads[i] + t + 1 == len(prompts[i])]
            steps.append({"step": n, "entries": [{"id": f"r{i}", "tokens": [prompts[i][heads[i] + t]], "want": [0]}
                                                 for i in live], "end": [f"r{i}" for i in ends]})
            n += 1
            t += 1
            live = [i for i in live if i not in ends]
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_user_runs_it(folders, tmp_path, dtype):
    from plain.files import read_model_folder
    from plain.model import forward_logits
    folder = folders["tiny-qwen3"]
    cfg, weights = read_model_folder(folder)
    prompts = random_prompts(320, [1, 7, 16, 70], seed=2)
    refs = [forward_logits(cfg, weights, p) for p in prompts]
    for schedule in ("whole", "tail", "batch"):
        steps = _trace_steps(prompts, schedule)
        out = tmp_path / f"{dtype}-{schedule}"
        max_tokens = 64 * 5 if schedule == "batch" else 128
        proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out",
                               str(out), "--max-tokens", str(max_tokens)],
                              input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                              timeout=900)
        assert proc.returncode == 0, proc.stderr
        assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
        got = {f"r{i}": [] for i in range(len(prompts))}
        for s in steps:
            data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, 320)
            at = 0
            for e in s["entries"]:
                got[e["id"]].append(data[at:at + len(e["want"])])
                at += len(e["want"])
            assert at == data.shape[0]
        for i, r in enumerate(refs):
            assert scaled_error(np.concatenate(got[f"r{i}"]), r) < TOL[dtype], (schedule, i)
