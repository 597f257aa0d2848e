#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3-8B shape in bfloat16 with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens a second at batch 8 with every sequence near
the benchmark context (the timed steps end at that many positions): K decode steps, each the
model's step function plus sampling, timed on the device with CUDA events after W warm-up steps.
``e2e`` is the same through the Python entry point (``Session.generate_batch``): host token ids in,
host token ids out, with the copies that go with them every step.  ``prefill`` times one prompt of
2,048 tokens; ``roofline`` is the decode step's bytes (every weight it uses once, and the cache of
the live sequences) over its time, against the measured copy bandwidth; ``points`` are decode at
batch 1 and 64.  Weights are random N(0, 0.02) drawn on the device, prompts are uniform random
token ids.  The weights (about 15 GB read a step) are far larger than the L2 cache, so nothing is
flushed between steps.  More than one GPU is outside this library: it says so and exits with 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA3_8B = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 128256, "max_position_embeddings": 8192,
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
}
QWEN3_8B = dict(LLAMA3_8B, architectures=["Qwen3ForCausalLM"], vocab_size=151936, max_position_embeddings=40960,
                intermediate_size=12288, num_hidden_layers=36, rope_theta=1000000.0, rms_norm_eps=1e-6)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64)
SHAPES = {"llama3-8b": ("Llama-3-8B shape", LLAMA3_8B), "qwen3-8b": ("Qwen3-8B shape", QWEN3_8B),
          "qwen3-32b": ("Qwen3-32B shape", QWEN3_32B)}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PREFILL_TOKENS = 2048


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            raw = json.load(fh)
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 6:
                continue
            try:
                clocks.append(float(cells[0]))
                max_clock = float(cells[1])
            except ValueError:
                continue
            for name, cell in zip(names, cells[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def weight_bytes_per_step(cfg, n_layers: int) -> int:
    """Bytes of every weight a decode step reads once: the layers' matrices and norms, the final
    norm and the output matrix (of the embedding only the batch's rows are read)."""
    d, f, hd = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    qw, kw = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    per_layer = (qw + 2 * kw) * d + d * qw + 3 * f * d + 2 * d
    return 2 * (n_layers * per_layer + d + cfg["vocab_size"] * d)


def kv_bytes_per_token(cfg, n_layers: int) -> int:
    return 2 * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * n_layers


def prefill_flops(cfg, n_layers: int, tokens: int) -> float:
    d, f, hd = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    qw, kw = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    per_token = 2 * n_layers * ((qw + 2 * kw) * d + d * qw + 3 * f * d)
    attention = n_layers * 2 * 2 * qw * tokens * tokens / 2  # QK^T and PV over the causal half
    return tokens * per_token + attention + 2 * cfg["vocab_size"] * d  # the output matrix on one row


def fill_batch(engine, batch: int, length: int, vocab: int, chunk_tokens: int = 16384):
    """Opens ``batch`` slots and runs uniform random prompts of ``length`` tokens through the model
    in pieces, so that every sequence's cache holds real keys and values.  Returns the slots."""
    import torch
    from xeno_rt_b200.engine import StepEntry
    gen = torch.Generator().manual_seed(1234)
    slots = [engine.open_slot() for _ in range(batch)]
    per_step = max(1, chunk_tokens // max(1, min(length, 2048)))
    for lo in range(0, batch, per_step):
        group = slots[lo:lo + per_step]
        done = 0
        while done < length:
            size = min(2048, length - done)
            tokens = torch.randint(0, vocab, (len(group), size), generator=gen).tolist()
            engine.step([StepEntry(s, t, []) for s, t in zip(group, tokens)])
            done += size
    torch.cuda.synchronize()
    return slots


def time_decode(model, batch: int, context: int, steps: int, warmup: int, sample_clocks: bool = False):
    """Device-timed decode: sequences of ``context - steps - warmup`` tokens, then warm-up and K
    timed steps of step function + sampling, fed with the sampled ids."""
    import torch
    from xeno_rt_b200.csrc import ops
    from xeno_rt_b200.engine import Engine, StepEntry
    from xeno_rt_b200.sampling import Sampler, SamplerConfig

    vocab = model.vocab_size
    start_len = context - steps - warmup
    engine = Engine(model, batch * ((context + 63) // 64 * 64), max_slots=batch)
    sampler = Sampler(engine.cache, vocab)
    slots = fill_batch(engine, batch, start_len, vocab)
    sampler.begin(slots, list(range(batch)))
    row_slot = torch.tensor(slots, dtype=torch.int32, device=model.device)
    configs = [SamplerConfig(temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0)] * batch
    tokens = [[1]] * batch

    def one_step(tokens):
        logits = engine.step([StepEntry(s, t, [0]) for s, t in zip(slots, tokens)])
        return sampler.sample(logits, row_slot, configs)

    for _ in range(warmup):
        ids = one_step(tokens)
        tokens = [[t] for t in ids.tolist()]
    torch.cuda.synchronize()
    sampler_clocks = ClockSampler()
    if sample_clocks:
        sampler_clocks.start()
        time.sleep(0.3)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = ops.launch_count()
    torch.cuda.synchronize()
    begin.record()
    for _ in range(steps):
        ids = one_step(tokens)
        # the next step's ids are known on the host only after a read; the device-timed loop
        # feeds a fixed id instead so that nothing waits on the host (the model's work is the same)
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end)
    launches = ops.launch_count() - launches_before
    clocks = sampler_clocks.stop() if sample_clocks else None
    for s in slots:
        engine.close_slot(s)
    del engine
    torch.cuda.empty_cache()
    return {"ms_per_step": ms / steps, "tokens_per_s": batch * steps / (ms / 1e3), "launches": launches,
            "clocks": clocks, "mean_context": context - steps / 2}


def time_prefill(model, tokens: int, iters: int, warmup: int):
    import torch
    from xeno_rt_b200.engine import Engine, StepEntry
    engine = Engine(model, (tokens + 63) // 64 * 64, max_slots=1)
    prompt = torch.randint(0, model.vocab_size, (tokens,), generator=torch.Generator().manual_seed(7)).tolist()
    times = []
    for i in range(warmup + iters):
        slot = engine.open_slot()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        engine.step([StepEntry(slot, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(begin.elapsed_time(end))
        engine.close_slot(slot)
    del engine
    torch.cuda.empty_cache()
    return statistics.median(times)


def time_e2e(model, batch: int, context: int, steps: int):
    """Decode tokens a second through Session.generate_batch: host ids in, host ids out.  At least 256
    decode steps: the first tenths of a second after the prompts' step (32 k tokens at full power) run
    about 8 % slower than the steady state (measured: 5.09 ms a step right after it, 4.71 ms after a
    pause of two seconds), and 64 steps would lie wholly inside that."""
    steps = max(steps, 256)
    import torch
    from xeno_rt_b200 import GenerateRequest, Runtime
    runtime = Runtime(model, max_batch=batch)
    session = runtime.new_session()
    gen = torch.Generator().manual_seed(99)
    prompt_len = context - steps - 1
    prompts = torch.randint(0, model.vocab_size, (batch, prompt_len), generator=gen).tolist()
    requests = [GenerateRequest(p, max_tokens=steps + 1, temperature=0.0, repetition_penalty=1.0, stop_ids=())
                for p in prompts]
    session.generate_batch(requests)  # warm-up: the decode graphs of these shapes are captured once
    results, stats = session.generate_batch(requests)
    lay_ints = 3 * batch + 3 * batch + 1
    out = {"value": stats.decode_tokens_per_second, "unit": "tokens/s", "h2d_bytes_per_step": 4 * lay_ints + 16 * batch,
           "d2h_bytes_per_step": 4 * batch, "decode_steps": stats.decode_steps,
           "prefill_s": round(stats.prefill_seconds, 4)}
    session.backend = None
    torch.cuda.empty_cache()
    return out


WORKLOADS = {
    # name: (shape, prompts, shortest, longest prompt, decode steps)
    "config3": ("qwen3-8b", 16, 64, 2048, 256),
    "config4": ("qwen3-32b", 8, 2048, 2048, 512),
}


def run_workload(args) -> int:
    """The two stated workloads beside the headline: 16 prompts of seeded uniform lengths in [64, 2048] in
    one step of unequal lengths, then 256 decode steps (Qwen3-8B shape); 8 prompts of 2,048 tokens, then 512
    decode steps (Qwen3-32B shape).  Both through ``Session.generate_batch`` (host token ids in and out,
    host clock), run three times: the first run captures the decode graphs, the second settles the
    allocator's blocks (a prompt step that has to ask the driver for memory takes up to twice as long),
    the third is timed.  Prints one JSON line with the prompts'
    tokens a second against the FLOP of the drawn lengths and the decoded tokens a second against the
    bytes a step has to read (every weight once, the cache of the live sequences at their mean length)."""
    import torch
    import xeno_rt_b200  # noqa: F401
    from xeno_rt_b200 import GenerateRequest, Runtime
    from xeno_rt_b200.engine import Model

    shape, n_prompts, shortest, longest, steps = WORKLOADS[args.workload]
    if args.steps != 64:  # the default of --steps belongs to the headline run
        steps = args.steps
    shape_name, shape_cfg = SHAPES[shape]
    cfg = dict(shape_cfg)
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = n_layers = args.layers or full_layers
    pk = peaks()
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    gen = torch.Generator().manual_seed(2024)
    lengths = torch.randint(shortest, longest + 1, (n_prompts,), generator=gen).tolist()
    prompts = [torch.randint(0, model.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    session = Runtime(model, max_batch=n_prompts).new_session()
    make = lambda: [GenerateRequest(p, max_tokens=steps + 1, temperature=0.0, repetition_penalty=1.0, stop_ids=())
                    for p in prompts]
    for _ in range(2):  # the first run captures the decode graphs, the second settles the allocator's blocks
        session.generate_batch(make())
    torch.cuda.synchronize()
    clocks = ClockSampler()
    clocks.start()
    results, stats = session.generate_batch(make())
    clock_record = clocks.stop()
    assert all(len(r.tokens) == steps + 1 for r in results)
    d, f, hd = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    qw, kw = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    per_token = 2 * n_layers * ((qw + 2 * kw) * d + d * qw + 3 * f * d)
    flops = (sum(lengths) * per_token + sum(n_layers * 2 * qw * n * n for n in lengths)
             + n_prompts * 2 * cfg["vocab_size"] * d)
    decode_s = stats.seconds - stats.prefill_seconds
    mean_tokens = sum(n + 1 + steps / 2 for n in lengths)
    bytes_step = weight_bytes_per_step(cfg, n_layers) + mean_tokens * kv_bytes_per_token(cfg, n_layers)
    achieved = bytes_step * stats.decode_steps / decode_s / 1e9
    print(json.dumps({
        "workload": args.workload, "impl": "ours", "model": shape_name, "layers": n_layers, "layers_of_model": full_layers,
        "prompts": n_prompts, "prompt_tokens": sum(lengths), "shortest": min(lengths), "longest": max(lengths),
        "decode_steps": stats.decode_steps, "through": "Session.generate_batch, host clock", "peaks": pk["source"],
        "prefill": {"value": round(sum(lengths) / stats.prefill_seconds, 1), "unit": "tokens/s",
                    "ms": round(stats.prefill_seconds * 1e3, 2), "tflops": round(flops / stats.prefill_seconds / 1e12, 1),
                    "frac": round(flops / stats.prefill_seconds / (pk["bf16_tflops"] * 1e12), 4)},
        "decode": {"value": round(stats.decode_tokens_per_second, 1), "unit": "tokens/s",
                   "ms_per_step": round(decode_s / stats.decode_steps * 1e3, 4), "achieved_gbs": round(achieved, 1),
                   "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clock_record}))
    return 0


def run_ours(args) -> int:
    import torch
    import xeno_rt_b200  # noqa: F401
    from xeno_rt_b200.engine import Model

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: bench.py needs a B200"}))
        return 1
    if apply_tuning(args):
        return 2
    shape_name, shape_cfg = SHAPES[args.shape]
    cfg = dict(shape_cfg)
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or full_layers
    # the positions the run needs (rotary tables are computed, not stored: only the cache's limit moves)
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], args.context, args.prefill_tokens)
    n_layers = cfg["num_hidden_layers"]
    pk = peaks()
    t0 = time.time()
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    torch.cuda.synchronize()
    setup_s = time.time() - t0
    return run_timed(args, model, cfg, shape_name, full_layers, n_layers, pk, setup_s)


def run_attention_only(args) -> int:
    """--only attention: the decode attention kernel alone for --batch sequences of --context keys with the shape's
    heads, --window keys visible (0: all), 20 launches back to back in a CUDA graph; one small JSON line.
    --splits-from context cuts a windowed layer's splits as a layer without a window would have them."""
    import math
    import torch
    import xeno_rt_b200  # noqa: F401
    from xeno_rt_b200.cache import BLOCK_TOKENS
    from xeno_rt_b200.csrc import ops
    from xeno_rt_b200.parts.attention_bf16 import FUSED_COMBINE_MAX, decode_split, visible_span

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: bench.py needs a B200"}))
        return 1
    if apply_tuning(args):
        return 2
    cfg = SHAPES[args.shape][1]
    heads, kv_heads = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    head_dim = cfg.get("head_dim", cfg["hidden_size"] // heads)
    dev = torch.device("cuda:0")
    batch, context, window = args.batch, args.context, args.window
    blocks_each = -(-context // BLOCK_TOKENS)
    k = torch.randn(batch * blocks_each + 1, kv_heads, BLOCK_TOKENS, head_dim, device=dev, dtype=torch.bfloat16)
    v = torch.randn_like(k)
    table = torch.arange(1, 1 + batch * blocks_each, dtype=torch.int32, device=dev).reshape(batch, blocks_each)
    table = torch.cat([torch.full((1, blocks_each), -1, dtype=torch.int32, device=dev), table])  # slot 0 stays empty
    q = torch.randn(batch, heads * head_dim, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
    slot = torch.arange(1, batch + 1, dtype=torch.int32, device=dev)
    span = visible_span(context, window) if args.splits_from == "window" else context
    chunk, n_splits = decode_split(batch, kv_heads, span, ops.device_state(dev)[2])
    fused = batch * kv_heads <= FUSED_COMBINE_MAX

    def launch():
        ops.attention_decode(out, q, k, v, slot, pos, table, heads, kv_heads, head_dim, 1 / math.sqrt(head_dim), window,
                             chunk, n_splits, fused=fused)

    for _ in range(max(3, args.warmup)):
        launch()
    graph, repeats = torch.cuda.CUDAGraph(), 20
    with torch.cuda.graph(graph):
        for _ in range(repeats):
            launch()
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    stop.record()
    torch.cuda.synchronize()
    ops.check_error_flag(dev)
    us = start.elapsed_time(stop) / repeats * 1000
    keys = min(context, window + BLOCK_TOKENS - 1) if window > 0 else context
    read = batch * keys * kv_heads * head_dim * 2 * 2
    print(json.dumps({"only": "attention", "us": round(us, 2), "batch": batch, "context": context, "window": window,
                      "keys_a_split": chunk, "splits": n_splits, "heads": heads, "kv_heads": kv_heads,
                      "head_dim": head_dim, "gbs_upper": round(read / us / 1000, 1),
                      "flush": "none: launches back to back; cache of %d MB" % (2 * k.numel() * 2 // 2**20)}))
    return 0


def apply_tuning(args) -> int:
    """--tuning KEY=VALUE,... onto the kernels' tuning; returns 2 after a message if a key is unknown."""
    if args.tuning:
        import dataclasses
        import xeno_rt_b200  # noqa: F401
        from xeno_rt_b200.csrc import ops
        fields = {f.name: f.type for f in dataclasses.fields(ops.Tuning)}
        changes = {}
        for item in args.tuning.split(","):
            key, _, value = item.partition("=")
            if key not in fields:
                print(f"bench.py: --tuning {key!r} is not one of {sorted(fields)}")
                return 2
            current = getattr(ops.Tuning(), key)
            changes[key] = (value.lower() in ("1", "true", "on")) if isinstance(current, bool) else type(current)(
                int(value, 0) if isinstance(current, int) else value)
        ops.set_tuning(dataclasses.replace(ops.tuning(), **changes))
    return 0


def run_timed(args, model, cfg, shape_name, full_layers, n_layers, pk, setup_s) -> int:
    import torch

    if args.only == "prefill":  # a short run for profiling: one prompt (of 2,048 tokens unless --prefill-tokens says otherwise)
        prefill_ms = time_prefill(model, args.prefill_tokens, iters=max(1, args.steps), warmup=args.warmup)
        flops = prefill_flops(cfg, n_layers, args.prefill_tokens)
        print(json.dumps({"only": "prefill", "ms": round(prefill_ms, 3), "tokens": args.prefill_tokens, "layers": n_layers,
                          "tokens_per_s": round(args.prefill_tokens / (prefill_ms / 1e3), 1),
                          "tflops": round(flops / (prefill_ms / 1e3) / 1e12, 1)}))
        return 0
    main = time_decode(model, args.batch, args.context, args.steps, args.warmup, sample_clocks=True)
    bytes_step = weight_bytes_per_step(cfg, n_layers) + args.batch * main["mean_context"] * kv_bytes_per_token(cfg, n_layers)
    achieved = bytes_step / (main["ms_per_step"] / 1e3) / 1e9
    points = {}
    if args.only == "decode":  # a short run for profiling: the headline step alone
        print(json.dumps({"only": "decode", "ms_per_step": round(main["ms_per_step"], 4),
                          "tokens_per_s": round(main["tokens_per_s"], 1), "roofline_gbs": round(achieved, 1),
                          "layers": n_layers, "batch": args.batch, "context": args.context}))
        return 0
    for b in (1, 64):
        r = time_decode(model, b, args.context, max(8, args.steps // 2), args.warmup)
        points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
    prefill_ms = time_prefill(model, PREFILL_TOKENS, iters=9, warmup=max(3, args.warmup // 2))
    flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    e2e = time_e2e(model, args.batch, args.context, args.steps)

    line = {
        "metric": f"decode tok/s @ batch {args.batch} ({shape_name.replace(' shape', '')} bf16, context {args.context})", "value": round(main["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        "impl": "ours",
        "config": {"model": shape_name, "layers": n_layers, "layers_of_model": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": args.context, "parallelism": "none (1 GPU)",
                   "cache_block_tokens": 64, "l2": "inputs larger than L2 (15 GB of weights a step), no flush",
                   "peaks": pk["source"], "setup_s": round(setup_s, 1)},
        "e2e": e2e,
        "gpu_launches": main["launches"],
        "clocks": main["clocks"],
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0 = all)")
    parser.add_argument("--shape", default="llama3-8b", choices=sorted(SHAPES),
                        help="the model shape to time (the default is the headline configuration)")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                        help="prompt length of --only prefill (the full line always uses 2,048)")
    parser.add_argument("--workload", default="", choices=["", *sorted(WORKLOADS)],
                        help="one of the two further workloads instead of the headline line (16 unequal prompts then "
                             "256 decode steps at the Qwen3-8B shape; 8 x 2,048 then 512 steps at the Qwen3-32B shape)")
    parser.add_argument("--tuning", default="", metavar="KEY=VALUE[,KEY=VALUE...]",
                        help="kernel variants to force, as fields of xeno_rt_b200.csrc.ops.Tuning (for comparisons)")
    parser.add_argument("--only", default="all", choices=["all", "decode", "prefill", "attention"],
                        help="a short run of one part, for profiling; prints its own small JSON line "
                             "(attention: the decode attention kernel alone)")
    parser.add_argument("--window", type=int, default=0, help="--only attention: keys a token sees (0 = all)")
    parser.add_argument("--splits-from", default="window", choices=["window", "context"],
                        help="--only attention with a window: cut the splits from the window's span (what the engine "
                             "does) or from the whole context (what a layer without a window gets)")
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (no setup.py or pyproject.toml, pip refuses it), there is "
                          "no cargo or rustc here, and its model path is CPU-only and takes GGUF-quantised weights only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3 and args.only == "all":
        args.warmup = 3
    if args.only == "attention":
        return run_attention_only(args)
    if args.workload:
        apply_tuning(args)
        return run_workload(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
