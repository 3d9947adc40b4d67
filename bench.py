#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama 3 shapes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 1b|3b|8b] [--profile]

Prints ONE JSON line. A "step" is one decode step of a batch of sequences (every
sequence's next token: model forward plus the greedy pick, as generation runs it).
`value` is decoded tokens per second timed on the device with CUDA events;
`e2e` is the same through the Python entry point (Session.generate: host token
ids in, host token ids out, every step's inputs copied from pinned host memory
and every step's picked ids read back). Also on the line: the prefill of one
2,048-token prompt, the decode step's HBM roofline, decode at other batch sizes,
and the plain CPU implementation's speed on a tiny configuration beside the
engine's (what the kernels are worth against the formulas run as written).

The default is the Llama 3.2 1B shape at context 4,096 and batch 8; `--shape 3b`
and `--shape 8b` run the other shapes the baseline lists (16 unequal prompts at
the 3B shape; context 8,192 and batches 1/8/32 at the 8B shape).

Before anything is timed, the build's logits are compared with the plain
implementation at the shape's full widths (see correctness_gate); a build that
fails prints no number. Weights are random (seeded), token ids synthetic; the
reference publishes no number for these configurations, so `vs_baseline` is null.
"""
import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def llama(hidden, inter, layers, heads, kv_heads, head_dim, factor, tied):
    return dict(
        architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=hidden, intermediate_size=inter,
        num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
        vocab_size=128256, rope_theta=500000.0,
        rope_scaling=dict(rope_type="llama3", factor=factor, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192),
        rms_norm_eps=1e-5, tie_word_embeddings=tied, max_position_embeddings=131072)


# name -> the shape's config.json, the benchmark context, the batch of the main number, the other
# batches measured, and how the requests' lengths are drawn
SHAPES = {
    "1b": dict(name="Llama-3.2-1B shape", config=llama(2048, 8192, 16, 32, 8, 64, 32.0, True), context=4096,
               batch=8, points=(1, 64), prompts=(256, 2048), to_context=True),
    "3b": dict(name="Llama-3.2-3B shape", config=llama(3072, 8192, 28, 24, 8, 128, 32.0, True), context=8192,
               batch=16, points=(), prompts=(64, 4096), to_context=False),
    "8b": dict(name="Llama-3.1-8B shape", config=llama(4096, 14336, 32, 32, 8, 128, 8.0, False), context=8192,
               batch=8, points=(1, 32), prompts=(256, 2048), to_context=True),
}
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                data = json.load(handle)
            return dict(hbm_gbs=float(data["hbm_gbs"]), bf16_tflops=float(data["bf16_tflops"]),
                        bf16_tflops_sustained=float(data.get("bf16_tflops_sustained", data["bf16_tflops"]))), "measured"
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi's SM clock and throttle reasons, sampled while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([f.strip() for f in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for fields in self.samples:
            if len(fields) < 7:
                continue
            try:
                clocks.append(int(float(fields[0])))
                max_clock = int(float(fields[1]))
            except ValueError:
                continue
            for name, flag in zip(names, fields[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=int(statistics.median(clocks)) if clocks else None, sm_max_mhz=max_clock,
                    reasons=sorted(reasons), samples=len(clocks))


def decode_bytes(config, kv_lens, batch):
    """Bytes a decode step has to read: every weight it uses once, and the live requests' cache."""
    h, inter, layers = config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]
    q = config["num_attention_heads"] * config["head_dim"]
    kv = config["num_key_value_heads"] * config["head_dim"]
    per_layer = (h * (q + 2 * kv) + q * h + 3 * h * inter) * 2 + 2 * h * 2
    weights = layers * per_layer + config["vocab_size"] * h * 2 + h * 2 + batch * h * 2
    cache = sum(kv_lens) * layers * 2 * kv * 2
    return weights + cache


def prefill_flops(config, tokens):
    h, inter, layers = config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]
    q = config["num_attention_heads"] * config["head_dim"]
    kv = config["num_key_value_heads"] * config["head_dim"]
    linear = 2 * tokens * (h * (q + 2 * kv) + q * h + 3 * h * inter)
    attention = 2 * tokens * tokens * config["head_dim"] * config["num_attention_heads"]  # causal QK^T + PV
    return layers * (linear + attention) + 2 * config["vocab_size"] * h


def tests_on_path():
    tests = os.path.join(ROOT, "tests")
    if tests not in sys.path:
        sys.path.insert(0, tests)


def correctness_gate(engine, config) -> str:
    """Numbers are recorded only from a build whose logits agree with the plain implementation
    (the reference times only what passed its numerical gate, tools/benchmarks/run.py:130-145).
    A model with the first two layers of the shape that is timed, at its full widths, is written
    as a folder and run in true float32 and in bfloat16: whole prompts, an unequal batch with
    decoding, and portions, against the plain CPU implementation under tests/. Some seconds;
    raises AssertionError."""
    tests_on_path()
    import helpers
    from llama_rs_metal_b200.engine.session import write_random_model
    started = time.perf_counter()
    folder = tempfile.mkdtemp(prefix="bench_gate_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
    try:
        write_random_model(folder, dict(config, num_hidden_layers=min(2, config["num_hidden_layers"])), seed=0, std=0.02)
        worst = {dtype: helpers.parity_with_plain(engine, folder, dtype, prompt_lengths=(150, 70, 9), decode_steps=3)
                 for dtype in ("float32", "bfloat16")}
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    return (f"passed: 2 layers at full widths vs the plain CPU implementation, worst error "
            f"{worst['float32']:.1e} (float32, allowed {helpers.TOLERANCE['float32']:.0e}) and "
            f"{worst['bfloat16']:.1e} (bfloat16, allowed {helpers.TOLERANCE['bfloat16']:.0e}) of the largest "
            f"logit, {time.perf_counter() - started:.0f} s")


def plain_cpu_point(engine):
    """The plain implementation on the CPU and the engine on the GPU, same tiny model (configuration A
    of the tests, float32), same greedy workload: tokens per second of each."""
    tests_on_path()
    import helpers
    import plain_llama
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    folder = tempfile.mkdtemp(prefix="bench_tiny_")
    try:
        helpers.make_model_dir(folder, "A")
        config, tensors = plain_llama.read_model(folder)
        prompts = [helpers.random_tokens(1 + i, n, 256) for i, n in enumerate((5, 11, 17))]
        steps = 8
        started = time.perf_counter()
        want = [plain_llama.greedy_continue(config, tensors, p, steps) for p in prompts]
        cpu = len(prompts) * steps / (time.perf_counter() - started)
        session = engine.load(folder, dtype="float32").session(context=128, max_batch=3)
        options = GenerationOptions(max_tokens=steps, sampling=Sampling(temperature=0.0))
        for _ in range(2):  # warm-up: the prompt step's graph is captured the second time its shape comes
            session.generate(prompts, options, stop_token_ids=())
        started = time.perf_counter()
        got = session.generate(prompts, options, stop_token_ids=())
        gpu = len(prompts) * steps / (time.perf_counter() - started)
        same = sum(a == b for r, w in zip(got, want) for a, b in zip(r.tokens, w))
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    return {"plain_cpu_tiny_a_tok_s": round(cpu, 1), "engine_tiny_a_tok_s": round(gpu, 1),
            "tiny_a_tokens_equal": f"{same}/{len(prompts) * steps}"}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=16)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--shape", default="1b", choices=sorted(SHAPES))
    parser.add_argument("--batch", type=int, default=None, help="batch of the main number (default: the shape's)")
    parser.add_argument("--context", type=int, default=None,
                        help="another context length than the shape's (further sizes: the requests then generate "
                             "to this length and are timed at their midpoints)")
    parser.add_argument("--prefill-tokens", type=int, default=None,
                        help="length of the prompt of the prefill figure (default 2,048), up to the context")
    parser.add_argument("--layers", type=int, default=None,
                        help="fewer layers than the shape has (both numbers are named in config)")
    parser.add_argument("--no-points", action="store_true", help="skip the other batch sizes, prefill and CPU extras")
    parser.add_argument("--no-gate", action="store_true",
                        help="skip the correctness gate (profiling runs only; the line then says so)")
    parser.add_argument("--only", choices=["prefill"], default=None,
                        help="run just this part (a small case for profiling); prints a shorter line")
    parser.add_argument("--timeline", choices=["decode", "prefill"], default=None,
                        help="print, to stderr, when each kernel of one step started and ended on the device (the "
                             "CUPTI activity trace that torch.profiler records: kernels inside a replayed graph and "
                             "their overlap under programmatic launch show as they ran); times nothing else")
    parser.add_argument("--profile", action="store_true",
                        help="time every kernel launch (LRM_PROFILE=1) and print the table to stderr; the "
                             "line's numbers are then those of unfused, uncaptured launches")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference runs only through Apple's Metal API on macOS (crates/metal-backend/"
                          "src/lib.rs:16-21) and is a Rust workspace; neither Metal nor cargo exists on this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is outside this library's scope (single-GPU engine)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.profile:
        os.environ["LRM_PROFILE"] = "1"

    import numpy as np
    import torch
    from llama_rs_metal_b200 import Engine, GenerationOptions, Sampling
    from llama_rs_metal_b200.engine.batch import StepEntry
    from llama_rs_metal_b200.sampling.device import DevicePick

    shape = SHAPES[args.shape]
    full_layers = shape["config"]["num_hidden_layers"]
    layers = args.layers or full_layers
    config = dict(shape["config"], num_hidden_layers=layers)
    context, batch_main = args.context or shape["context"], args.batch or shape["batch"]
    prefill_tokens = min(args.prefill_tokens or PREFILL_TOKENS, context)
    peaks, peak_source = load_peaks()
    engine = Engine(0)
    gate = "skipped (--no-gate)"
    if not args.no_gate:
        try:
            gate = correctness_gate(engine, config)   # raises: no numbers from a build that computes wrongly
        except AssertionError as failure:
            print(f"correctness gate failed, nothing was timed: {failure}", file=sys.stderr)
            return 1
    model = engine.random(config, seed=0, std=0.02)   # drawn on the device: seconds even at the 8B shape
    vocab = config["vocab_size"]
    rng = np.random.default_rng(0)
    low, high = shape["prompts"]

    def start_lengths(batch):
        """Prompt lengths are U[low, high]. Where requests generate to the full context, the timed
        steps run at the midpoint of that generation (where a step costs its average); where a fixed
        number of steps follows the prompts, they start right after the prompts."""
        # The same batch gets the same lengths wherever it is timed (on the device, end to end); the
        # seed is one at which the sample means of the batches timed here lie within 1.5 % of the
        # distributions' means, so that no figure is flattered by a batch of short prompts.
        prompts = np.random.default_rng(7820 + batch).integers(low, high + 1, size=batch)
        if shape["to_context"]:
            return [int((p + context) // 2) for p in prompts]
        return [int(p) for p in prompts]

    def fill(session, lengths):
        """Open a slot per sequence and run its tokens up to `lengths` through real prefill steps."""
        slots = []
        for i in range(0, len(lengths), 8):
            group = lengths[i:i + 8]
            entries = []
            for n in group:
                slot = session.open_slot()
                slots.append(slot)
                entries.append(StepEntry(slot, rng.integers(0, vocab, size=n).tolist(), ()))
            session.step(entries)
        return slots

    def time_decode(batch, steps, warmup, sample_clocks=False):
        session = model.session(context=context, max_batch=batch)
        lengths = start_lengths(batch)
        slots = fill(session, lengths)
        tokens = rng.integers(0, vocab, size=(warmup + steps, batch))
        greedy = DevicePick(None, 0, [0] * batch)

        def one(i):  # the step generation runs: tokens in, the chosen tokens out, no logits kept
            if args.profile:  # uncaptured, so that every launch passes through its timed wrapper
                return session.runner.step_pick([StepEntry(s, [int(t)], (0,)) for s, t in zip(slots, tokens[i])], greedy)
            return session.runner.decode_ahead(slots, tokens[i].tolist(), None, greedy)
        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
            time.sleep(0.3)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        launches = 0
        for i in range(warmup, warmup + steps):
            one(i)
            launches += session.runner.last_launches
        end.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sample_clocks else None
        session.runner.check_device_status()
        ms = begin.elapsed_time(end) / steps
        mid = [n + warmup + steps // 2 for n in lengths]
        for s in slots:
            session.close_slot(s)
        return dict(ms=ms, tokens_per_s=batch * 1000.0 / ms, bytes=decode_bytes(config, mid, batch),
                    kv_mean=sum(mid) / batch, launches=launches, clocks=clocks)

    def time_e2e(batch, steps):
        session = model.session(context=context, max_batch=batch)
        prompts = [rng.integers(0, vocab, size=n).tolist() for n in start_lengths(batch)]
        options = GenerationOptions(max_tokens=steps + 1, sampling=Sampling(temperature=0.0))
        session.generate(prompts, options, stop_token_ids=())   # warm-up: the same steps once, untimed
        torch.cuda.synchronize()
        stamps = []
        session.generate(prompts, options, stop_token_ids=(),
                         on_token=lambda request, token: stamps.append(time.perf_counter()))
        torch.cuda.synchronize()
        done = time.perf_counter()
        first = stamps[batch - 1]           # every request's first token (the prefill's) is out
        groups = len(session.cache.kv_groups)
        return batch * steps / (done - first), ((8 + groups) * batch + 1) * 4, batch * 4

    def time_prefill(tokens, reps=9):
        session = model.session(context=context, max_batch=1)
        ids = rng.integers(0, vocab, size=tokens).tolist()
        times = []
        for rep in range(reps + 2):
            slot = session.open_slot()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            session.runner.step([StepEntry(slot, ids, (tokens - 1,))])
            end.record()
            torch.cuda.synchronize()
            session.close_slot(slot)
            if rep >= 2:
                times.append(begin.elapsed_time(end))
        session.runner.check_device_status()
        return statistics.median(times)

    def timeline(what):
        """One step under the activity trace: per kernel its start since the step's first kernel, its
        duration and the gap to the kernel before it (negative: they overlapped), then sums by kernel."""
        from torch.profiler import ProfilerActivity, profile as activity_trace
        if what == "decode":
            session = model.session(context=context, max_batch=batch_main)
            slots = fill(session, start_lengths(batch_main))
            tokens = rng.integers(0, vocab, size=(24, batch_main))
            greedy = DevicePick(None, 0, [0] * batch_main)
            run = lambda i: session.runner.decode_ahead(slots, tokens[i].tolist(), None, greedy)
            warm, traced = range(16), range(16, 20)
        else:
            session = model.session(context=context, max_batch=1)
            ids = rng.integers(0, vocab, size=prefill_tokens).tolist()

            def run(i):
                slot = session.open_slot()
                session.runner.step([StepEntry(slot, ids, (prefill_tokens - 1,))])
                torch.cuda.synchronize()
                session.close_slot(slot)
            warm, traced = range(4), range(4, 5)
        for i in warm:
            run(i)
        torch.cuda.synchronize()
        with activity_trace(activities=[ProfilerActivity.CUDA]) as trace:
            for i in traced:
                run(i)
            torch.cuda.synchronize()
        events = sorted((e for e in trace.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                        key=lambda e: e.time_range.start)
        first = max(i for i, e in enumerate(events) if "embed_rows" in e.name)   # the last step traced
        step = events[first:]
        origin, before = step[0].time_range.start, step[0].time_range.start
        print(f"{'start us':>9s} {'us':>7s} {'gap us':>7s}  kernel", file=sys.stderr)
        for e in step:
            begin, end = e.time_range.start, e.time_range.end
            print(f"{begin - origin:9.1f} {end - begin:7.1f} {begin - before:7.1f}  {e.name[:110]}", file=sys.stderr)
            before = end
        totals = {}
        for e in step:
            calls, us = totals.get(e.name[:90], (0, 0.0))
            totals[e.name[:90]] = (calls + 1, us + e.time_range.end - e.time_range.start)
        print(f"one {what} step: {step[-1].time_range.end - origin:.1f} us from first start to last end, "
              f"{len(step)} kernels; sums of durations (overlapping kernels count twice):", file=sys.stderr)
        for name, (calls, us) in sorted(totals.items(), key=lambda item: -item[1][1]):
            print(f"{us:9.1f} us {calls:4d} x  {name}", file=sys.stderr)

    if args.timeline:
        timeline(args.timeline)
        print(json.dumps({"timeline": args.timeline, "shape": shape["name"], "layers": layers, "gate": gate,
                          "note": "the table is on stderr; nothing was timed for the record"}))
        return 0
    if args.only == "prefill":
        ms = time_prefill(prefill_tokens, reps=max(1, args.steps))
        flops = prefill_flops(config, prefill_tokens)
        print(json.dumps({"metric": f"prefill tok/s, one {prefill_tokens}-token prompt",
                          "value": round(prefill_tokens / (ms * 1e-3), 1),
                          "unit": "tok/s", "ms": round(ms, 3), "layers": layers, "shape": shape["name"],
                          "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4), "peaks": peak_source,
                          "gate": gate}))
        return 0
    steps = args.steps
    if not shape["to_context"]:
        steps = min(steps, 256)  # the 3B workload is 256 decode steps after the prompts
    main_run = time_decode(batch_main, steps, args.warmup, sample_clocks=True)
    e2e_value, h2d, d2h = time_e2e(batch_main, steps)
    achieved = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
    cfg = config
    lengths_note = (f"U[{low},{high}], generating to {context}; timed at each request's midpoint" if shape["to_context"]
                    else f"U[{low},{high}], then {steps} decode steps")
    line = {
        "metric": f"decode tok/s at batch {batch_main}, context {context} ({shape['name']}, random bf16 weights)",
        "value": round(main_run["tokens_per_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random-init weights",
        "impl": "ours", "gate": gate,
        "config": {
            "model": shape["name"], "layers": layers, "layers_of_config": full_layers,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied_head": cfg["tie_word_embeddings"], "global_batch": batch_main, "seq_len": context,
            "kv_len_mean": round(main_run["kv_mean"], 1), "prompt_lengths": lengths_note,
            "parallelism": "single GPU", "l2": "step reads > L2 (weights alone are GBs)",
            "peaks": peak_source, "cuda_graph": not args.profile,
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(main_run["launches"]),
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
    }
    if not args.no_points:
        ms = time_prefill(prefill_tokens)
        flops = prefill_flops(config, prefill_tokens)
        line["prefill"] = {"value": round(prefill_tokens / (ms * 1e-3), 1), "tokens": prefill_tokens,
                           "ms": round(ms, 3), "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
        points = {}
        for batch in shape["points"]:
            run = time_decode(batch, max(16, steps // 2), 4)
            points[f"decode_b{batch}"] = round(run["tokens_per_s"], 1)
            points[f"decode_b{batch}_hbm_frac"] = round(run["bytes"] / (run["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
        for tokens in (128, 512):  # short prompts: what one request waits for before its first token
            points[f"prefill_{tokens}_ms"] = round(time_prefill(tokens), 3)
        points.update(plain_cpu_point(engine))
        line["points"] = points
    print(json.dumps(line))
    if args.profile:
        from llama_rs_metal_b200.kernels import profile
        profile.report()
        profile.reset()
    return 0


if __name__ == "__main__":
    sys.exit(main())
