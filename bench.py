#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama 3.2 1B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line. A "step" is one decode step of a batch of 8 sequences at
context 4,096 (every sequence's next token: model forward plus the greedy pick).
`value` is decoded tokens per second timed on the device with CUDA events;
`e2e` is the same through the Python entry point (Session.generate: host token
ids in, host token ids out, every step's inputs copied from pinned host memory
and every step's picked ids read back). Also on the line: the prefill of one
2,048-token prompt, the decode step's HBM roofline, decode at batch 1 and 64.

Weights are random (seeded), token ids synthetic; the reference publishes no
number for this configuration, so `vs_baseline` is null.
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

# The Llama 3.2 1B shape: the configuration the benchmark is quoted on
LLAMA_1B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=2048, intermediate_size=8192,
    num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
    vocab_size=128256, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)
FULL_LAYERS = 16
CONTEXT = 4096
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


def decode_bytes(config, layers, kv_lens, batch):
    """Bytes a decode step has to read: every weight it uses once, and the live requests' cache."""
    h, inter = config["hidden_size"], config["intermediate_size"]
    q = config["num_attention_heads"] * config["head_dim"]
    kv = config["num_key_value_heads"] * config["head_dim"]
    per_layer = (h * (q + 2 * kv) + q * h + 3 * h * inter) * 2 + 2 * h * 2
    weights = layers * per_layer + config["vocab_size"] * h * 2 + h * 2 + batch * h * 2
    cache = sum(kv_lens) * layers * 2 * kv * 2
    return weights + cache


def prefill_flops(config, layers, tokens):
    h, inter = config["hidden_size"], config["intermediate_size"]
    q = config["num_attention_heads"] * config["head_dim"]
    kv = config["num_key_value_heads"] * config["head_dim"]
    linear = 2 * tokens * (h * (q + 2 * kv) + q * h + 3 * h * inter)
    attention = 2 * tokens * tokens * config["head_dim"] * config["num_attention_heads"]  # causal QK^T + PV
    return layers * (linear + attention) + 2 * config["vocab_size"] * h


def correctness_gate(engine, model_dir) -> str:
    """Numbers are recorded only from a build whose logits agree with the plain implementation
    (the reference times only what passed its numerical gate, tools/benchmarks/run.py:130-145).
    The first two layers of the very weights that are timed, at their full widths, run in true
    float32 and in bfloat16, whole prompts, an unequal batch with decoding, and portions, against
    the plain CPU implementation under tests/. Takes some seconds; raises AssertionError."""
    tests = os.path.join(ROOT, "tests")
    if tests not in sys.path:
        sys.path.insert(0, tests)
    import helpers
    started = time.perf_counter()
    small = helpers.narrowed_copy(model_dir, model_dir + "_gate", min(2, json.load(
        open(os.path.join(model_dir, "config.json")))["num_hidden_layers"]))
    worst = {}
    for dtype in ("float32", "bfloat16"):
        worst[dtype] = helpers.parity_with_plain(engine, small, dtype, prompt_lengths=(150, 70, 9), decode_steps=3)
    return (f"passed: 2 layers at full widths vs the plain CPU implementation, worst error "
            f"{worst['float32']:.1e} (float32, allowed {helpers.TOLERANCE['float32']:.0e}) and "
            f"{worst['bfloat16']:.1e} (bfloat16, allowed {helpers.TOLERANCE['bfloat16']:.0e}) of the largest "
            f"logit, {time.perf_counter() - started:.0f} s")


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=16)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=FULL_LAYERS,
                        help="fewer layers than the configuration's 16 (named in config when used)")
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 / prefill extras")
    parser.add_argument("--no-gate", action="store_true",
                        help="skip the correctness gate (profiling runs only; the line then says so)")
    parser.add_argument("--only", choices=["prefill"], default=None,
                        help="run just this part (a small case for profiling); prints a shorter line")
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

    import numpy as np
    import torch
    from llama_rs_metal_b200 import Engine, GenerationOptions, Sampling
    from llama_rs_metal_b200.engine.batch import StepEntry
    from llama_rs_metal_b200.engine.session import write_random_model
    from llama_rs_metal_b200.kernels import ops

    peaks, peak_source = load_peaks()
    config = dict(LLAMA_1B, num_hidden_layers=args.layers)
    scratch = tempfile.mkdtemp(prefix="bench_model_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
    gate = "skipped (--no-gate)"
    try:
        write_random_model(scratch, config, seed=0, std=0.02)
        engine = Engine(0)
        if not args.no_gate:
            gate = correctness_gate(engine, scratch)   # raises: no numbers from a build that computes wrongly
        model = engine.load(scratch, dtype="bfloat16")
    except AssertionError as failure:
        print(f"correctness gate failed, nothing was timed: {failure}", file=sys.stderr)
        return 1
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
        shutil.rmtree(scratch + "_gate", ignore_errors=True)
    vocab = config["vocab_size"]
    rng = np.random.default_rng(0)

    def start_lengths(batch):
        """Each request's prompt is U[256, 2048] tokens and it generates to 4,096 in total; the
        timed steps run at the midpoint of that generation, where a step costs its average."""
        prompts = rng.integers(256, 2049, size=batch)
        return [int((p + CONTEXT) // 2) for p in prompts]

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
        session = model.session(context=CONTEXT, max_batch=batch)
        lengths = start_lengths(batch)
        slots = fill(session, lengths)
        tokens = rng.integers(0, vocab, size=(warmup + steps, batch))

        def one(i):
            logits = session.runner.step([StepEntry(s, [int(t)], (0,)) for s, t in zip(slots, tokens[i])], borrow=True)
            return logits.greedy_ids if hasattr(logits, "greedy_ids") else ops.argmax_rows(logits)
        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
            time.sleep(0.3)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph_launches = 0
        for i in range(warmup, warmup + steps):
            one(i)
            graph_launches += session.runner.last_launches
        end.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sample_clocks else None
        ms = begin.elapsed_time(end) / steps
        mid = [n + warmup + steps // 2 for n in lengths]
        launches = graph_launches           # the step's kernels, the greedy pick's two among them
        for s in slots:
            session.close_slot(s)
        return dict(ms=ms, tokens_per_s=batch * 1000.0 / ms, bytes=decode_bytes(config, args.layers, mid, batch),
                    kv_mean=sum(mid) / batch, launches=launches, clocks=clocks)

    def time_e2e(batch, steps):
        session = model.session(context=CONTEXT, max_batch=batch)
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
        return batch * steps / (done - first), (8 * batch + 1) * 4, batch * 4

    def time_prefill(tokens, reps=5):
        session = model.session(context=CONTEXT, max_batch=1)
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
        return statistics.median(times)

    if args.only == "prefill":
        ms = time_prefill(PREFILL_TOKENS, reps=max(1, args.steps))
        flops = prefill_flops(config, args.layers, PREFILL_TOKENS)
        print(json.dumps({"metric": "prefill tok/s, one 2048-token prompt", "value": round(PREFILL_TOKENS / (ms * 1e-3), 1),
                          "unit": "tok/s", "ms": round(ms, 3), "layers": args.layers,
                          "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4), "peaks": peak_source,
                          "gate": gate}))
        return 0
    main_run = time_decode(args.batch, args.steps, args.warmup, sample_clocks=True)
    e2e_value, h2d, d2h = time_e2e(args.batch, args.steps)
    achieved = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8, context 4096 (Llama 3.2 1B shape, random bf16 weights)",
        "value": round(main_run["tokens_per_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random-init weights",
        "impl": "ours", "gate": gate,
        "config": {
            "model": "Llama-3.2-1B shape", "layers": args.layers, "layers_of_config": FULL_LAYERS,
            "hidden": 2048, "heads": 32, "kv_heads": 8, "head_dim": 64, "intermediate": 8192,
            "vocab": 128256, "global_batch": args.batch, "seq_len": CONTEXT,
            "kv_len_mean": round(main_run["kv_mean"], 1), "prompt_lengths": "U[256,2048], generating to 4096; "
            "timed at each request's midpoint", "parallelism": "single GPU", "l2": "step reads > L2 (weights 2.5 GB)",
            "peaks": peak_source, "cuda_graph": True,
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(main_run["launches"]),
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
    }
    if not args.no_points:
        ms = time_prefill(PREFILL_TOKENS)
        flops = prefill_flops(config, args.layers, PREFILL_TOKENS)
        line["prefill"] = {"value": round(PREFILL_TOKENS / (ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                           "ms": round(ms, 3), "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
        points = {}
        for batch in (1, 64):
            run = time_decode(batch, max(16, args.steps // 2), 4)
            points[f"decode_b{batch}"] = round(run["tokens_per_s"], 1)
            points[f"decode_b{batch}_hbm_frac"] = round(run["bytes"] / (run["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
