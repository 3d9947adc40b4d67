"""Shared by the tests: the tiny configurations, request sets, tolerances, trace replay driver."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny Llama configurations that differ in every size and option, and a third with
# awkward sizes (width 68 is no multiple of 8, vocabulary 307 is prime, 100 is no multiple of 8).
TINY = {
    "A": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=64,
                    intermediate_size=192, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=16, vocab_size=256, rope_theta=10000.0,
                    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=128),
        seed=0, std=0.02, norm_mean=1.0, norm_std=0.0),
    "B": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=96,
                    intermediate_size=256, num_hidden_layers=3, num_attention_heads=3,
                    num_key_value_heads=1, head_dim=32, vocab_size=512, rope_theta=500000.0,
                    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                      high_freq_factor=4.0, original_max_position_embeddings=64),
                    rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256),
        seed=7, std=0.05, norm_mean=1.0, norm_std=0.1),
    "C": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=68,
                    intermediate_size=100, num_hidden_layers=1, num_attention_heads=6,
                    num_key_value_heads=3, head_dim=48, vocab_size=307, rope_theta=1000.0,
                    rope_scaling=dict(rope_type="linear", factor=2.0),
                    rms_norm_eps=1e-4, tie_word_embeddings=False, max_position_embeddings=512),
        seed=3, std=0.08, norm_mean=1.0, norm_std=0.2),
}


def make_model_dir(path, name, dtype=torch.bfloat16):
    from llama_rs_metal_b200.engine.session import write_random_model
    spec = TINY[name]
    return write_random_model(path, spec["config"], seed=spec["seed"], std=spec["std"],
                              norm_mean=spec["norm_mean"], norm_std=spec["norm_std"], dtype=dtype)


def random_tokens(seed, length, vocab):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=length)]


# --------------------------------------------------------------------------- tolerances
# Error is measured against the largest |logit| of the reference rows compared.
#  float32: the engine's sums are float32 in another order than the oracle's float64;
#           a few 1e-6 relative per layer.
#  bfloat16: activations and cache are rounded to 8 bits of mantissa (2^-9 relative)
#           between kernels; a few rounding steps per layer add up to about a percent.
TOLERANCE = {"float32": 2e-5, "bfloat16": 3e-2}


def assert_logits_close(got, ref, dtype, what=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite logits"
    scale = max(float(np.abs(ref).max()), 1e-30)
    err = np.abs(got - ref).max(axis=-1) / scale
    worst = int(err.argmax())
    assert err[worst] <= TOLERANCE[dtype], (
        f"{what}: row {worst} is off by {err[worst]:.3e} of the largest logit "
        f"(allowed {TOLERANCE[dtype]:.1e}); first wrong row "
        f"{int(np.argmax(err > TOLERANCE[dtype]))}")


# --------------------------------------------------------------------------- traces
class Trace:
    """Steps for bin/trace_run plus, for each step, which (request, position) each row is."""

    def __init__(self):
        self.steps = []
        self.rows = {}

    def add(self, entries, end=()):
        """entries: list of (request id, tokens, first position, want places)."""
        step = len(self.steps)
        self.steps.append({"step": step, "end": list(end), "entries": [
            {"id": rid, "tokens": list(tokens), "want": list(want)} for rid, tokens, _, want in entries]})
        rows = [(rid, first + p) for rid, _, first, want in entries for p in want]
        if rows:
            self.rows[step] = rows
        return step

    def whole(self, name, tokens):
        self.add([(name, tokens, 0, range(len(tokens)))], end=[name])

    def tail_one_by_one(self, name, tokens, tail=32):
        head = max(1, len(tokens) - tail)
        self.add([(name, tokens[:head], 0, range(head))], end=[name] if head == len(tokens) else [])
        for p in range(head, len(tokens)):
            self.add([(name, [tokens[p]], p, [0])], end=[name] if p == len(tokens) - 1 else [])

    def batch(self, requests, prompt_lengths):
        """requests: {name: tokens}. Prompts (the first prompt_lengths[name] tokens) in one
        step, then one token each per step; a request ends after its last token."""
        names = list(requests)
        done_at = {n: len(requests[n]) for n in names}
        at = {n: prompt_lengths[n] for n in names}
        entries = [(n, requests[n][:at[n]], 0, range(at[n])) for n in names]
        self.add(entries, end=[n for n in names if at[n] == done_at[n]])
        live = [n for n in names if at[n] < done_at[n]]
        while live:
            entries = [(n, [requests[n][at[n]]], at[n], [0]) for n in live]
            for n in live:
                at[n] += 1
            self.add(entries, end=[n for n in live if at[n] == done_at[n]])
            live = [n for n in live if at[n] < done_at[n]]


def run_trace(model_dir, dtype, trace, max_tokens, out_dir, timeout=900):
    """Drive bin/trace_run step by step (next step only after `done`); {step: float32 [rows, vocab]}."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for step in trace.steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {step['step']}", f"trace_run answered {line!r} to step {step['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    with open(os.path.join(model_dir, "config.json")) as handle:
        vocab = json.load(handle)["vocab_size"]
    out = {}
    for step, rows in trace.rows.items():
        data = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
        assert data.size == len(rows) * vocab, f"step {step}: {data.size} floats for {len(rows)} rows"
        out[step] = data.reshape(len(rows), vocab)
    return out


def check_trace(trace, outputs, reference_logits, dtype):
    """reference_logits: {request: float64 [T, vocab]} from the plain implementation; a trace
    names a request "<mode>:<request>" so that one request can be replayed in several ways."""
    for step in sorted(trace.rows):
        rows = trace.rows[step]
        ref = np.stack([reference_logits[rid.split(":")[-1]][pos] for rid, pos in rows])
        assert_logits_close(outputs[step], ref, dtype,
                            what=f"step {step} ({rows[0][0]} pos {rows[0][1]} ..)")
