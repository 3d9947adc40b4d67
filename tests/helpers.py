"""Shared by the tests: the tiny configurations, request sets, tolerances, trace replay driver."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny Llama configurations that differ in every size and option, a third with awkward
# sizes (width 68 is no multiple of 8, vocabulary 307 is prime, 100 is no multiple of 8), and two
# narrow ones with the head geometry of the sizes the benchmark is quoted on, so that whole models
# run through the tensor-core kernels: D has head size 64 in groups of 4 (the 1B geometry, tied,
# llama3 factor 32), E head size 128 with an untied head (the 3B / 8B geometry).
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
    "D": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=512,
                    intermediate_size=1536, num_hidden_layers=2, num_attention_heads=8,
                    num_key_value_heads=2, head_dim=64, vocab_size=2048, rope_theta=500000.0,
                    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0,
                                      high_freq_factor=4.0, original_max_position_embeddings=8192),
                    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024),
        seed=11, std=0.04, norm_mean=1.0, norm_std=0.05),
    "E": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=384,
                    intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=128, vocab_size=1000, rope_theta=500000.0,
                    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                      high_freq_factor=4.0, original_max_position_embeddings=8192),
                    rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=1024),
        seed=13, std=0.05, norm_mean=1.0, norm_std=0.05),
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


# --------------------------------------------------------------------------- sampling twin
def gumbel_twin(logits, temperature, seed, key):
    """The device sampler's perturbed scores, restated on the CPU with the same integer hash
    (csrc/sampling.cu): the chosen id is the argmax of what this returns."""
    import math
    mask = (1 << 64) - 1

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)
    scores = []
    for i, v in enumerate(logits):
        z = mix((mix((seed + 0x9E3779B97F4A7C15 * (key + 1)) & mask) + i) & mask)
        u = (float(z >> 40) + 0.5) / 16777216.0
        scores.append(float(v) / temperature - math.log(-math.log(u)))
    return scores


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

    def chunks(self, name, tokens, sizes):
        """The sequence in portions: `sizes` is a list of portion lengths (the last one repeats
        until the tokens run out), each portion a step of its own onto the started sequence."""
        at, i = 0, 0
        while at < len(tokens):
            n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
            self.add([(name, tokens[at:at + n], at, range(n))], end=[name] if at + n == len(tokens) else [])
            at, i = at + n, i + 1

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


# --------------------------------------------------------------------------- parity at large widths
_PLAIN_ROWS = {}


def narrowed_copy(model_dir, out_dir, layers):
    """A model folder with the first `layers` layers of `model_dir`: its config.json with
    num_hidden_layers lowered and a link to the same model.safetensors (the loader skips the
    tensors of the layers the smaller model has no use for)."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json")) as handle:
        config = json.load(handle)
    config["num_hidden_layers"] = layers
    with open(os.path.join(out_dir, "config.json"), "w") as handle:
        json.dump(config, handle)
    link = os.path.join(out_dir, "model.safetensors")
    if os.path.lexists(link):
        os.remove(link)
    os.symlink(os.path.abspath(os.path.join(model_dir, "model.safetensors")), link)
    return out_dir


def parity_with_plain(engine, model_dir, dtype, prompt_lengths=(300, 170, 40), decode_steps=8, seed=5,
                      chunk=64, keep=4):
    """Run the engine on a model folder in three ways and compare with the plain implementation:
    every prompt alone and whole; all prompts as one batch of unequal lengths followed by
    `decode_steps` steps of one (given, random) token each; the first prompt in portions of
    `chunk` tokens. Logits are compared at each prompt's first position and last `keep` positions
    and at every decoded position. Returns the largest error as a fraction of the largest
    reference logit (assert_logits_close's measure); raises AssertionError beyond the tolerance.
    Works for models too large for a float64 copy (the plain side reads tensors one at a time)."""
    import plain_llama as P
    from llama_rs_metal_b200.cache import Cache
    from llama_rs_metal_b200.engine.batch import StepEntry
    from llama_rs_metal_b200.engine.session import build_model
    from llama_rs_metal_b200.engine.step import StepRunner
    from llama_rs_metal_b200.runtime import Runtime, parse_dtype

    config, tensors = P.read_model_lazily(model_dir)
    vocab = config["vocab_size"]
    seqs = [random_tokens(seed + i, n + decode_steps, vocab) for i, n in enumerate(prompt_lengths)]

    def places(n):
        return sorted(set([0] + list(range(max(0, n - keep), n))))
    wanted = [places(n) + list(range(n, n + decode_steps)) for n in prompt_lengths]
    key = (os.path.realpath(os.path.join(model_dir, "model.safetensors")), config["num_hidden_layers"],
           tuple(prompt_lengths), decode_steps, seed, keep)
    if key not in _PLAIN_ROWS:  # both dtypes compare with the same rows
        _PLAIN_ROWS[key] = [P.forward(config, tensors, s, rows=w).numpy() for s, w in zip(seqs, wanted)]
    refs = _PLAIN_ROWS[key]

    rt = Runtime(engine.device, parse_dtype(dtype))
    _, _, model, _ = build_model(model_dir, rt)
    budget = sum(-(-(n + decode_steps) // 64) * 64 for n in prompt_lengths)
    cache = Cache(model.cache_requests(), rt.dtype, rt.device, budget, len(seqs), max(len(s) for s in seqs))
    runner = StepRunner(model, cache, rt)
    worst = 0.0

    def compare(got, ref, what):
        nonlocal worst
        assert_logits_close(got, ref, dtype, what)
        scale = max(float(np.abs(ref).max()), 1e-30)
        worst = max(worst, float(np.abs(np.asarray(got, dtype=np.float64) - ref).max()) / scale)

    for b, (s, n) in enumerate(zip(seqs, prompt_lengths)):                 # alone and whole
        slot = cache.open_slot()
        out = runner.step([StepEntry(slot, s[:n], places(n))]).cpu().numpy()
        compare(out, refs[b][:len(places(n))], f"prompt {b} alone")
        cache.close_slot(slot)
    slots = [cache.open_slot() for _ in seqs]                              # unequal batch, then decoding
    out = runner.step([StepEntry(sl, s[:n], places(n)) for sl, s, n in zip(slots, seqs, prompt_lengths)]).cpu().numpy()
    row = 0
    for b, n in enumerate(prompt_lengths):
        compare(out[row:row + len(places(n))], refs[b][:len(places(n))], f"prompt {b} in the batch")
        row += len(places(n))
    for step in range(decode_steps):
        out = runner.step([StepEntry(sl, [s[n + step]], [0]) for sl, s, n in zip(slots, seqs, prompt_lengths)])
        out = out.cpu().numpy()
        for b, n in enumerate(prompt_lengths):
            compare(out[b:b + 1], refs[b][len(places(n)) + step][None], f"sequence {b}, decode step {step}")
    for sl in slots:
        cache.close_slot(sl)
    slot, n = cache.open_slot(), prompt_lengths[0]                          # the first prompt in portions
    rows = {}
    for at in range(0, n, chunk):
        m = min(chunk, n - at)
        want = [p - at for p in places(n) if at <= p < at + m]
        out = runner.step([StepEntry(slot, seqs[0][at:at + m], want)]).cpu().numpy()
        for i, p in enumerate(want):
            rows[p + at] = out[i]
    compare(np.stack([rows[p] for p in places(n)]), refs[0][:len(places(n))], f"prompt 0 in portions of {chunk}")
    cache.close_slot(slot)
    runner.check_device_status()
    return worst
