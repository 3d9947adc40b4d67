"""The generation loop's decisions, with stand-ins for the device (no GPU)."""
import numpy as np
import pytest

from llama_rs_metal_b200.engine.generate import generate, plan_batches
from llama_rs_metal_b200.errors import CacheMemoryError, CancelledError, ContextError, OptionsError
from llama_rs_metal_b200.sampling import GenerationOptions, Sampling, SplitMix64, sample_host


class ScriptedStepper:
    """Slots like the cache's; logits are one-hot on a scripted next token:
    next(sequence) = (sum of its tokens * 7 + its length) % vocab."""

    def __init__(self, slots=4, vocab=50):
        self.vocab, self.free, self.live = vocab, list(range(slots - 1, -1, -1)), {}
        self.log = []
        self.opened = []

    def open_slot(self):
        if not self.free:
            raise CacheMemoryError("no slot")
        slot = self.free.pop()
        self.live[slot] = []
        self.opened.append(slot)
        return slot

    def close_slot(self, slot):
        assert slot in self.live, "closed twice"
        del self.live[slot]
        self.free.append(slot)
        self.free.sort(reverse=True)

    def step(self, entries):
        lengths = {len(self.live[e.slot]) for e in entries}
        if lengths == {0}:
            kind = "prefill"
        else:
            assert 0 not in lengths and all(len(e.tokens) == 1 for e in entries), "mixed step"
            kind = "decode"
        self.log.append((kind, [(e.slot, list(e.tokens)) for e in entries]))
        rows = []
        for e in entries:
            self.live[e.slot].extend(e.tokens)
            assert list(e.want) == [len(e.tokens) - 1]
            seq = self.live[e.slot]
            row = np.zeros(self.vocab, dtype=np.float32)
            row[(sum(seq) * 7 + len(seq)) % self.vocab] = 10.0
            rows.append(row)
        return np.stack(rows)


class ArgmaxSampler:
    def pick(self, logits, requests, steps, histories):
        self.last = (list(requests), list(steps))
        return [int(np.argmax(r)) for r in logits]


def expected(prompt, n, vocab=50, stop=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = (sum(seq) * 7 + len(seq)) % vocab
        if t in stop:
            return out, "eos"
        out.append(t)
        seq.append(t)
    return out, "length"


def run(prompts, max_tokens=5, stop=(), slots=4, **kw):
    stepper = ScriptedStepper(slots=slots)
    results = generate(stepper, ArgmaxSampler(), prompts,
                       GenerationOptions(max_tokens=max_tokens, sampling=Sampling(temperature=0.0)),
                       stop_token_ids=stop, max_batch=slots, **kw)
    assert not stepper.live, "a slot was not given back"
    return stepper, results


def test_unequal_prompts_one_prefill_then_one_token_each():
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9, 10]]
    stepper, results = run(prompts, max_tokens=4)
    assert [r.tokens for r in results] == [expected(p, 4)[0] for p in prompts]
    assert all(r.finish_reason == "length" for r in results)
    kinds = [k for k, _ in stepper.log]
    assert kinds == ["prefill", "decode", "decode", "decode"]   # N tokens: 1 prefill + N-1 decodes
    assert [tokens for _, tokens in stepper.log[0][1]] == prompts


def test_stop_token_is_neither_emitted_nor_fed_and_the_batch_shrinks():
    prompts = [[1, 2, 3], [4], [9, 9]]
    full = [expected(p, 6)[0] for p in prompts]
    stop = {full[1][2]}                         # the second request's third token
    stepper, results = run(prompts, max_tokens=6, stop=stop)
    for r, p in zip(results, prompts):
        tokens, reason = expected(p, 6, stop=stop)
        assert (r.tokens, r.finish_reason) == (tokens, reason)
    assert results[1].finish_reason == "eos" and len(results[1].tokens) == 2
    sizes = [len(entries) for _, entries in stepper.log]
    assert sizes[0] == 3 and sizes[-1] < 3      # finished sequences leave the batch
    fed = [t for _, entries in stepper.log[1:] for _, toks in entries for t in toks]
    assert not (stop & set(fed) - {t for r in results if r.finish_reason != "eos" for t in r.tokens})


def test_more_requests_than_slots_run_as_batches_that_reuse_slots():
    prompts = [[i + 1] * (i % 3 + 1) for i in range(7)]
    stepper, results = run(prompts, max_tokens=3, slots=3)
    assert [r.tokens for r in results] == [expected(p, 3)[0] for p in prompts]
    prefills = [entries for kind, entries in stepper.log if kind == "prefill"]
    assert [len(e) for e in prefills] == [3, 3, 1]
    assert set(stepper.opened) == {0, 1, 2} and len(stepper.opened) == 7


def test_context_reason_when_the_pending_token_does_not_fit():
    stepper, results = run([[1, 2, 3, 4]], max_tokens=10, context=6)
    # cache may hold 6 tokens: 4 prompt + 2 fed; the third sampled token stays pending
    assert results[0].finish_reason == "context" and len(results[0].tokens) == 3
    assert results[0].tokens == expected([1, 2, 3, 4], 3)[0]


def test_cancel_between_steps():
    calls = {"n": 0}

    def cancelled():
        calls["n"] += 1
        return calls["n"] > 3
    stepper, results = run([[1, 2], [3]], max_tokens=50, cancelled=cancelled)
    assert all(r.finish_reason == "cancelled" for r in results)
    assert 0 < len(results[0].tokens) < 50
    with pytest.raises(CancelledError):
        run([[1]], cancelled=lambda: True)


def test_bad_requests_are_rejected_before_anything_runs():
    with pytest.raises(OptionsError):
        run([[1], []])
    with pytest.raises(OptionsError):
        run([[1]], max_tokens=0)
    with pytest.raises(ContextError):
        run([[1] * 9], context=8)
    with pytest.raises(OptionsError):
        generate(ScriptedStepper(), ArgmaxSampler(), [[1]],
                 GenerationOptions(sampling=Sampling(temperature=float("nan"))))


def test_batches_respect_the_token_budget():
    assert plan_batches([10, 10, 10], max_batch=8, token_budget=128, page_size=64,
                        max_new_tokens=4, context=1000) == [[0, 1], [2]]
    assert plan_batches([100, 10], 8, 256, 64, 30, 1000) == [[0, 1]]       # 192 + 64 tokens fit
    assert plan_batches([100, 10], 8, 255, 64, 30, 1000) == [[0], [1]]     # 129 tokens round up to 192
    with pytest.raises(ContextError):
        plan_batches([300], 8, 256, 64, 4, 1000)


def test_sampler_sees_request_numbers_and_step_counts():
    stepper = ScriptedStepper()
    sampler = ArgmaxSampler()
    generate(stepper, sampler, [[1], [2], [3]], GenerationOptions(max_tokens=3, sampling=Sampling(temperature=0.0)),
             max_batch=2)
    assert sampler.last == ([2], [2])


# ------------------------------------------------------------------ the host sampler
def test_reference_sampler_unit_cases():
    # crates/llama-rs/src/sampling.rs:125-138
    greedy = Sampling(temperature=0.0)
    assert sample_host(np.array([1.0, 3.0, 3.0]), [], SplitMix64(0), greedy) == 1
    default = Sampling()
    picks = {sample_host(np.array([1.0, 2.0, 3.0]), [], SplitMix64(7), default) for _ in range(20)}
    assert len(picks) == 1
    with pytest.raises(OptionsError):
        Sampling(temperature=float("nan")).validate()
    with pytest.raises(OptionsError):
        sample_host(np.array([1.0, float("inf")]), [], SplitMix64(0), default)


def test_host_sampler_equals_the_plain_sampler():
    import plain_llama
    rng = np.random.default_rng(0)
    for case in range(200):
        logits = rng.normal(size=97).astype(np.float32) * 3
        history = [int(t) for t in rng.integers(0, 97, size=80)]
        opts = Sampling(temperature=[0.0, 0.7, 1.3][case % 3], top_k=[0, 5, 40, 200][case % 4],
                        top_p=[1.0, 0.9, 0.5][case % 3], repeat_penalty=[1.0, 1.3][case % 2],
                        repeat_last_n=[64, 10][case % 2], seed=case)
        got = sample_host(logits, history, SplitMix64(case), opts)
        want = plain_llama.sample(logits, history, plain_llama.SplitMix64(case), opts.temperature,
                                  opts.top_k, opts.top_p, opts.repeat_penalty, opts.repeat_last_n)
        assert got == want, case


def test_repeat_penalty_and_top_k_change_the_choice():
    logits = np.array([5.0, 4.9, 1.0, -2.0])
    assert sample_host(logits, [0], SplitMix64(0), Sampling(temperature=0.0, repeat_penalty=2.0)) == 1
    only_top = {sample_host(logits, [], SplitMix64(s), Sampling(temperature=5.0, top_k=2, top_p=1.0))
                for s in range(200)}
    assert only_top == {0, 1}


class AheadStepper(ScriptedStepper):
    """The scripted stepper with a decode step whose tokens the host has not seen yet: what a
    step chose stays 'on the device' (a list the host may only read through ids())."""

    can_decode_ahead = True

    class Pending:
        def __init__(self, chosen):
            self.device_ids, self.read = chosen, False

        def ids(self):
            self.read = True
            return list(self.device_ids)

    def decode_ahead(self, slots, tokens, previous, picker):
        fed = list(previous.device_ids) if tokens is None else list(tokens)
        assert len(fed) == len(slots)
        self.log.append(("ahead" if tokens is None else "decode", [(s, [t]) for s, t in zip(slots, fed)]))
        rows = []
        for slot, token in zip(slots, fed):
            seq = self.live[slot]  # a slot that was closed meanwhile would fail here
            assert seq, "decode before the prompt"
            seq.append(token)
            row = np.zeros(self.vocab, dtype=np.float32)
            row[(sum(seq) * 7 + len(seq)) % self.vocab] = 10.0
            rows.append(row)
        return self.Pending(picker(np.stack(rows)))


class AheadSampler(ArgmaxSampler):
    def device_picker(self, requests, steps):
        return lambda logits: [int(np.argmax(r)) for r in logits]


@pytest.mark.parametrize("seed", range(12))
def test_running_one_step_ahead_changes_no_decision(seed):
    rng = np.random.default_rng(seed)
    prompts = [[int(t) for t in rng.integers(0, 50, size=int(rng.integers(1, 9)))] for _ in range(int(rng.integers(1, 8)))]
    stop = [int(t) for t in rng.integers(0, 50, size=int(rng.integers(0, 6)))]
    max_tokens = int(rng.integers(1, 12))
    context = int(rng.integers(9, 16))
    options = GenerationOptions(max_tokens=max_tokens, sampling=Sampling(temperature=0.0))
    plain = ScriptedStepper(slots=3)
    want = generate(plain, ArgmaxSampler(), prompts, options, stop_token_ids=stop, max_batch=3, context=context)
    ahead = AheadStepper(slots=3)
    emitted = []
    got = generate(ahead, AheadSampler(), prompts, options, stop_token_ids=stop, max_batch=3, context=context,
                   on_token=lambda request, token: emitted.append((request, token)))
    assert not ahead.live, "a slot was not given back"
    assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in want]
    assert sorted(emitted) == sorted((r.request, t) for r in got for t in r.tokens)
    # no token is fed that the plain loop does not feed, except to a sequence that a stop token
    # had just ended (its row is dropped)
    fed_plain = sum(len(rows) for kind, rows in plain.log if kind == "decode")
    fed_ahead = sum(len(rows) for kind, rows in ahead.log if kind != "prefill")
    ended_by_stop = sum(r.finish_reason == "eos" for r in got)
    assert fed_plain <= fed_ahead <= fed_plain + ended_by_stop


def test_running_ahead_keeps_a_step_in_flight():
    stepper = AheadStepper(slots=2)
    options = GenerationOptions(max_tokens=6, sampling=Sampling(temperature=0.0))
    generate(stepper, AheadSampler(), [[1, 2], [3]], options, max_batch=2)
    kinds = [k for k, _ in stepper.log]
    assert kinds == ["prefill", "decode", "ahead", "ahead", "ahead", "ahead"]


class RewindStepper(AheadStepper):
    """An ahead stepper whose last step can be taken back (what a cache of keys and values allows)."""

    can_rewind = True

    def rewind(self, slots, tokens=1):
        assert tokens == 1
        kind, rows = self.log[-1]
        assert kind == "ahead" and {s for s, _ in rows} >= set(slots), "only the step in flight is taken back"
        self.log[-1] = ("dropped", rows)
        for slot in slots:
            self.live[slot].pop()


@pytest.mark.parametrize("seed", range(12))
def test_a_step_in_flight_is_dropped_whole_when_a_stop_token_ends_a_sequence(seed):
    """With a stepper that can take a step back, every step that counts is a step the plain loop
    runs: same sequences, same tokens, in the same order. (Equal batches are what makes the
    device results equal bit for bit.)"""
    rng = np.random.default_rng(100 + seed)
    prompts = [[int(t) for t in rng.integers(0, 50, size=int(rng.integers(1, 9)))] for _ in range(int(rng.integers(2, 8)))]
    stop = [int(t) for t in rng.integers(0, 50, size=int(rng.integers(1, 8)))]
    options = GenerationOptions(max_tokens=int(rng.integers(2, 12)), sampling=Sampling(temperature=0.0))
    context = int(rng.integers(9, 16))
    plain = ScriptedStepper(slots=3)
    want = generate(plain, ArgmaxSampler(), prompts, options, stop_token_ids=stop, max_batch=3, context=context)
    ahead = RewindStepper(slots=3)
    got = generate(ahead, AheadSampler(), prompts, options, stop_token_ids=stop, max_batch=3, context=context)
    assert not ahead.live
    assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in want]
    counted = [rows for kind, rows in ahead.log if kind in ("decode", "ahead")]
    assert counted == [rows for kind, rows in plain.log if kind == "decode"]
