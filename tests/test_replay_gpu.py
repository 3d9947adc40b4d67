"""Trace replay through bin/trace_run, compared with the plain implementation.

The same requests are replayed whole, with their last 32 tokens one by one, in
batches of unequal lengths that run one after another so that slots and pages are
used again, and in portions (chunks of 17 as the reference's gate cuts them,
tools/benchmarks/verify.py:222-225, and 4 + 5 as crates/llama-rs/tests/sessions.rs:10-37);
in float32 and in bfloat16; on every tiny configuration.
"""
import numpy as np
import pytest

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu

LENGTHS = [5, 11, 17, 70, 40, 33, 1, 64, 65, 130]


def requests_for(name):
    vocab = helpers.TINY[name]["config"]["vocab_size"]
    return {f"r{i}": helpers.random_tokens(100 + i, n, vocab) for i, n in enumerate(LENGTHS)}


@pytest.fixture(scope="module")
def references(plain_models):
    out = {}
    for name, (cfg, tensors) in plain_models.items():
        out[name] = {rid: P.forward(cfg, tensors, tokens).numpy()
                     for rid, tokens in requests_for(name).items()}
    return out


def build_trace(requests):
    trace = helpers.Trace()
    for rid, tokens in requests.items():
        trace.whole("whole:" + rid, tokens)
    for rid, tokens in requests.items():
        trace.tail_one_by_one("tail:" + rid, tokens)
    for rid, tokens in requests.items():       # portions onto a started sequence
        if len(tokens) > 17:
            trace.chunks("chunks17:" + rid, tokens, [17])
        if len(tokens) >= 9:
            trace.chunks("four-five:" + rid, tokens[:9], [4, 5])
    trace.chunks("ragged:r9", requests["r9"], [1, 2, 63, 64])   # cuts at 1, 3, 66, 130: a page's edge inside a portion
    # three batches one after another; in each, shorter requests end earlier
    groups = [["r0", "r1", "r2"], ["r3", "r4", "r5", "r6"], ["r7", "r8", "r9", "r1"]]
    for g, names in enumerate(groups):
        batch = {f"batch{g}:{n}": requests[n] for n in names}
        prompts = {f"batch{g}:{n}": max(1, len(requests[n]) - (4 + 3 * i)) for i, n in enumerate(names)}
        trace.batch(batch, prompts)
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_replay_whole_tail_and_batches(name, dtype, model_dirs, references, tmp_path):
    requests = requests_for(name)
    trace = build_trace(requests)
    # the most that is live at once: the last batch, each request rounded up to 64
    need = max(sum(-(-len(requests[n]) // 64) * 64 for n in g)
               for g in (["r0", "r1", "r2"], ["r3", "r4", "r5", "r6"], ["r7", "r8", "r9", "r1"]))
    outputs = helpers.run_trace(model_dirs[name], dtype, trace, need, str(tmp_path))
    helpers.check_trace(trace, outputs, references[name], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("count", [24, 64])
def test_replay_large_batches_of_short_requests(count, dtype, model_dirs, plain_models, tmp_path):
    """Batches of 24 and 64 sequences on the configuration with the 1B head geometry: decode steps of
    9-64 rows take other matrix-product and attention kernels than the small batches above."""
    vocab = helpers.TINY["D"]["config"]["vocab_size"]
    lengths = [3 + (7 * i) % 38 for i in range(count)]           # 3 .. 40 tokens, unequal
    requests = {f"q{i}": helpers.random_tokens(500 + i, n + 6, vocab) for i, n in enumerate(lengths)}
    cfg, tensors = plain_models["D"]
    refs = {rid: P.forward(cfg, tensors, tokens).numpy() for rid, tokens in requests.items()}
    trace = helpers.Trace()
    trace.batch({"big:" + rid: tokens for rid, tokens in requests.items()},
                {"big:" + rid: len(tokens) - 6 + (i % 3) for i, (rid, tokens) in enumerate(requests.items())})
    outputs = helpers.run_trace(model_dirs["D"], dtype, trace, 64 * count, str(tmp_path))
    helpers.check_trace(trace, outputs, refs, dtype)


def test_two_replays_of_one_trace_give_the_same_bits(model_dirs, tmp_path):
    """bfloat16 too is reproducible run to run: no result depends on which CTA finishes first."""
    requests = requests_for("D")
    trace = helpers.Trace()
    trace.batch({f"b:{n}": requests[n] for n in ("r3", "r4", "r5", "r9")},
                {f"b:{n}": max(1, len(requests[n]) - 20) for n in ("r3", "r4", "r5", "r9")})
    trace.chunks("c:r9", requests["r9"], [17])
    first = helpers.run_trace(model_dirs["D"], "bfloat16", trace, 512, str(tmp_path / "one"))
    second = helpers.run_trace(model_dirs["D"], "bfloat16", trace, 512, str(tmp_path / "two"))
    assert sorted(first) == sorted(second)
    for step in first:
        assert np.array_equal(first[step], second[step]), f"step {step} differs between two runs"


def test_replay_rejects_a_trace_that_outgrows_max_tokens(model_dirs, tmp_path):
    trace = helpers.Trace()
    trace.whole("whole:r", helpers.random_tokens(1, 200, 256))
    with pytest.raises(AssertionError):
        helpers.run_trace(model_dirs["A"], "float32", trace, 128, str(tmp_path))
