"""Trace replay through bin/trace_run, compared with the plain implementation.

The same requests are replayed whole, with their last 32 tokens one by one, and in
batches of unequal lengths that run one after another so that slots and pages are
used again; in float32 and in bfloat16; on every tiny configuration.
"""
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
    # three batches one after another; in each, shorter requests end earlier
    groups = [["r0", "r1", "r2"], ["r3", "r4", "r5", "r6"], ["r7", "r8", "r9", "r1"]]
    for g, names in enumerate(groups):
        batch = {f"batch{g}:{n}": requests[n] for n in names}
        prompts = {f"batch{g}:{n}": max(1, len(requests[n]) - (4 + 3 * i)) for i, n in enumerate(names)}
        trace.batch(batch, prompts)
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_whole_tail_and_batches(name, dtype, model_dirs, references, tmp_path):
    requests = requests_for(name)
    trace = build_trace(requests)
    # the most that is live at once: the last batch, each request rounded up to 64
    need = max(sum(-(-len(requests[n]) // 64) * 64 for n in g)
               for g in (["r0", "r1", "r2"], ["r3", "r4", "r5", "r6"], ["r7", "r8", "r9", "r1"]))
    outputs = helpers.run_trace(model_dirs[name], dtype, trace, need, str(tmp_path))
    helpers.check_trace(trace, outputs, references[name], dtype)


def test_replay_rejects_a_trace_that_outgrows_max_tokens(model_dirs, tmp_path):
    trace = helpers.Trace()
    trace.whole("whole:r", helpers.random_tokens(1, 200, 256))
    with pytest.raises(AssertionError):
        helpers.run_trace(model_dirs["A"], "float32", trace, 128, str(tmp_path))
