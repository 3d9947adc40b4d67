"""The engine in-process: parts alone, cutting invariance, long decoding, generation, a toy mixer."""

import numpy as np
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def engine():
    from llama_rs_metal_b200 import Engine
    return Engine()


def open_runner(engine, model_dir, dtype, max_tokens=2048, max_slots=8):
    from llama_rs_metal_b200.cache import Cache
    from llama_rs_metal_b200.engine.session import build_model
    from llama_rs_metal_b200.engine.step import StepRunner
    from llama_rs_metal_b200.runtime import Runtime, parse_dtype
    rt = Runtime(engine.device, parse_dtype(dtype))
    _, plan, model, _ = build_model(model_dir, rt)
    cache = Cache(model.cache_requests(), rt.dtype, rt.device, max_tokens, max_slots, max_tokens)
    return StepRunner(model, cache, rt), cache, model


def entry(slot, tokens, want=None):
    from llama_rs_metal_b200.engine.batch import StepEntry
    return StepEntry(slot, tokens, range(len(tokens)) if want is None else want)


# --------------------------------------------------------------------------- cutting invariance
@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_float32_logits_are_identical_however_the_tokens_are_cut(engine, model_dirs, name):
    vocab = helpers.TINY[name]["config"]["vocab_size"]
    seqs = [helpers.random_tokens(40 + i, n, vocab) for i, n in enumerate([70, 9, 33])]
    runner, cache, _ = open_runner(engine, model_dirs[name], "float32")
    whole = []
    for s in seqs:
        slot = cache.open_slot()
        whole.append(runner.step([entry(slot, s)]).clone())
        cache.close_slot(slot)
    # one batch: prompts of 3 tokens, then token by token; shorter sequences end earlier
    slots = [cache.open_slot() for _ in seqs]
    got = [[] for _ in seqs]
    out = runner.step([entry(sl, s[:3]) for sl, s in zip(slots, seqs)])
    for b in range(3):
        got[b].append(out[3 * b:3 * b + 3])
    for p in range(3, 70):
        live = [b for b in range(3) if p < len(seqs[b])]
        out = runner.step([entry(slots[b], [seqs[b][p]]) for b in live])
        for row, b in enumerate(live):
            got[b].append(out[row:row + 1])
    for b in range(3):
        assert torch.equal(torch.cat(got[b]), whole[b]), f"sequence {b} differs between whole and batched decoding"
        cache.close_slot(slots[b])
    # portions onto started sequences: chunks of 17 (tools/benchmarks/verify.py:222-225), 4 + 5
    # (crates/llama-rs/tests/sessions.rs:10-37), and cuts at 1, 2, 63, 64, 65
    for sizes in ([17], [4, 5], [1, 1, 61, 1, 1]):
        slots = [cache.open_slot() for _ in seqs]
        got, at, i = [[] for _ in seqs], [0] * 3, 0
        while any(at[b] < len(seqs[b]) for b in range(3)):
            n = sizes[min(i, len(sizes) - 1)]
            live = [b for b in range(3) if at[b] < len(seqs[b])]
            out = runner.step([entry(slots[b], seqs[b][at[b]:at[b] + n]) for b in live])
            row = 0
            for b in live:
                m = min(n, len(seqs[b]) - at[b])
                got[b].append(out[row:row + m])
                row, at[b] = row + m, at[b] + m
            i += 1
        for b in range(3):
            assert torch.equal(torch.cat(got[b]), whole[b]), f"sequence {b} differs when cut into portions {sizes}"
            cache.close_slot(slots[b])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_padding_and_company_change_no_result(engine, model_dirs, dtype):
    runner, cache, _ = open_runner(engine, model_dirs["B"], dtype)
    a, b = helpers.random_tokens(1, 20, 512), helpers.random_tokens(2, 64, 512)
    s = cache.open_slot()
    alone = runner.step([entry(s, a)]).clone()
    cache.close_slot(s)
    s1, s2 = cache.open_slot(), cache.open_slot()
    both = runner.step([entry(s2, b), entry(s1, a)])
    if dtype == "float32":
        assert torch.equal(both[64:], alone)
    else:
        helpers.assert_logits_close(both[64:].cpu(), alone.cpu(), dtype)


# --------------------------------------------------------------------------- long decoding, first tokens
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_and_first_tokens(engine, model_dirs, plain_models, name, dtype):
    vocab = helpers.TINY[name]["config"]["vocab_size"]
    tokens = helpers.random_tokens(77, 400, vocab)           # crosses six page boundaries
    ref = P.forward(*plain_models[name], tokens).numpy()
    runner, cache, _ = open_runner(engine, model_dirs[name], dtype)
    slot = cache.open_slot()
    rows = [runner.step([entry(slot, tokens[:1])])]           # a prompt of one token
    for p in range(1, 400):
        rows.append(runner.step([entry(slot, [tokens[p]])]))
    got = torch.cat(rows).cpu().numpy()
    helpers.assert_logits_close(got[:8], ref[:8], dtype, "first tokens")
    helpers.assert_logits_close(got, ref, dtype, "long decoding")
    assert cache.length(slot) == 400


def test_a_used_slot_does_not_leak_into_its_next_sequence(engine, model_dirs, plain_models):
    runner, cache, _ = open_runner(engine, model_dirs["A"], "float32", max_tokens=256, max_slots=1)
    first, second = helpers.random_tokens(5, 200, 256), helpers.random_tokens(6, 90, 256)
    s = cache.open_slot()
    runner.step([entry(s, first, [])])
    cache.close_slot(s)
    s = cache.open_slot()
    got = [runner.step([entry(s, second[:50])])]
    got += [runner.step([entry(s, [t])]) for t in second[50:]]
    ref = P.forward(*plain_models["A"], second).numpy()
    helpers.assert_logits_close(torch.cat(got).cpu().numpy(), ref, "float32", "second tenant of the slot")


def test_rejected_steps_change_nothing(engine, model_dirs):
    from llama_rs_metal_b200.errors import CacheMemoryError, InvalidError
    runner, cache, _ = open_runner(engine, model_dirs["A"], "float32", max_tokens=128, max_slots=2)
    a, b = cache.open_slot(), cache.open_slot()
    good = runner.step([entry(a, [1, 2, 3])]).clone()
    with pytest.raises(InvalidError, match="outside vocabulary"):
        runner.step([entry(a, [256])])
    with pytest.raises(InvalidError):
        runner.step([entry(a, [4]), entry(b, [])])             # an entry without a token
    with pytest.raises(InvalidError):
        runner.step([entry(a, [4]), entry(a, [5])])
    with pytest.raises(InvalidError):
        runner.step([entry(a, [4], [1])])
    with pytest.raises(CacheMemoryError):
        runner.step([entry(b, [1] * 100)])                     # 64 + 128 tokens of pages in a 128-token cache
    assert cache.length(a) == 3 and cache.length(b) == 0
    cache.close_slot(a)
    a = cache.open_slot()
    assert torch.equal(runner.step([entry(a, [1, 2, 3])]), good)


# --------------------------------------------------------------------------- parts alone
def context_for(runtime, lengths, before=None, dest_rows=()):
    from llama_rs_metal_b200.engine.batch import StepEntry, pack_step
    before = before or [0] * len(lengths)
    entries = [StepEntry(i, [0] * n, []) for i, n in enumerate(lengths)]
    return pack_step(entries, before, runtime, "prefill" if not any(before) else "decode", dest_rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parts_alone(engine, dtype):
    from llama_rs_metal_b200.parts import (Attention, GatedMLP, PartSpec, PreNormBlock, RMSNorm,
                                           ScheduleEntry)
    from llama_rs_metal_b200.cache import Cache
    from llama_rs_metal_b200.runtime import Runtime, parse_dtype
    rt = Runtime(engine.device, parse_dtype(dtype))
    tol = helpers.TOLERANCE[dtype] * 2
    h, Hq, Hk, d, I = 72, 6, 2, 32, 104
    g = torch.Generator().manual_seed(0)

    def w(*shape, scale=0.1):
        return (torch.randn(*shape, generator=g) * scale).to(rt.dtype)

    lengths = [7, 1, 30]
    T = sum(lengths)
    ctx = context_for(rt, lengths)
    hidden = torch.randn(T, h, generator=g)

    norm = RMSNorm(h, 1e-3)
    nw = 1 + w(h)
    norm.bind({"weight": nw.to(DEV)}, rt)
    want_x = P.rms_norm(hidden.double(), nw.double(), 1e-3)
    x = norm.forward(hidden.to(DEV), ctx)
    assert x.dtype == rt.dtype
    helpers.assert_logits_close(x.float().cpu(), want_x, dtype, "norm part")

    mlp = GatedMLP(h, I)
    mw = {"gate_proj.weight": w(I, h), "up_proj.weight": w(I, h), "down_proj.weight": w(h, I)}
    mlp.bind({k: v.to(DEV) for k, v in mw.items()}, rt)
    resid = hidden.to(DEV).clone()
    out = mlp.forward(x, ctx, residual=resid)
    want = hidden.double() + P.gated_mlp(x.double().cpu(), *(mw[k].double() for k in
                                         ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
    helpers.assert_logits_close(out.cpu(), want, dtype, "feed-forward part")

    attn = Attention(h, Hq, Hk, d, position=PartSpec("rope", dict(head_dim=d, rotary_dim=16, theta=100.0)),
                     window=5)
    aw = {"q_proj.weight": w(Hq * d, h), "k_proj.weight": w(Hk * d, h), "v_proj.weight": w(Hk * d, h),
          "o_proj.weight": w(h, Hq * d)}
    attn.bind({k: v.to(DEV) for k, v in aw.items()}, rt)
    cache = Cache([attn.cache_request()], rt.dtype, rt.device, 256, 3, 128)
    for _ in lengths:
        cache.open_slot()
    cache.grow(list(enumerate(lengths)))
    cache.sync()
    ctx = context_for(rt, lengths, dest_rows=cache.destination_rows([0, 1, 2], [0, 0, 0], lengths))
    ctx.entry = ScheduleEntry(0, 0)
    resid = hidden.to(DEV).clone()
    out = attn.forward(x, ctx, cache.view(0), residual=resid)
    xd = x.double().cpu()
    inv = np.asarray([100.0 ** (-2.0 * i / 16) for i in range(8)]).astype(np.float32)
    want, at = [], 0
    for n in lengths:
        xs = xd[at:at + n]
        q = P.rope(P.linear(xs, aw["q_proj.weight"].double()).view(n, Hq, d), range(n), inv, 16)
        k = P.rope(P.linear(xs, aw["k_proj.weight"].double()).view(n, Hk, d), range(n), inv, 16)
        v = P.linear(xs, aw["v_proj.weight"].double()).view(n, Hk, d)
        want.append(P.linear(P.attention(q, k, v, window=5).reshape(n, Hq * d), aw["o_proj.weight"].double()))
        at += n
    helpers.assert_logits_close(out.cpu(), hidden.double() + torch.cat(want), dtype, "attention part")

    block = PreNormBlock(mixer=attn, feed_forward=mlp, mixer_norm=norm, feed_forward_norm=norm)
    out = block.forward(hidden.to(DEV).clone(), ctx, cache.view(0))
    ctx.settle(out)
    # the block is the two parts behind the norm: hidden += attention(norm(hidden)); += mlp(norm(hidden))
    after_mixer = hidden.double() + torch.cat(want)
    x2 = P.rms_norm(after_mixer, nw.double(), 1e-3)
    want_block = after_mixer + P.gated_mlp(x2, *(mw[k].double() for k in
                                           ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
    helpers.assert_logits_close(out.cpu(), want_block, dtype, "pre-norm block")


# --------------------------------------------------------------------------- generation
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(engine, model_dirs, plain_models, name, dtype):
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    vocab = helpers.TINY[name]["config"]["vocab_size"]
    prompts = [helpers.random_tokens(20 + i, n, vocab) for i, n in enumerate([5, 11, 17, 1, 64])]
    model = engine.load(model_dirs[name], dtype=dtype)
    session = model.session(context=128, max_batch=2)          # five requests through two slots
    results = session.generate(prompts, GenerationOptions(max_tokens=8, sampling=Sampling(temperature=0.0)),
                               stop_token_ids=())
    cfg, tensors = plain_models[name]
    margin = helpers.TOLERANCE[dtype] * 2
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and len(result.tokens) == 8
        seq = list(prompt)
        for token in result.tokens:
            logits = P.forward(cfg, tensors, seq)[-1].numpy()
            best = int(np.argmax(logits))
            # the engine's pick is the oracle's, or within rounding of it
            assert token == best or logits[best] - logits[token] <= margin * np.abs(logits).max(), \
                f"picked {token}, the plain implementation picks {best}"
            seq.append(token)
    assert session.cache.slots.held == 0 and session.cache.held_pages() == [0]


def test_stop_ids_context_and_temperature_through_the_entry_point(engine, model_dirs, plain_models):
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    model = engine.load(model_dirs["B"], dtype="float32")
    session = model.session(context=64, max_batch=4)
    prompts = [helpers.random_tokens(30 + i, n, 512) for i, n in enumerate([1, 9, 33, 60])]
    greedy = GenerationOptions(max_tokens=12, sampling=Sampling(temperature=0.0))
    free = session.generate(prompts, greedy, stop_token_ids=())
    assert free[3].finish_reason == "context" and len(free[3].tokens) == 5     # 60 + 4 fed = 64
    stop = free[1].tokens[3]
    cut = free[1].tokens.index(stop)
    stopped = session.generate(prompts, greedy, stop_token_ids=[stop])
    assert stopped[1].finish_reason == "eos" and stopped[1].tokens == free[1].tokens[:cut]
    # temperature 0.8, seed 9: repeatable, and independent of which requests share the batch
    hot = GenerationOptions(max_tokens=12, sampling=Sampling(temperature=0.8, top_k=0, top_p=1.0, seed=9))
    a = session.generate(prompts[:3], hot, stop_token_ids=())
    b = session.generate(prompts[:3], hot, stop_token_ids=())
    assert [r.tokens for r in a] == [r.tokens for r in b]
    assert a[0].tokens != free[0].tokens or a[1].tokens != free[1].tokens
    alone = model.session(context=64, max_batch=1).generate(prompts[:1], hot, stop_token_ids=())
    assert alone[0].tokens == a[0].tokens
    # the reference's host sampler (top-k, top-p, penalty) runs too and is repeatable
    ref = GenerationOptions(max_tokens=6, sampling=Sampling(repeat_penalty=1.1, seed=3))
    assert [r.tokens for r in session.generate(prompts[:2], ref, stop_token_ids=())] == \
           [r.tokens for r in session.generate(prompts[:2], ref, stop_token_ids=())]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_one_step_ahead_equals_step_by_step(engine, model_dirs, dtype):
    """With CUDA graphs the loop keeps one decode step in flight and feeds tokens on the
    device; without them it waits for every token. Same tokens and reasons either way:
    greedy and temperature, with stop ids that end sequences at different steps, a context
    that ends one, and more requests than slots."""
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    model = engine.load(model_dirs["A"], dtype=dtype)
    prompts = [helpers.random_tokens(70 + i, n, 256) for i, n in enumerate([3, 14, 40, 7, 66, 21, 1])]
    ahead = model.session(context=80, max_batch=3)
    plain = model.session(context=80, max_batch=3)
    plain.runner.use_graphs = False
    assert ahead.can_decode_ahead and not plain.can_decode_ahead
    for sampling in (Sampling(temperature=0.0), Sampling(temperature=0.9, top_k=0, top_p=1.0, seed=4)):
        options = GenerationOptions(max_tokens=24, sampling=sampling)
        free = plain.generate(prompts, options, stop_token_ids=())
        stops = sorted({free[0].tokens[5], free[1].tokens[11], free[3].tokens[0], free[5].tokens[23]})
        for stop_ids in ((), stops):
            want = plain.generate(prompts, options, stop_token_ids=stop_ids)
            got = ahead.generate(prompts, options, stop_token_ids=stop_ids)
            assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in want]
        assert {r.finish_reason for r in want} >= {"eos", "length", "context"}
    assert ahead.cache.slots.held == 0 and ahead.cache.held_pages() == [0]


def test_session_own_sequence_prefill_decode_reset(engine, model_dirs, plain_models):
    model = engine.load(model_dirs["A"], dtype="float32")
    session = model.session(context=96)
    tokens = helpers.random_tokens(3, 40, 256)
    ref = P.forward(*plain_models["A"], tokens).numpy()
    helpers.assert_logits_close(session.prefill(tokens[:30]).cpu().numpy()[None], ref[29:30], "float32")
    for p in range(30, 40):
        last = session.decode(tokens[p])
    helpers.assert_logits_close(last.cpu().numpy()[None], ref[39:40], "float32")
    assert session.tokens() == tokens
    k, v = session.snapshot(0)
    assert k.shape == (40, 2, 16) and torch.isfinite(k).all()
    from llama_rs_metal_b200.errors import ContextError
    with pytest.raises(ContextError):
        session.prefill([1] * 60)
    assert session.tokens() == tokens
    session.reset()
    assert session.tokens() == [] and session.logits() is None
    helpers.assert_logits_close(session.prefill(tokens[:30]).cpu().numpy()[None], ref[29:30], "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_adjacent_rotary_pairs_match_the_plain_implementation(engine, tmp_path, dtype):
    """rope_traditional=true pairs dimensions (2i, 2i+1); the engine reorders the query and key
    rows once and rotates split-half. Whole prompts, prompts in a batch and decoding must match
    the plain implementation, which rotates adjacent pairs directly (partial rotary width too)."""
    from llama_rs_metal_b200.engine.session import write_random_model
    cfg = dict(helpers.TINY["B"]["config"], rope_traditional=True, partial_rotary_factor=0.5)
    folder = write_random_model(str(tmp_path), cfg, seed=8, std=0.05, norm_std=0.1)
    plain_cfg, tensors = P.read_model(folder)
    assert plain_cfg["rope_traditional"] is True
    runner, cache, model = open_runner(engine, folder, dtype, max_tokens=1024, max_slots=3)
    seqs = [helpers.random_tokens(90 + i, n, 512) for i, n in enumerate([70, 9])]
    refs = [P.forward(plain_cfg, tensors, s).numpy() for s in seqs]
    straight = [P.forward(dict(plain_cfg, rope_traditional=False), tensors, s).numpy() for s in seqs]
    assert np.abs(refs[0] - straight[0]).max() > 1e-3          # the pairing matters for these weights
    slots = [cache.open_slot() for _ in seqs]
    prompts = [40, 4]
    out = runner.step([entry(sl, s[:p]) for sl, s, p in zip(slots, seqs, prompts)]).cpu()
    helpers.assert_logits_close(out[:40], refs[0][:40], dtype, "adjacent pairs, prompt")
    helpers.assert_logits_close(out[40:], refs[1][:4], dtype, "adjacent pairs, short prompt")
    for step in range(30):
        live = [b for b in (0, 1) if prompts[b] + step < len(seqs[b])]
        out = runner.step([entry(slots[b], [seqs[b][prompts[b] + step]]) for b in live]).cpu()
        for r, b in enumerate(live):
            helpers.assert_logits_close(out[r:r + 1], refs[b][prompts[b] + step][None], dtype, "adjacent pairs, decoding")


# --------------------------------------------------------------------------- a toy mixer with state
def test_a_toy_mixer_with_state_can_be_registered_built_and_stepped(engine, tmp_path):
    """A running-mean mixer, defined here: per-sequence state = (sum of inputs, count).
    It is registered, put into every second layer of a toy architecture next to the
    library's attention, and stepped; no file of the library changes."""
    from dataclasses import dataclass
    from llama_rs_metal_b200.config.base import read_int
    from llama_rs_metal_b200.engine.session import write_random_model
    from llama_rs_metal_b200.parts import LayerSpec, Mixer, ModelPlan, PartSpec, ScheduleEntry, StateRequest
    from llama_rs_metal_b200.registry import register_architecture, register_mixer
    from llama_rs_metal_b200.weights import TensorSpec

    @register_mixer("running_mean")
    class RunningMean(Mixer):
        def __init__(self, hidden_size):
            self.h = hidden_size

        def tensors(self):
            return {"mix.weight": TensorSpec((self.h,))}

        def bind(self, weights, runtime):
            self.w = weights["mix.weight"].float()

        def cache_request(self):
            return StateRequest((self.h + 1,))

        def forward(self, x, ctx, cache, residual):
            state = cache.state
            cu, slots = ctx.cu_seqlens.tolist(), ctx.slots.tolist()
            xs = x.float()
            for b, slot in enumerate(slots):
                rows = xs[cu[b]:cu[b + 1]]
                sums = state[slot, :self.h] + rows.cumsum(0)
                counts = state[slot, self.h] + torch.arange(1, rows.shape[0] + 1, device=x.device)
                residual[cu[b]:cu[b + 1]] += sums / counts[:, None] * self.w
                state[slot, :self.h] = sums[-1]
                state[slot, self.h] = counts[-1]
            return residual

    @dataclass(frozen=True)
    class ToyConfig:
        hidden: int
        layers: int
        vocab: int

        @classmethod
        def from_dict(cls, d):
            return cls(read_int(d, "hidden"), read_int(d, "layers"), read_int(d, "vocab"))

        def to_dict(self):
            return dict(architectures=["ToyForCausalLM"], hidden=self.hidden, layers=self.layers, vocab=self.vocab)

    def toy_plan(c):
        layers = []
        for i in range(c.layers):
            p = f"blocks.{i}."
            mixer = PartSpec("running_mean", dict(hidden_size=c.hidden), prefix=p) if i % 2 == 0 else \
                PartSpec("attention", dict(hidden_size=c.hidden, num_heads=2, num_kv_heads=1, head_dim=16,
                                           position=None), prefix=p + "attn.")
            layers.append(LayerSpec("pre_norm", mixer,
                                    PartSpec("gated_mlp", dict(hidden_size=c.hidden, intermediate_size=40), prefix=p + "ff."),
                                    PartSpec("rms_norm", dict(size=c.hidden, eps=1e-5), prefix=p + "n1."),
                                    PartSpec("rms_norm", dict(size=c.hidden, eps=1e-5), prefix=p + "n2.")))
        return ModelPlan(c.hidden, c.vocab, 1 << 20, "embed.weight", tuple(layers),
                         tuple(ScheduleEntry(i, i) for i in range(c.layers)),
                         PartSpec("rms_norm", dict(size=c.hidden, eps=1e-5), prefix="final."), "head.weight")

    register_architecture("ToyForCausalLM", ToyConfig, toy_plan)
    folder = write_random_model(str(tmp_path), dict(architectures=["ToyForCausalLM"], hidden=24, layers=3, vocab=50),
                                seed=1, std=0.2)
    runner, cache, model = open_runner(engine, folder, "float32", max_tokens=512, max_slots=3)
    assert [type(r).__name__ for r in model.cache_requests()] == ["StateRequest", "KeyValueRequest", "StateRequest"]
    seqs = [helpers.random_tokens(i, n, 50) for i, n in enumerate([12, 5])]
    whole = []
    for s in seqs:
        slot = cache.open_slot()
        whole.append(runner.step([entry(slot, s)]).clone())
        cache.close_slot(slot)
    slots = [cache.open_slot(), cache.open_slot()]              # reused slots: state starts at zero again
    got = [[], []]
    out = runner.step([entry(slots[0], seqs[0][:4]), entry(slots[1], seqs[1][:2])])
    got[0].append(out[:4])
    got[1].append(out[4:])
    for p in range(2, 12):
        live = [b for b in (0, 1) if p + (2 if b == 0 else 0) < len(seqs[b])]
        if not live:
            break
        step = [entry(slots[b], [seqs[b][p + (2 if b == 0 else 0)]]) for b in live]
        out = runner.step(step)
        for row, b in enumerate(live):
            got[b].append(out[row:row + 1])
    for b in (0, 1):
        assert torch.allclose(torch.cat(got[b]), whole[b], rtol=1e-5, atol=1e-6)


# --------------------------------------------------------------------------- layer order and windows as data
def _llama_like_plan(config, window=None, schedule=None):
    """The library's Llama plan with a window on every attention and another layer order."""
    import dataclasses
    from llama_rs_metal_b200.models.llama import llama_plan
    from llama_rs_metal_b200.parts import PartSpec
    plan = llama_plan(config)
    layers = []
    for layer in plan.layers:
        params = dict(layer.mixer.params, window=window)
        layers.append(layer.with_parts(mixer=PartSpec("attention", params, layer.mixer.prefix)))
    return dataclasses.replace(plan, layers=tuple(layers), schedule=tuple(schedule or plan.schedule))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_attention_in_a_whole_model_matches_the_plain_implementation(engine, tmp_path, dtype):
    """A window of 40 keys on every layer: the windowed cache group drops pages, prompts longer
    than the window and decoding across page boundaries must still match the oracle."""
    from llama_rs_metal_b200.config import LlamaConfig
    from llama_rs_metal_b200.engine.session import write_random_model
    from llama_rs_metal_b200.registry import register_architecture

    register_architecture("WindowedLlamaForTest", LlamaConfig, lambda c: _llama_like_plan(c, window=40))
    cfg = dict(helpers.TINY["B"]["config"], architectures=["WindowedLlamaForTest"], model_type="windowed_test")
    folder = write_random_model(str(tmp_path), cfg, seed=5, std=0.05, norm_std=0.1)
    plain_cfg, tensors = P.read_model(folder)
    runner, cache, model = open_runner(engine, folder, dtype, max_tokens=1024, max_slots=3)
    assert cache.kv_groups[0].request.window == 40
    seqs = [helpers.random_tokens(60 + i, n, 512) for i, n in enumerate([200, 30])]
    refs = [P.forward(plain_cfg, tensors, s, window=40).numpy() for s in seqs]
    slots = [cache.open_slot() for _ in seqs]
    prompts = [150, 10]
    out = runner.step([entry(sl, s[:p]) for sl, s, p in zip(slots, seqs, prompts)])
    helpers.assert_logits_close(out[:150].cpu(), refs[0][:150], dtype, "windowed prompt")
    helpers.assert_logits_close(out[150:].cpu(), refs[1][:10], dtype, "windowed short prompt")
    rows = [[], []]
    for step in range(50):
        live = [b for b in (0, 1) if prompts[b] + step < len(seqs[b])]
        out = runner.step([entry(slots[b], [seqs[b][prompts[b] + step]]) for b in live])
        for r, b in enumerate(live):
            rows[b].append(out[r:r + 1].clone())
    helpers.assert_logits_close(torch.cat(rows[0]).cpu(), refs[0][150:200], dtype, "windowed decoding")
    helpers.assert_logits_close(torch.cat(rows[1]).cpu(), refs[1][10:30], dtype, "windowed decoding, short")
    # only the pages that still hold visible positions are kept: 200 tokens, window 40 -> pages 2 and 3
    kept = (cache.kv_groups[0].table_host[slots[0]] >= 0).nonzero()[0].tolist()
    assert kept == [2, 3]


def test_a_schedule_may_run_a_layer_twice_and_share_another_layers_cache(engine, tmp_path):
    """Order of layers is data: layer 0, then layer 1 reading layer 0's keys and values, then
    layer 0 again on a cache entry of its own. Whole prompts and token-by-token decoding must
    agree bit for bit in float32, and the result must differ from the plain order."""
    from llama_rs_metal_b200.config import LlamaConfig
    from llama_rs_metal_b200.engine.session import write_random_model
    from llama_rs_metal_b200.parts import ScheduleEntry
    from llama_rs_metal_b200.registry import register_architecture

    order = [ScheduleEntry(0, 0), ScheduleEntry(1, 0, writes_cache=False), ScheduleEntry(0, 1)]
    register_architecture("ReorderedLlamaForTest", LlamaConfig, lambda c: _llama_like_plan(c, schedule=order))
    cfg = dict(helpers.TINY["A"]["config"], architectures=["ReorderedLlamaForTest"], model_type="reordered_test")
    folder = write_random_model(str(tmp_path / "re"), cfg, seed=2, std=0.1)
    plain_folder = write_random_model(str(tmp_path / "plain"), helpers.TINY["A"]["config"], seed=2, std=0.1)
    runner, cache, model = open_runner(engine, folder, "float32", max_tokens=512, max_slots=2)
    assert len(model.cache_requests()) == 2                       # two cache entries for three executed layers
    tokens = helpers.random_tokens(9, 80, 256)
    slot = cache.open_slot()
    whole = runner.step([entry(slot, tokens)]).clone()
    cache.close_slot(slot)
    slot = cache.open_slot()
    rows = [runner.step([entry(slot, tokens[:30])]).clone()]
    rows += [runner.step([entry(slot, [t])]).clone() for t in tokens[30:]]
    assert torch.equal(torch.cat(rows), whole)
    straight, cache2, _ = open_runner(engine, plain_folder, "float32", max_tokens=512, max_slots=2)
    other = straight.step([entry(cache2.open_slot(), tokens)])
    assert not torch.allclose(other, whole, atol=1e-3)


# --------------------------------------------------------------------------- other parts, defined here
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_feed_forward_position_norm_and_block_are_registered_from_outside(engine, tmp_path, dtype):
    """A feed-forward with routing (top-1 of three experts), a learned absolute position added to q
    and k, a LayerNorm with bias and a block that feeds mixer and feed-forward from one norm, all
    defined here and registered under new names: a model of them loads, steps with the library's
    attention, cache and step function, and agrees with a plain restatement, whole and cut into
    steps, alone and in a batch of unequal lengths. No file of the library changes."""
    from dataclasses import dataclass
    from llama_rs_metal_b200.config.base import read_int
    from llama_rs_metal_b200.engine.session import write_random_model
    from llama_rs_metal_b200.parts import (Block, FeedForward, LayerSpec, ModelPlan, Norm, PartSpec, PositionEncoding,
                                           ScheduleEntry)
    from llama_rs_metal_b200.registry import (register_architecture, register_block, register_feed_forward,
                                              register_norm, register_position_encoding)
    from llama_rs_metal_b200.weights import TensorSpec

    E, F_, H, HEADS, KV, D, MAXPOS = 3, 20, 40, 4, 2, 32, 96

    @register_feed_forward("toy_routed")
    class Routed(FeedForward):
        def __init__(self, hidden_size, experts, inner):
            self.h, self.e, self.f = hidden_size, experts, inner

        def tensors(self):
            return {"router.weight": TensorSpec((self.e, self.h)), "up.weight": TensorSpec((self.e, self.f, self.h)),
                    "down.weight": TensorSpec((self.e, self.h, self.f))}

        def bind(self, weights, runtime):
            self.w = {k: v.float() for k, v in weights.items()}

        def forward(self, x, ctx, residual):
            xs = x.float()
            prob = torch.softmax(xs @ self.w["router.weight"].T, dim=-1)        # router in float32
            best = prob.argmax(dim=-1)
            for e in range(self.e):
                rows = (best == e).nonzero().flatten()
                if rows.numel():
                    inner = torch.relu(xs[rows] @ self.w["up.weight"][e].T)
                    residual[rows] += (inner @ self.w["down.weight"][e].T) * prob[rows, e:e + 1]
            return residual

    @register_position_encoding("toy_learned")
    class Learned(PositionEncoding):
        def __init__(self, head_dim, positions):
            self.d, self.n = head_dim, positions

        def tensors(self):
            return {"table": TensorSpec((self.n, self.d))}

        def bind(self, weights, runtime):
            self.table = weights["table"]

        def rotary_table(self):
            return None

        def apply(self, q, k, ctx):
            add = self.table[ctx.positions.long()][:, None, :]
            return (q.float() + add.float()).to(q.dtype), (k.float() + add.float()).to(k.dtype)

    @register_norm("toy_layer_norm")
    class LayerNorm(Norm):
        def __init__(self, size, eps):
            self.size, self.eps = size, eps

        def tensors(self):
            return {"weight": TensorSpec((self.size,)), "bias": TensorSpec((self.size,))}

        def bind(self, weights, runtime):
            self.w, self.b, self.dtype = weights["weight"].float(), weights["bias"].float(), runtime.dtype

        def forward(self, hidden, ctx, rows=None):
            x = hidden if rows is None else hidden[rows.long()]
            return torch.nn.functional.layer_norm(x, (self.size,), self.w, self.b, self.eps).to(self.dtype)

    @register_block("toy_parallel")
    class Parallel(Block):
        def forward(self, hidden, ctx, cache):
            x = self.mixer_norm.forward(hidden, ctx)
            hidden = self.mixer.forward(x, ctx, cache, residual=hidden)
            return self.feed_forward.forward(x, ctx, residual=hidden)

    @dataclass(frozen=True)
    class Config:
        layers: int
        vocab: int

        @classmethod
        def from_dict(cls, d):
            return cls(read_int(d, "layers"), read_int(d, "vocab"))

        def to_dict(self):
            return dict(architectures=["ToyPartsForCausalLM"], layers=self.layers, vocab=self.vocab)

    def plan(c):
        layers = []
        for i in range(c.layers):
            p = f"l{i}."
            norm = PartSpec("toy_layer_norm", dict(size=H, eps=1e-4), prefix=p + "norm.")
            layers.append(LayerSpec(
                "toy_parallel",
                PartSpec("attention", dict(hidden_size=H, num_heads=HEADS, num_kv_heads=KV, head_dim=D,
                                           position=PartSpec("toy_learned", dict(head_dim=D, positions=MAXPOS))),
                         prefix=p + "attn."),
                PartSpec("toy_routed", dict(hidden_size=H, experts=E, inner=F_), prefix=p + "ff."), norm, norm))
        return ModelPlan(H, c.vocab, MAXPOS, "embed.weight", tuple(layers),
                         tuple(ScheduleEntry(i, i) for i in range(c.layers)),
                         PartSpec("toy_layer_norm", dict(size=H, eps=1e-4), prefix="final."), "head.weight")

    register_architecture("ToyPartsForCausalLM", Config, plan)
    folder = write_random_model(str(tmp_path), dict(architectures=["ToyPartsForCausalLM"], layers=2, vocab=70),
                                seed=3, std=0.3)
    _, w = P.read_model(folder)
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).double() for k, v in w.items()}

    margin = 1e-4 if dtype == "float32" else 0.015

    def oracle(tokens):
        """Logits, and how many leading rows are safe to compare: a router decision that hangs
        on less than `margin` may fall the other way in the engine's precision, and every later
        token sees that token through attention."""
        n = len(tokens)
        safe = n
        hidden = w["embed.weight"][torch.tensor(tokens)]
        ln = lambda x, p: torch.nn.functional.layer_norm(x, (H,), w[p + "weight"], w[p + "bias"], 1e-4)
        for i in range(2):
            p = f"l{i}."
            x = ln(hidden, p + "norm.")
            add = w[p + "attn.position.table"][:n][:, None, :]
            q = (x @ w[p + "attn.q_proj.weight"].T).view(n, HEADS, D) + add
            k = (x @ w[p + "attn.k_proj.weight"].T).view(n, KV, D) + add
            v = (x @ w[p + "attn.v_proj.weight"].T).view(n, KV, D)
            mixed = P.attention(q, k, v).reshape(n, HEADS * D) @ w[p + "attn.o_proj.weight"].T
            prob = torch.softmax(x @ w[p + "ff.router.weight"].T, dim=-1)
            best = prob.argmax(dim=-1)
            top2 = prob.topk(2, dim=-1).values
            close_call = ((top2[:, 0] - top2[:, 1]) < margin).nonzero().flatten()
            if close_call.numel():
                safe = min(safe, int(close_call[0]))
            routed = torch.zeros_like(hidden)
            for t in range(n):
                e = int(best[t])
                routed[t] = (torch.relu(x[t] @ w[p + "ff.up.weight"][e].T) @ w[p + "ff.down.weight"][e].T) * prob[t, e]
            hidden = hidden + mixed + routed
        return ln(hidden, "final.") @ w["head.weight"].T, safe

    runner, cache, model = open_runner(engine, folder, dtype, max_tokens=512, max_slots=3)
    seqs = [helpers.random_tokens(80 + i, n, 70) for i, n in enumerate([70, 9, 33])]
    refs, safe = zip(*[oracle(s) for s in seqs])
    assert sum(safe) >= 40, "the test's weights leave too few unambiguous router decisions"
    for s, ref, ok in zip(seqs, refs, safe):                         # each alone and whole
        slot = cache.open_slot()
        helpers.assert_logits_close(runner.step([entry(slot, s)]).cpu()[:ok], ref[:ok], dtype, "toy parts, whole")
        cache.close_slot(slot)
    slots = [cache.open_slot() for _ in seqs]                        # unequal prompts in one step, then one token each
    prompts = [40, 3, 20]
    out = runner.step([entry(sl, s[:p]) for sl, s, p in zip(slots, seqs, prompts)]).cpu()
    at = 0
    for s, ref, p, ok in zip(seqs, refs, prompts, safe):
        helpers.assert_logits_close(out[at:at + min(p, ok)], ref[:min(p, ok)], dtype, "toy parts, prompts in a batch")
        at += p
    for step in range(30):
        live = [b for b in range(3) if prompts[b] + step < len(seqs[b])]
        out = runner.step([entry(slots[b], [seqs[b][prompts[b] + step]]) for b in live]).cpu()
        for r, b in enumerate(live):
            if prompts[b] + step < safe[b]:
                helpers.assert_logits_close(out[r:r + 1], refs[b][prompts[b] + step][None], dtype, "toy parts, decoding")
        for b in range(3):
            if prompts[b] + step + 1 == len(seqs[b]):
                cache.close_slot(slots[b])


# --------------------------------------------------------------------------- portions and mixed steps
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_portions_and_mixed_steps_match_the_plain_implementation(engine, model_dirs, plain_models, name, dtype):
    """One step may bring several tokens onto a started sequence, and sequences that start may
    share a step with sequences that go on: cuts at 1, 2, 63, 64 and 65 tokens, a request that
    joins late, all compared with the plain implementation's whole sequences."""
    vocab = helpers.TINY[name]["config"]["vocab_size"]
    seqs = [helpers.random_tokens(300 + i, n, vocab) for i, n in enumerate([200, 131, 66])]
    refs = [P.forward(*plain_models[name], s).numpy() for s in seqs]
    runner, cache, _ = open_runner(engine, model_dirs[name], dtype)
    slots = [cache.open_slot() for _ in seqs]
    at = [0, 0, 0]
    plan = [  # tokens each sequence brings, step by step (0: it sits this step out)
        (1, 0, 0), (2, 63, 0), (63, 1, 0), (64, 2, 5), (65, 64, 1), (5, 1, 60),
    ]
    for step in plan:
        entries, rows = [], []
        for b, n in enumerate(step):
            n = min(n, len(seqs[b]) - at[b])
            if n > 0:
                entries.append(entry(slots[b], seqs[b][at[b]:at[b] + n]))
                rows.append((b, at[b], n))
                at[b] += n
        out = runner.step(entries).cpu()
        row = 0
        for b, first, n in rows:
            helpers.assert_logits_close(out[row:row + n], refs[b][first:first + n], dtype,
                                        f"sequence {b}, positions {first}..{first + n - 1}")
            row += n
    assert [cache.length(s) for s in slots] == at


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_portions_keep_the_pages_their_first_query_sees(engine, tmp_path, dtype):
    """A window of 40 keys and portions of 70 tokens: a portion's first query still sees keys
    that the sequence's new length would let go, so those pages stay until the step is over."""
    from llama_rs_metal_b200.config import LlamaConfig
    from llama_rs_metal_b200.engine.session import write_random_model
    from llama_rs_metal_b200.registry import register_architecture

    register_architecture("WindowedLlamaForTest", LlamaConfig, lambda c: _llama_like_plan(c, window=40))
    cfg = dict(helpers.TINY["B"]["config"], architectures=["WindowedLlamaForTest"], model_type="windowed_test")
    folder = write_random_model(str(tmp_path), cfg, seed=5, std=0.05, norm_std=0.1)
    plain_cfg, tensors = P.read_model(folder)
    runner, cache, _ = open_runner(engine, folder, dtype, max_tokens=1024, max_slots=2)
    tokens = helpers.random_tokens(61, 250, 512)
    ref = P.forward(plain_cfg, tensors, tokens, window=40).numpy()
    slot = cache.open_slot()
    at = 0
    for n in (30, 70, 70, 1, 1, 70, 8):
        out = runner.step([entry(slot, tokens[at:at + n])]).cpu()
        helpers.assert_logits_close(out, ref[at:at + n], dtype, f"windowed portion at {at}")
        at += n
    assert at == 250
    kept = (cache.kv_groups[0].table_host[slot] >= 0).nonzero()[0].tolist()
    assert kept == [3]  # the last portion's first query (position 242) sees keys from 203: page 3 on


# --------------------------------------------------------------------------- failures and memory
def test_a_device_status_poisons_the_session_until_reset(engine, model_dirs, plain_models):
    """What a kernel that gave up on a bounded wait leaves behind is a code in the status word.
    Written there from the host (no kernel is made to fail), it must stop the session before any
    logits are handed out, keep it stopped until reset, and leave a reset session exact again
    (crates/model-runtime/src/session.rs:156-159, 101)."""
    from llama_rs_metal_b200.errors import LlamaError, PoisonedError
    from llama_rs_metal_b200.kernels import gemm_dispatch
    model = engine.load(model_dirs["D"], dtype="bfloat16")
    session = model.session(context=256)
    tokens = helpers.random_tokens(4, 90, 2048)
    ref = P.forward(*plain_models["D"], tokens).numpy()
    good = session.prefill(tokens[:70]).clone()
    helpers.assert_logits_close(good.cpu().numpy()[None], ref[69:70], "bfloat16")
    session.reset()
    session.prefill(tokens[:20])
    gemm_dispatch.check_status()
    word = gemm_dispatch._status_word(engine.device)
    word.fill_(2)                                   # "gave up waiting for operand tiles"
    with pytest.raises(LlamaError, match="gave up waiting for operand tiles"):
        session.prefill(tokens[20:90])              # 70 rows: a portion through the tensor-core kernels
    assert int(word.item()) == 0                    # read and cleared
    with pytest.raises(PoisonedError):
        session.decode(5)
    with pytest.raises(PoisonedError):
        session.prefill([1, 2, 3])
    session.reset()
    assert session.tokens() == []
    assert torch.equal(session.prefill(tokens[:70]), good)
    # the same through the generation loop, where the captured decode step runs the kernels
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    session.reset()
    batch = model.session(context=128, max_batch=40)
    prompts = [helpers.random_tokens(50 + i, 5 + i % 9, 2048) for i in range(40)]
    options = GenerationOptions(max_tokens=4, sampling=Sampling(temperature=0.0))
    want = [r.tokens for r in batch.generate(prompts, options, stop_token_ids=())]
    word.fill_(3)
    with pytest.raises(LlamaError, match="gave up waiting"):
        batch.generate(prompts, options, stop_token_ids=())
    assert batch.runner.poisoned and batch.cache.slots.held == 0
    with pytest.raises(PoisonedError):
        batch.generate(prompts, options, stop_token_ids=())
    batch.reset()
    assert [r.tokens for r in batch.generate(prompts, options, stop_token_ids=())] == want


def test_a_replayed_graph_marks_the_status_word_for_reading(engine, model_dirs):
    """Kernels inside a replayed CUDA graph do not pass through their Python wrappers; the replay
    itself has to say that the status word must be read."""
    from llama_rs_metal_b200.kernels import gemm_dispatch
    runner, cache, _ = open_runner(engine, model_dirs["D"], "bfloat16", max_tokens=4096, max_slots=48)
    slots = [cache.open_slot() for _ in range(40)]
    runner.step([entry(s, helpers.random_tokens(s, 4 + s % 11, 2048), []) for s in slots])
    runner.step([entry(s, [7]) for s in slots])     # captures the decode step of 40 rows
    graph = next(iter(runner._graphs.values()))
    assert graph.reports_status                     # 40 rows: the O and down products run on tcgen05 in K slices
    gemm_dispatch.check_status()
    assert not gemm_dispatch._status_dirty
    runner.step([entry(s, [8]) for s in slots])     # a replay only
    assert gemm_dispatch._status_dirty
    gemm_dispatch.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_device_memory_is_constant_over_many_decode_steps(engine, model_dirs, dtype):
    """After warm-up, decoding allocates nothing more: three rounds of 64 steps leave the bytes
    in use where they were (crates/llama-rs/tests/sessions.rs:65-83)."""
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    model = engine.load(model_dirs["A"], dtype=dtype)
    session = model.session(context=128, max_batch=3)
    prompts = [helpers.random_tokens(i, 3 + i, 256) for i in range(3)]
    options = GenerationOptions(max_tokens=65, sampling=Sampling(temperature=0.0))
    for _ in range(2):                                             # warm-up: graphs (the prompt step's is
        session.generate(prompts, options, stop_token_ids=())      # captured the second time), staging buffers
    torch.cuda.synchronize()
    in_use, reserved = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        results = session.generate(prompts, options, stop_token_ids=())
        assert all(len(r.tokens) == 65 for r in results)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == in_use and torch.cuda.memory_reserved() == reserved
    assert torch.cuda.mem_get_info()[0] >= free_before             # nothing was taken from the driver either
    # and the runner keeps a bounded number of captured steps
    assert len(session.runner._graphs) <= session.runner.max_graphs


# --------------------------------------------------------------------------- reproducibility
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_forty_random_generations_one_step_ahead_equal_step_by_step(engine, model_dirs, dtype):
    """Random prompts, budgets, contexts, stop ids and sampling, forty times over: generation
    that keeps a step in flight (CUDA graphs, tokens fed on the device) and generation that waits
    for every token give the same tokens and reasons, in bfloat16 too. That needs results that do
    not depend on timing (no sums meeting by atomics), the same launch geometry with and without
    graphs, and a step in flight that is dropped when a stop token shrinks the batch."""
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    name = "D"
    vocab = helpers.TINY[name]["config"]["vocab_size"]
    model = engine.load(model_dirs[name], dtype=dtype)
    rng = np.random.default_rng(2024)
    sessions = {}
    for trial in range(40):
        max_batch = int(rng.choice([1, 3, 12]))
        context = int(rng.choice([48, 80, 200]))
        if (max_batch, context) not in sessions:
            ahead, plain = model.session(context=context, max_batch=max_batch), model.session(context=context, max_batch=max_batch)
            plain.runner.use_graphs = False
            sessions[(max_batch, context)] = (ahead, plain)
        ahead, plain = sessions[(max_batch, context)]
        count = int(rng.integers(1, 2 * max_batch + 2))
        prompts = [[int(t) for t in rng.integers(0, vocab, size=int(rng.integers(1, 40)))] for _ in range(count)]
        sampling = Sampling(temperature=0.0) if trial % 2 == 0 else \
            Sampling(temperature=float(rng.choice([0.7, 1.0])), top_k=0, top_p=1.0, seed=int(rng.integers(0, 1000)))
        options = GenerationOptions(max_tokens=int(rng.integers(1, 30)), sampling=sampling)
        free = plain.generate(prompts, options, stop_token_ids=())
        emitted = [t for r in free for t in r.tokens]
        stops = sorted({emitted[int(i)] for i in rng.integers(0, len(emitted), size=int(rng.integers(0, 4)))}) if emitted else []
        want = plain.generate(prompts, options, stop_token_ids=stops)
        got = ahead.generate(prompts, options, stop_token_ids=stops)
        assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in want], \
            f"trial {trial}: batch {max_batch}, context {context}, {count} prompts, stops {stops}"
        assert ahead.cache.slots.held == 0 and plain.cache.slots.held == 0


# --------------------------------------------------------------------------- the stated workloads
def test_tiny_b_workload_as_stated_with_temperature_sampling(engine, model_dirs, plain_models):
    """Five prompts of 1, 9, 33, 64 and 130 tokens (ids from seed 8), then 12 steps at temperature
    0.8 with sampling seed 9, in float32: every sampled token is the plain implementation's logits
    through the sampler's CPU twin (a different token only where two perturbed scores tie within
    rounding)."""
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    rng = np.random.default_rng(8)
    prompts = [[int(t) for t in rng.integers(0, 512, size=n)] for n in (1, 9, 33, 64, 130)]
    model = engine.load(model_dirs["B"], dtype="float32")
    session = model.session(context=256, max_batch=5)
    options = GenerationOptions(max_tokens=12, sampling=Sampling(temperature=0.8, top_k=0, top_p=1.0, seed=9))
    results = session.generate(prompts, options, stop_token_ids=())
    cfg, tensors = plain_models["B"]
    for request, (prompt, result) in enumerate(zip(prompts, results)):
        assert result.finish_reason == "length" and len(result.tokens) == 12
        seq = list(prompt)
        for step, token in enumerate(result.tokens):
            logits = P.forward(cfg, tensors, seq)[-1].numpy()
            scores = helpers.gumbel_twin(logits.tolist(), 0.8, 9, (request << 32) | step)
            assert scores[token] >= max(scores) - 1e-3, \
                f"request {request}, step {step}: sampled {token}, the twin draws {int(np.argmax(scores))}"
            seq.append(token)
    # the decoding positions go past original_max_position_embeddings = 64: all three branches of
    # the llama3 rule are in use (low, high and the smooth band between)
    from llama_rs_metal_b200.parts.rope import RotaryEmbedding
    spec = model.plan.layers[0].mixer.params["position"].params
    factors = [f0 / f for f0, f in zip(RotaryEmbedding(**dict(spec, scaling="default")).inverse_frequencies(),
                                       RotaryEmbedding(**spec).inverse_frequencies())]
    assert min(factors) == 1.0 and abs(max(factors) - 8.0) < 1e-9 and any(1.0 < f < 8.0 - 1e-9 for f in factors)


# --------------------------------------------------------------------------- another block, model-level scales
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_block_with_roles_of_its_own_and_scaled_embedding_and_logits(engine, tmp_path, dtype):
    """A block that norms each part's output before it joins the stream (two more norms per layer
    than the library's block has roles for), a scale on the embedding and one on the logits:
    registered here, built from a plan, stepped whole and in portions, compared with a plain
    restatement. The library's attention, feed-forward, norm, cache and step function run it as
    they are."""
    import dataclasses
    from llama_rs_metal_b200.config import LlamaConfig
    from llama_rs_metal_b200.engine.session import write_random_model
    from llama_rs_metal_b200.kernels import ops
    from llama_rs_metal_b200.models.llama import llama_plan
    from llama_rs_metal_b200.parts import Block, LayerSpec, PartSpec
    from llama_rs_metal_b200.registry import register_architecture, register_block

    @register_block("toy_sandwich")
    class Sandwich(Block):
        roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm",
                 "feed_forward_norm": "norm", "after_mixer_norm": "norm", "after_feed_forward_norm": "norm"}
        graph_safe = True

        def forward(self, hidden, ctx, cache):
            x = self.mixer_norm.forward(hidden, ctx)
            mixed = self.mixer.forward(x, ctx, cache, residual=torch.zeros_like(hidden))
            ops.add_(hidden, self.after_mixer_norm.forward(mixed, ctx))
            x = self.feed_forward_norm.forward(hidden, ctx)
            fed = self.feed_forward.forward(x, ctx, residual=torch.zeros_like(hidden))
            return ops.add_(hidden, self.after_feed_forward_norm.forward(fed, ctx))

    EMBED, LOGIT = 8.0, 0.25

    def plan(config):
        base = llama_plan(config)
        layers = []
        for i, layer in enumerate(base.layers):
            norm = layer.mixer_norm
            p = f"model.layers.{i}."
            layers.append(LayerSpec("toy_sandwich", parts=dict(
                layer.parts,
                after_mixer_norm=PartSpec(norm.kind, norm.params, prefix=p + "after_attention_norm."),
                after_feed_forward_norm=PartSpec(norm.kind, norm.params, prefix=p + "after_mlp_norm."))))
        return dataclasses.replace(base, layers=tuple(layers), embedding_scale=EMBED, logit_scale=LOGIT)

    register_architecture("SandwichLlamaForTest", LlamaConfig, plan)
    cfg = dict(helpers.TINY["B"]["config"], architectures=["SandwichLlamaForTest"], model_type="sandwich_test")
    folder = write_random_model(str(tmp_path), cfg, seed=21, std=0.05, norm_std=0.1)
    c, w = P.read_model(folder)
    Hq, Hk, d, eps = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"], c["rms_norm_eps"]
    inv = P.rope_inverse_frequencies(c, d)

    def oracle(tokens):
        n = len(tokens)
        hidden = P.embedding(w["model.embed_tokens.weight"], tokens) * EMBED
        for i in range(c["num_hidden_layers"]):
            p = f"model.layers.{i}."
            x = P.rms_norm(hidden, w[p + "input_layernorm.weight"], eps)
            q = P.rope(P.linear(x, w[p + "self_attn.q_proj.weight"]).view(n, Hq, d), range(n), inv, d)
            k = P.rope(P.linear(x, w[p + "self_attn.k_proj.weight"]).view(n, Hk, d), range(n), inv, d)
            v = P.linear(x, w[p + "self_attn.v_proj.weight"]).view(n, Hk, d)
            mixed = P.linear(P.attention(q, k, v).reshape(n, Hq * d), w[p + "self_attn.o_proj.weight"])
            hidden = hidden + P.rms_norm(mixed, w[p + "after_attention_norm.weight"], eps)
            x = P.rms_norm(hidden, w[p + "post_attention_layernorm.weight"], eps)
            fed = P.gated_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
            hidden = hidden + P.rms_norm(fed, w[p + "after_mlp_norm.weight"], eps)
        return P.linear(P.rms_norm(hidden, w["model.norm.weight"], eps), w["lm_head.weight"]) * LOGIT

    runner, cache, model = open_runner(engine, folder, dtype, max_tokens=512, max_slots=2)
    assert len(model.blocks[0].parts) == 6
    tokens = helpers.random_tokens(33, 90, 512)
    ref = oracle(tokens).numpy()
    plain = P.forward(c, w, tokens).numpy()
    assert np.abs(ref - plain).max() > 1e-2 * np.abs(plain).max()     # the arrangement and the scales matter
    slot = cache.open_slot()
    helpers.assert_logits_close(runner.step([entry(slot, tokens)]).cpu(), ref, dtype, "sandwich block, whole")
    cache.close_slot(slot)
    slot = cache.open_slot()
    rows = [runner.step([entry(slot, tokens[:40])]), runner.step([entry(slot, tokens[40:57])])]
    rows += [runner.step([entry(slot, [t])]) for t in tokens[57:]]
    helpers.assert_logits_close(torch.cat(rows).cpu(), ref, dtype, "sandwich block, in steps")


def test_a_windowed_model_generates_one_step_ahead(engine, tmp_path):
    """A model whose cache group has a window keeps the decode bookkeeping in arrays and the
    generation loop one step ahead like any other; tokens equal step-by-step generation."""
    from llama_rs_metal_b200 import GenerationOptions, Sampling
    from llama_rs_metal_b200.config import LlamaConfig
    from llama_rs_metal_b200.engine.session import write_random_model
    from llama_rs_metal_b200.registry import register_architecture
    register_architecture("WindowedLlamaForTest", LlamaConfig, lambda c: _llama_like_plan(c, window=40))
    cfg = dict(helpers.TINY["B"]["config"], architectures=["WindowedLlamaForTest"], model_type="windowed_test")
    folder = write_random_model(str(tmp_path), cfg, seed=5, std=0.05, norm_std=0.1)
    plain_cfg, tensors = P.read_model(folder)
    for dtype in ("float32", "bfloat16"):
        model = engine.load(folder, dtype=dtype)
        ahead, plain = model.session(context=256, max_batch=3), model.session(context=256, max_batch=3)
        plain.runner.use_graphs = False
        assert ahead.can_decode_ahead
        prompts = [helpers.random_tokens(70 + i, n, 512) for i, n in enumerate([3, 90, 45, 7])]
        options = GenerationOptions(max_tokens=100, sampling=Sampling(temperature=0.0))
        want = plain.generate(prompts, options, stop_token_ids=())
        got = ahead.generate(prompts, options, stop_token_ids=())
        assert [r.tokens for r in got] == [r.tokens for r in want]
        assert ahead.cache.held_pages() == [0]
        if dtype == "float32":
            seq = list(prompts[1])
            for token in want[1].tokens[:20]:
                logits = P.forward(plain_cfg, tensors, seq, window=40)[-1].numpy()
                best = int(np.argmax(logits))
                assert token == best or logits[best] - logits[token] <= 4e-5 * np.abs(logits).max()
                seq.append(token)


# --------------------------------------------------------------------------- short prompts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompt_steps_are_filled_to_whole_rows_and_replayed_from_a_graph(engine, model_dirs, plain_models, dtype):
    """A prompt step of a few hundred tokens is filled up to a whole number of 64 rows with a
    sequence of padding, so that steps of different sizes share a geometry; the second step of a
    geometry is captured in a CUDA graph and later ones replay it. Padding changes no result, and
    the replayed step gives the bits of the uncaptured one."""
    vocab = helpers.TINY["D"]["config"]["vocab_size"]
    runner, cache, _ = open_runner(engine, model_dirs["D"], dtype)
    assert runner.pads_prompts
    sets = [[helpers.random_tokens(400 + 10 * s + i, n, vocab) for i, n in enumerate(lengths)]
            for s, lengths in enumerate(([5, 70, 33], [9, 66, 30], [5, 70, 33], [33, 70, 5], [1, 127]))]
    sets[2] = sets[0]
    outs = []
    for prompts in sets:
        slots = [cache.open_slot() for _ in prompts]
        out = runner.step([entry(sl, p) for sl, p in zip(slots, prompts)]).clone()
        at = 0
        for p in prompts:
            ref = P.forward(*plain_models["D"], p).numpy()
            helpers.assert_logits_close(out[at:at + len(p)].cpu(), ref, dtype, f"prompt of {len(p)} in a filled step")
            at += len(p)
        assert out.shape[0] == at                                  # no row of padding comes back
        # decoding goes on from what the filled step stored
        nxt = runner.step([entry(slots[0], [3])]).cpu()
        ref = P.forward(*plain_models["D"], prompts[0] + [3]).numpy()
        helpers.assert_logits_close(nxt, ref[-1:], dtype, "decoding after a filled step")
        for sl in slots:
            cache.close_slot(sl)
        outs.append(out)
    prompt_graphs = [k for k in runner._graphs if k[0] == "prefill"]
    # wanted rows differ between the sets (108, 105, 108, 108, 128 logits), so three geometries were
    # seen; the third set repeats the first one's and is captured, the fourth has that geometry with
    # other lengths and replays the graph: whatever a step derives from its positions (the table of
    # rotation angles) has to be derived inside the graph
    assert len(prompt_graphs) == 1 and prompt_graphs[0][1] == 128
    assert torch.equal(outs[2], outs[0])                           # replayed = uncaptured, bit for bit
