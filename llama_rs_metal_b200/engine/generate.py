"""The generation loop: batches of unequal prompts, stop tokens, early finishers.

Per sequence it takes the reference's decisions in the reference's order
(crates/llama-rs/src/generation.rs:14-70): cancelled -> "cancelled"; budget
used up -> "length"; a pending token that no longer fits -> "context"; sample;
a stop id ends the sequence with "eos" and is neither emitted, counted nor fed;
otherwise the token is emitted and becomes pending. The last emitted token is
never fed, so N tokens cost one prefill and N-1 decode steps.

Across sequences: requests are cut into batches in the order given; a batch's
prompts run in one step, then each unfinished sequence gets one token per step;
a finished sequence leaves the batch and gives its slot back at once; when a
batch is empty the next one starts, reusing those slots.

The loop owns no device code: it drives a `stepper` (open_slot, close_slot,
step) and a `sampler` (pick), so its decisions are testable with stand-ins.
A stepper that can enqueue a decode step whose tokens are still on the device
(`can_decode_ahead`, `decode_ahead`) and a sampler that can choose on the device
(`device_picker`) are driven one step ahead of the host; the results are the same.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Iterable, List, Optional, Sequence

from ..errors import CancelledError, ContextError, InvalidError, OptionsError
from ..sampling.options import GenerationOptions
from .batch import StepEntry


@dataclass
class GenerationResult:
    request: int
    prompt: List[int]
    tokens: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None  # "eos" | "length" | "context" | "cancelled"


@dataclass
class _Live:
    result: GenerationResult
    slot: int
    pending: Optional[int] = None

    @property
    def cached(self) -> int:
        """Tokens the cache holds for this sequence (the pending one is not yet fed)."""
        return len(self.result.prompt) + len(self.result.tokens) - (1 if self.pending is not None else 0)


def plan_batches(prompt_lengths: Sequence[int], max_batch: int, token_budget: int,
                 page_size: int, max_new_tokens: int, context: int) -> List[List[int]]:
    """Cut requests, in order, into batches that fit `max_batch` slots and the cache's tokens.

    A request is charged for the most it can ever hold: prompt + max_new_tokens - 1
    (the last token is never fed), capped by the context, rounded up to whole pages.
    """
    batches, current, used = [], [], 0
    for i, n in enumerate(prompt_lengths):
        most = min(context, n + max_new_tokens - 1)
        cost = -(-max(most, n) // page_size) * page_size
        if cost > token_budget:
            raise ContextError(token_budget, cost)
        if current and (len(current) >= max_batch or used + cost > token_budget):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += cost
    if current:
        batches.append(current)
    return batches


def generate(stepper, sampler, prompts: Sequence[Sequence[int]], options: GenerationOptions,
             stop_token_ids: Iterable[int] = (), max_batch: int = 64, context: int = 1 << 30,
             token_budget: int = 1 << 40, page_size: int = 64,
             cancelled: Callable[[], bool] = lambda: False,
             on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
    """Generate for every prompt; results come back in the order of `prompts`."""
    options.validate()
    if max_batch <= 0:
        raise OptionsError("max_batch must be positive")
    stop = frozenset(int(t) for t in stop_token_ids)
    results = []
    for i, prompt in enumerate(prompts):
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise OptionsError("prompt must contain at least one token")  # llama-rs session.rs:48-52
        if len(prompt) > context:
            raise ContextError(context, len(prompt))
        results.append(GenerationResult(request=i, prompt=prompt))
    if cancelled():
        raise CancelledError("cancelled before generation started")

    batches = plan_batches([len(r.prompt) for r in results], max_batch, token_budget, page_size,
                           options.max_tokens, context)
    for members in batches:
        live = [_Live(results[i], stepper.open_slot()) for i in members]
        try:
            _run_batch(stepper, sampler, live, options, stop, context, cancelled, on_token)
        finally:
            for seq in live:  # only those still holding a slot (an error ended the batch)
                if seq.slot is not None:
                    stepper.close_slot(seq.slot)
                    seq.slot = None
    return results


def _finish(stepper, seq: _Live, reason: str) -> None:
    seq.result.finish_reason = reason
    seq.pending = None
    stepper.close_slot(seq.slot)  # given back at once: the next batch may take it
    seq.slot = None


def _settle(stepper, seqs: List[_Live], picked: Sequence[int], options, stop, on_token) -> List[_Live]:
    """Take one chosen token per sequence: a stop id ends it, else the token is emitted and
    becomes pending unless the budget is used up. Returns the sequences that go on."""
    if len(picked) != len(seqs):
        raise InvalidError("sampler returned a different number of tokens than rows")
    still = []
    for seq, token in zip(seqs, picked):
        token = int(token)
        if token < 0:
            raise OptionsError("invalid GPU logits")  # a row without a finite maximum
        if token in stop:
            _finish(stepper, seq, "eos")  # not emitted, not counted, not fed
            continue
        seq.result.tokens.append(token)
        if on_token is not None:
            on_token(seq.result.request, token)
        if len(seq.result.tokens) >= options.max_tokens:
            _finish(stepper, seq, "length")
            continue
        seq.pending = token
        still.append(seq)
    return still


def _run_batch(stepper, sampler, live: List[_Live], options, stop, context, cancelled, on_token) -> None:
    active = list(live)
    first = True
    check = getattr(stepper, "check_device_status", None)
    run_ahead = (getattr(stepper, "can_decode_ahead", False) and hasattr(sampler, "device_picker")
                 and sampler.device_picker([0], [0]) is not None)
    while active:
        if cancelled():
            for seq in active:
                _finish(stepper, seq, "cancelled")
            return
        if first:
            entries = [StepEntry(seq.slot, seq.result.prompt, [len(seq.result.prompt) - 1])
                       for seq in active]
            first = False
        else:
            # a pending token that would not fit ends its sequence (generation.rs:24-27)
            fitting = []
            for seq in active:
                if seq.cached >= context:
                    _finish(stepper, seq, "context")
                else:
                    fitting.append(seq)
            active = fitting
            if not active:
                return
            if run_ahead:
                active = _decode_ahead(stepper, sampler, active, options, stop, context, cancelled, on_token)
                continue
            entries = [StepEntry(seq.slot, [seq.pending], [0]) for seq in active]
            for seq in active:
                seq.pending = None
        requests = [seq.result.request for seq in active]
        steps = [len(seq.result.tokens) for seq in active]
        device = sampler.device_picker(requests, steps) if hasattr(sampler, "device_picker") else None
        if device is not None and hasattr(stepper, "step_pick"):
            # tokens only: the step chooses on the device and writes no logits
            picked = stepper.step_pick(entries, device)
        else:
            logits = stepper.step(entries)
            picked = sampler.pick(logits, requests, steps,
                                  [seq.result.prompt + seq.result.tokens for seq in active])
        if check is not None:
            check()  # the pick above already synchronized with the device
        active = _settle(stepper, active, picked, options, stop, on_token)


def _decode_ahead(stepper, sampler, active: List[_Live], options, stop, context, cancelled, on_token) -> List[_Live]:
    """Decode steps for a set of sequences that stays the same, with one step always in flight.

    The step after the current one is enqueued before the host has seen the current step's
    tokens: it takes them from the device. What the host can foresee (the token budget, the
    context) decides whether that next step may be enqueued at all; a stop token it cannot
    foresee, so when one ends a sequence the step already in flight has carried that sequence
    one token too far, in a batch that the plain loop would not have formed. Where the stepper
    can take a step back (`can_rewind`: keys and values are just written again) the step in
    flight is dropped whole and the caller runs it again for the smaller set, so every token
    comes from exactly the batches the plain loop runs and the results are the same bit for
    bit. Otherwise (sequences with fixed-size state) only the ended sequence's row is dropped
    (rows do not depend on one another beyond rounding, and the slot is closed anyway) and the
    other rows of that step count as usual. The decisions per sequence are those of the plain
    loop, in its order. Returns the sequences that go on, each with its pending token.
    """
    check = getattr(stepper, "check_device_status", None)
    slots = [seq.slot for seq in active]
    requests = [seq.result.request for seq in active]

    def picker(offset: int):
        return sampler.device_picker(requests, [len(seq.result.tokens) + offset for seq in active])

    tokens = [seq.pending for seq in active]
    for seq in active:
        seq.pending = None
    current = stepper.decode_ahead(slots, tokens, None, picker(0))
    while True:
        # may every sequence take one more step after this one, as far as the host can tell?
        foreseeable = not cancelled() and all(
            len(seq.result.tokens) + 1 < options.max_tokens and seq.cached < context for seq in active)
        following = stepper.decode_ahead(slots, None, current, picker(1)) if foreseeable else None
        picked = current.ids()
        if check is not None:
            check()
        still = _settle(stepper, active, picked, options, stop, on_token)
        if following is None:
            return still
        if len(still) == len(active):
            for seq in active:
                seq.pending = None  # fed from the device by the step in flight
            current = following
            continue
        # a stop token ended some: the step in flight still carried them
        if getattr(stepper, "can_rewind", False):
            if still:
                stepper.rewind([seq.slot for seq in still], 1)  # that step never happened
            return still  # each with the token it just emitted pending, to be fed again
        picked = following.ids()
        if check is not None:
            check()
        row_of = {id(seq): row for row, seq in enumerate(active)}
        for seq in still:
            seq.pending = None
        return _settle(stepper, still, [picked[row_of[id(seq)]] for seq in still], options, stop, on_token)
