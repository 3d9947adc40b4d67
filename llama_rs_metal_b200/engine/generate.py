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


def _run_batch(stepper, sampler, live: List[_Live], options, stop, context, cancelled, on_token) -> None:
    active = list(live)
    first = True
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
            entries = [StepEntry(seq.slot, [seq.pending], [0]) for seq in active]
            for seq in active:
                seq.pending = None
        logits = stepper.step(entries)
        picked = sampler.pick(
            logits,
            [seq.result.request for seq in active],
            [len(seq.result.tokens) for seq in active],
            [seq.result.prompt + seq.result.tokens for seq in active])
        check = getattr(stepper, "check_device_status", None)
        if check is not None:
            check()  # the pick above already synchronized with the device
        if len(picked) != len(active):
            raise InvalidError("sampler returned a different number of tokens than rows")
        still = []
        for seq, token in zip(active, picked):
            token = int(token)
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
        active = still
