"""Token choice for a batch of rows: on the device where a kernel exists, else on the host."""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..errors import OptionsError
from ..kernels import ops
from .host import SplitMix64, sample_host
from .options import Sampling


class DevicePick:
    """How a step's tokens are chosen on the device: greedy (`temperature` None) or a draw from
    softmax(logits / temperature) whose noise is keyed by (seed, keys[row]). Called on logits it
    enqueues the choice and returns int32 [rows] ids without waiting; a stepper that reads the
    fields instead can choose inside the head product and never write the logits."""

    def __init__(self, temperature, seed: int, keys: Sequence[int]):
        self.temperature, self.seed, self.keys = temperature, seed, list(keys)

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        if self.temperature is None:
            ready = getattr(logits, "greedy_ids", None)
            return ready if ready is not None and ready.shape[0] == logits.shape[0] else ops.argmax_rows(logits)
        keys = torch.tensor(self.keys, dtype=torch.int64).pin_memory().to(logits.device, non_blocking=True)
        return ops.sample_gumbel_rows(logits, self.temperature, self.seed, keys)


class BatchSampler:
    """Picks one token per row of a step's logits.

    Greedy: device argmax, lowest id on ties; a row with non-finite logits is an
    error ("invalid GPU logits", crates/llama-rs/src/generation.rs:33-40).
    Plain temperature (no top-k/top-p/penalty): device Gumbel-max, keyed by
    (seed, request, step) so a row's draw does not depend on its batch.
    Anything else: the reference's host sampler on logits copied back, one
    SplitMix64 stream per request seeded with seed + request number.
    """

    def __init__(self, options: Sampling):
        options.validate()
        self.options = options
        self._rngs = {}

    def device_picker(self, requests: Sequence[int], steps: Sequence[int]):
        """For greedy and plain-temperature sampling: a function logits -> int32 [rows] device
        tensor of chosen ids that enqueues work but never waits for the device; None for the
        host sampler. -1 in its result marks a row with non-finite logits."""
        o = self.options
        keys = [(r << 32) | s for r, s in zip(requests, steps)]
        if o.greedy:
            return DevicePick(None, 0, keys)
        if o.plain_temperature:
            return DevicePick(o.temperature, o.seed, keys)
        return None

    def pick(self, logits: torch.Tensor, requests: Sequence[int], steps: Sequence[int],
             histories: Sequence[Sequence[int]]) -> List[int]:
        o = self.options
        if o.greedy:
            ready = getattr(logits, "greedy_ids", None)  # a decode step computes it in its graph
            ids = (ready if ready is not None and ready.shape[0] == logits.shape[0]
                   else ops.argmax_rows(logits)).tolist()
            if any(i < 0 for i in ids):
                raise OptionsError("invalid GPU logits")
            return ids
        if o.plain_temperature:
            keys = torch.tensor([(r << 32) | s for r, s in zip(requests, steps)], dtype=torch.int64)
            keys = keys.to(logits.device)
            ids = ops.sample_gumbel_rows(logits, o.temperature, o.seed, keys).tolist()
            if any(i < 0 for i in ids):
                raise OptionsError("invalid GPU logits")
            return ids
        rows = logits.detach().to("cpu").numpy()
        out = []
        for row, request, history in zip(rows, requests, histories):
            rng = self._rngs.setdefault(request, SplitMix64(o.seed + request))
            out.append(sample_host(row, history, rng, o))
        return out
