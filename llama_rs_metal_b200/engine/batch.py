"""What one step carries: its entries as given, and the packed device-side description."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..runtime import Runtime


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the places among
    these tokens (0-based) whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepContext:
    """Device-side description of a step, read by every part.

    T tokens of B sequences are packed one sequence after another.
    """

    runtime: Runtime
    # "prefill": every sequence starts at position 0 (attention may read the step's own keys);
    # "decode": one token onto each started sequence; "extend": anything else (several tokens
    # onto started sequences, or a mix): keys are stored first, attention reads the cache
    phase: str
    num_tokens: int
    num_seqs: int
    max_seq_len: int  # most tokens one sequence brings this step
    max_kv_len: int  # longest sequence after this step, or an upper bound of it (launch geometry only)
    token_ids: torch.Tensor  # int32 [T]
    positions: torch.Tensor  # int32 [T]
    seq_of_token: torch.Tensor  # int32 [T]
    cu_seqlens: torch.Tensor  # int32 [B+1]
    slots: torch.Tensor  # int32 [B]
    kv_lens: torch.Tensor  # int32 [B], lengths after this step
    wanted_rows: torch.Tensor  # int32 [n], packed row numbers whose logits are wanted
    dest_rows: List[torch.Tensor] = field(default_factory=list)  # per key/value group: int32 [T]
    entry: Any = None  # the schedule entry being run
    fresh_kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)
    # Partial sums [n, T, h] (float32) that belong to the residual stream but are not added to it
    # yet: the K slices of a narrow product, which the next norm adds in its own pass instead of
    # atomics meeting in memory. A part may leave them only while `may_defer` is set, which a
    # block does right before it passes the part's output through a norm with `folds_pending`;
    # `next_folds_pending` tells a block whether whatever reads the stream after it does so.
    pending: Any = None
    scratch: Dict[Any, Any] = field(default_factory=dict)  # what kernels' dispatchers keep for the length of a step
    kv_fill: int = 4  # mean sequence length in quarters of the longest, rounded up (launch geometry only)
    # int32 [B]: the sequences by falling length after this step (ties by number), brought with the
    # step's other arrays so that a kernel may read it before it waits for the kernels ahead of it
    longest_first: Optional[torch.Tensor] = None
    may_defer: bool = False
    next_folds_pending: bool = False

    def take_pending(self):
        """The pending partial sums (the caller adds them); none are pending afterwards."""
        pending, self.pending = self.pending, None
        return pending

    def settle(self, residual: torch.Tensor) -> torch.Tensor:
        """Add pending partial sums into `residual` now (for a reader that cannot fold them)."""
        pending = self.take_pending()
        if pending is not None:
            from ..kernels import ops
            ops.add_planes_(residual, pending)
        return residual


def pack_host(entries: Sequence[StepEntry], lengths_before: Sequence[int], dest_rows=(), pad_to: int = 0):
    """The step's int32 arrays in one host buffer, laid out as
    [token ids T | positions T | sequence of token T | cu_seqlens B+1 | slots B | kv lengths B |
     sequences longest first B | wanted rows n | destination rows T per key/value group].

    The order by length is made here, on the host, because kernels read it before they wait for
    the kernels ahead of them: only what a copy brought before the step's first kernel is safe
    to read there.

    With `pad_to` > the step's tokens (a prompt step only) the step is filled up to that many
    rows with a sequence of padding of its own: token 0 at positions 0, 1, ..., stored nowhere
    (destination -1), in no slot (-1), wanted by nobody. T and B then count it, so that steps of
    different sizes share one launch geometry; rows do not depend on one another, so padding
    changes no result."""
    counts = [len(e.tokens) for e in entries]
    real_T, real_B = sum(counts), len(entries)
    padding = max(0, pad_to - real_T)
    T, B = real_T + padding, real_B + (1 if padding else 0)
    n_want = sum(len(e.want) for e in entries)
    base = 3 * T + (B + 1) + 3 * B + n_want
    host = np.empty(base + T * len(dest_rows), dtype=np.int32)
    for g, rows in enumerate(dest_rows):
        host[base + g * T:base + g * T + real_T] = rows
        host[base + g * T + real_T:base + (g + 1) * T] = -1
    token_ids, positions, seq_of = host[:T], host[T:2 * T], host[2 * T:3 * T]
    o = 3 * T
    cu, slots, kv_lens, longest_first, wanted = host[o:o + B + 1], host[o + B + 1:o + 2 * B + 1], \
        host[o + 2 * B + 1:o + 3 * B + 1], host[o + 3 * B + 1:o + 4 * B + 1], host[o + 4 * B + 1:base]
    if padding:
        token_ids[real_T:] = 0
        positions[real_T:] = np.arange(padding, dtype=np.int32)
        seq_of[real_T:] = real_B
        cu[B] = T
        slots[real_B] = -1
        kv_lens[real_B] = padding
        counts = counts + [padding]
    at, w = 0, 0
    cu[0] = 0
    for b, (e, before) in enumerate(zip(entries, lengths_before)):
        n = counts[b]
        token_ids[at:at + n] = np.asarray(e.tokens, dtype=np.int64)
        positions[at:at + n] = np.arange(before, before + n, dtype=np.int32)
        seq_of[at:at + n] = b
        slots[b] = e.slot
        kv_lens[b] = before + n
        for p in e.want:
            wanted[w] = at + p
            w += 1
        at += n
        cu[b + 1] = at
    longest_first[:] = np.argsort(-kv_lens, kind="stable")
    return host, T, B, n_want, max(counts), int(kv_lens.max())


def context_over(dev: torch.Tensor, runtime: Runtime, phase: str, T: int, B: int, n_want: int,
                 max_seq_len: int, max_kv_len: int, groups: int = 0, kv_fill: int = 4) -> StepContext:
    """A StepContext whose arrays are slices of `dev`, a device copy of pack_host's buffer."""
    o = 3 * T
    base = o + 4 * B + 1 + n_want
    return StepContext(
        dest_rows=[dev[base + g * T:base + (g + 1) * T] for g in range(groups)],
        runtime=runtime, phase=phase, num_tokens=T, num_seqs=B, max_seq_len=max_seq_len,
        max_kv_len=max_kv_len, kv_fill=kv_fill,
        token_ids=dev[:T], positions=dev[T:2 * T], seq_of_token=dev[2 * T:3 * T],
        cu_seqlens=dev[o:o + B + 1], slots=dev[o + B + 1:o + 2 * B + 1],
        kv_lens=dev[o + 2 * B + 1:o + 3 * B + 1], longest_first=dev[o + 3 * B + 1:o + 4 * B + 1],
        wanted_rows=dev[o + 4 * B + 1:base])


def pack_step(entries: Sequence[StepEntry], lengths_before: Sequence[int], runtime: Runtime,
              phase: str, dest_rows=(), pad_to: int = 0) -> StepContext:
    """Build the packed int32 arrays on the host and copy them to the device in one transfer."""
    host, T, B, n_want, max_seq_len, max_kv_len = pack_host(entries, lengths_before, dest_rows, pad_to)
    device = runtime.device
    if device.type == "cuda":
        dev = torch.from_numpy(host).pin_memory().to(device, non_blocking=True)
    else:
        dev = torch.from_numpy(host).to(device)
    return context_over(dev, runtime, phase, T, B, n_want, max_seq_len, max_kv_len, len(dest_rows))
