"""The step function: run the tokens a step brings, as one batch, from the cache.

A step is a list of entries, one per sequence, each bringing one or more tokens
that go on from where its sequence stands. Three phases share one forward pass:
every sequence at its first token is a *prefill* step (whole prompts of unequal
lengths; attention reads the step's own keys); every sequence going on by
exactly one token is a *decode* step; anything else (several tokens onto a
started sequence, as the reference's prefill on a session with history does,
crates/model-runtime/src/session.rs:105-164, or a mix of the above) is an
*extend* step: keys and values are stored first and attention reads the cache.
Everything is checked before anything is launched or changed, so a rejected
step leaves the cache as it was (the reference validates before submitting for
the same reason, session.rs:114-130). Sequences' lengths advance only after
the step's kernels are enqueued.

A decode step's launches are captured once per (batch size, length bucket) in
a CUDA graph and replayed: its int32 inputs live in a static device buffer
that each step overwrites with one host-to-device copy. Launch geometry
depends on the lengths only through the bucket, with or without graphs, so
both ways compute the same bits.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import Cache
from ..errors import InvalidError, PoisonedError, UnsupportedError
from ..kernels import ops
from ..runtime import Runtime
from .batch import StepEntry, context_over, pack_host
from .model import DecoderModel


def classify_step(entries: Sequence[StepEntry], lengths_before: Sequence[int]) -> str:
    """ "prefill", "decode" or "extend"; raises for an empty or malformed step."""
    if not entries:
        raise InvalidError("a step needs at least one entry")
    if any(len(e.tokens) == 0 for e in entries):
        raise InvalidError("every entry of a step brings at least one token")
    if all(n == 0 for n in lengths_before):
        return "prefill"
    if all(n > 0 for n in lengths_before) and all(len(e.tokens) == 1 for e in entries):
        return "decode"
    return "extend"


def validate_entries(entries: Sequence[StepEntry], vocab_size: int) -> None:
    seen = set()
    for e in entries:
        if e.slot in seen:
            raise InvalidError(f"slot {e.slot} appears twice in one step")
        seen.add(e.slot)
        for t in e.tokens:
            if not 0 <= int(t) < vocab_size:
                raise InvalidError("token outside vocabulary")  # session.rs:125-130
        for p in e.want:
            if not 0 <= int(p) < len(e.tokens):
                raise InvalidError(f"wanted place {p} is outside the {len(e.tokens)} tokens of the entry")


def _tell_profiler(before: Sequence[int], counts: Sequence[int], phase: str = "") -> None:
    """What the per-kernel timing cannot read off the kernels' arguments: how many cached tokens
    the step's attention reads and how many (query, key) pairs its causal triangle has."""
    from ..kernels import profile
    if profile.enabled:
        profile.hints["phase"] = phase
        profile.hints["kv_tokens"] = float(sum(b + n for b, n in zip(before, counts)))
        profile.hints["pairs"] = float(sum(n * b + n * (n + 1) // 2 for b, n in zip(before, counts)))


def fill_class(lengths) -> int:
    """How unequal the sequences of a decode step are: their mean length in quarters of the longest,
    rounded up (4: about equal, 1: one long sequence among short ones). Decode attention sizes its
    clusters by it; it is part of a captured step's geometry."""
    longest = int(max(lengths)) if len(lengths) else 0
    if longest <= 0:
        return 4
    mean = float(sum(int(n) for n in lengths)) / len(lengths)
    return max(1, min(4, -(-int(4 * mean) // longest)))


def length_bucket(n: int) -> int:
    """Launch geometry of decode attention depends on the longest sequence only through this."""
    bucket = 256
    while bucket < n:
        bucket *= 2
    return bucket


class _StepGraph:
    """One captured step of a fixed geometry: static inputs, the graph, and what it leaves: float32
    logits [wanted, vocab] with their greedy choice, or (for a caller that only wants tokens,
    `choice` = (temperature or None, seed)) just the chosen ids, picked in the head product's
    epilogue where a kernel can. A decode step has one token and one wanted row per sequence; a
    short prompt step is filled up to a whole number of 64 rows (see pack_host)."""

    RING = 4

    def __init__(self, runner: "StepRunner", phase: str, tokens: int, seqs: int, wanted: int, max_seq_len: int,
                 max_kv_len: int, choice=None, kv_fill: int = 4):
        rt = runner.runtime
        self.batch, self.choice = seqs, choice
        groups = len(runner.cache.kv_groups)
        self.size = (3 + groups) * tokens + 4 * seqs + 1 + wanted  # pack_host's layout
        # behind it, 8-byte aligned: one int64 key per wanted row for the noise of temperature sampling
        self.keys_at = self.size + (self.size & 1)
        total = self.keys_at + 2 * max(wanted, 1)
        self.static = torch.zeros(total, dtype=torch.int32, device=rt.device)
        self.keys = self.static[self.keys_at:self.keys_at + 2 * wanted].view(torch.int64)
        self.ctx = context_over(self.static, rt, phase, tokens, seqs, wanted, max_seq_len, max_kv_len, groups, kv_fill)
        self.pinned = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.ids: Optional[torch.Tensor] = None  # int32 [B]: the chosen tokens (graphs with a `choice`)
        self.events = [torch.cuda.Event() for _ in range(self.RING)]
        self.turn = 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.greedy: Optional[torch.Tensor] = None  # int32 [B]: argmax of every row, part of the graph
        self.launches = 0
        self.reports_status = False  # the graph holds kernels that write the device status word

    def upload(self, host: np.ndarray, keys: Optional[Sequence[int]] = None) -> None:
        i = self.turn % self.RING
        self.turn += 1
        self.events[i].synchronize()  # the copy that last used this staging buffer is done
        staged = self.pinned[i].numpy()
        staged[:self.size] = host
        if keys is not None:
            staged[self.keys_at:self.keys_at + 2 * len(keys)].view(np.int64)[:] = keys
        self.static.copy_(self.pinned[i], non_blocking=True)
        self.events[i].record()


class PendingPicks:
    """Token ids a step chose on the device, on their way to a pinned host buffer."""

    def __init__(self, capacity: int):
        self.host = torch.zeros(capacity, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.device_ids: Optional[torch.Tensor] = None
        self.batch = 0

    def launch(self, device_ids: torch.Tensor, batch: int) -> None:
        self.device_ids, self.batch = device_ids, batch
        self.host[:batch].copy_(device_ids, non_blocking=True)
        self.event.record()

    def ids(self) -> List[int]:
        """The chosen ids (waits for the step that chose them, not for later ones)."""
        self.event.synchronize()
        return self.host[:self.batch].tolist()


class StepRunner:
    """Binds a model and a cache and runs steps on the current CUDA stream."""

    def __init__(self, model: DecoderModel, cache: Cache, runtime: Runtime, use_graphs: bool = True):
        self.model, self.cache, self.runtime = model, cache, runtime
        self.poisoned = False
        self.steps_run = 0
        from ..kernels import profile
        # per-kernel timing (LRM_PROFILE=1) needs every launch to pass through its wrapper
        self.use_graphs = (use_graphs and runtime.device.type == "cuda" and model.graph_safe
                           and not profile.enabled)
        # captured decode steps by (batch size, length bucket), least recently used first; each
        # holds its own [batch, vocab] logits, so only the newest `max_graphs` are kept
        self._graphs: "OrderedDict[Tuple, _StepGraph]" = OrderedDict()
        self.max_graphs = 32
        # Short prompt steps are filled up to whole 64 rows (with or without graphs, so that both ways
        # launch the same kernels on the same shapes): steps of a few hundred tokens are bound by the
        # host's time per launch, and a geometry seen for the second time is captured and replayed.
        # Only for models whose parts never look at the step's arrays on the host.
        self.pads_prompts = model.graph_safe
        self._prompt_shapes_seen = set()
        self._pool = None
        self.last_launches = 0  # kernels of this library launched by the last step
        # pinned buffers for the ids of steps that do not wait (two are in flight at most)
        self._pending_ring: List[PendingPicks] = []
        self._pending_turn = 0

    # -- the public step ----------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], borrow: bool = False) -> torch.Tensor:
        """float32 logits [wanted places, vocab] on the device, in entry order then `want` order.

        With `borrow` the result may be a buffer the next step overwrites (the
        generation loop samples from it at once); otherwise it is the caller's. A borrowed
        result of a decode step that wants every row carries `greedy_ids`, the int32 argmax
        of each row (lowest id on ties, -1 for a row with a non-finite logit).
        """
        if self.poisoned:
            raise PoisonedError("a device error poisoned this session; reset it")
        entries = list(entries)
        cache = self.cache
        if self.use_graphs and entries and all(len(e.tokens) == 1 for e in entries):
            logits = self._decode_vectorized(entries, borrow)
            if logits is not None:
                return logits
        return self._run(entries, None, borrow)

    def step_pick(self, entries: Sequence[StepEntry], picker) -> List[int]:
        """A step for a caller that wants tokens, not logits: runs the entries like step() and
        returns, on the host, the token chosen at every wanted place (entry order, then `want`
        order) by `picker` (a sampling.device.DevicePick: greedy, or temperature sampling with one
        key per wanted place). The head product chooses in its epilogue where a kernel can, so no
        logits are written. -1 marks a place whose logits were not finite."""
        if self.poisoned:
            raise PoisonedError("a device error poisoned this session; reset it")
        entries = list(entries)
        cache = self.cache
        if (self.use_graphs and entries and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
                and all(cache.open_mask[e.slot] and cache.lengths[e.slot] > 0 for e in entries
                        if 0 <= e.slot < cache.max_slots)):
            return self.decode_ahead([e.slot for e in entries], [e.tokens[0] for e in entries], None, picker).ids()
        return self._run(entries, picker, True).tolist()

    PROMPT_PAD_LIMIT = 1024  # prompt steps of up to this many tokens are filled up to whole 64 rows

    def _run(self, entries: List[StepEntry], picker, borrow: bool) -> torch.Tensor:
        """The general path of step() (picker None: logits) and step_pick() (chosen ids)."""
        cache = self.cache
        validate_entries(entries, self.model.plan.vocab_size)
        before = [cache.length(e.slot) for e in entries]
        phase = classify_step(entries, before)
        counts = [len(e.tokens) for e in entries]
        if phase == "prefill":  # attention reads the step's own keys: the cache keeps what later steps see
            growth = [(e.slot, n + c) for e, n, c in zip(entries, before, counts)]
        else:                   # attention reads the cache from each portion's first query on
            growth = [(e.slot, n + c, n) for e, n, c in zip(entries, before, counts)]
        cache.check_growth(growth)  # raises before anything changes
        cache.grow(growth)
        cache.sync()
        dest_rows = cache.destination_rows([e.slot for e in entries], before, counts)
        _tell_profiler(before, counts, phase)
        try:
            if phase == "decode" and self.use_graphs and picker is None:
                result = self._decode_with_graph(entries, before, borrow, dest_rows)
            else:
                result = self._run_packed(entries, before, counts, phase, dest_rows, picker, borrow)
        except Exception:
            self.poisoned = True
            raise
        cache.commit(growth)
        self.steps_run += 1
        return result

    def _run_packed(self, entries, before, counts, phase: str, dest_rows, picker, borrow: bool) -> torch.Tensor:
        rt = self.runtime
        pad_to = 0
        if phase == "prefill" and self.pads_prompts and sum(counts) <= self.PROMPT_PAD_LIMIT:
            pad_to = -(-sum(counts) // 64) * 64
        host, T, B, n_want, max_seq_len, max_kv_len = pack_host(entries, before, dest_rows, pad_to)
        if pad_to:  # the geometry of every step that fills the same rows
            max_seq_len = max_kv_len = -(-max_seq_len // 64) * 64
        kv_fill = 4
        if phase == "decode":  # the geometry a captured step would have
            max_kv_len = length_bucket(max_kv_len)
            kv_fill = fill_class([b + n for b, n in zip(before, counts)])
        choice, keys = None, None
        if picker is not None:
            choice = (picker.temperature, picker.seed)
            if picker.temperature is not None:
                if len(picker.keys) != n_want:
                    raise InvalidError("one sampling key per wanted place")
                keys = picker.keys
        key = (phase, T, B, n_want, max_seq_len, max_kv_len, choice, kv_fill)
        if pad_to and self.use_graphs and key in self._prompt_shapes_seen:
            graph = self._graph_of(key)  # a geometry that came before: captured once, replayed since
            graph.upload(host, keys)
            self._launch(graph)
            if picker is not None:
                return graph.ids
            return graph.logits if borrow else graph.logits.clone()
        if pad_to:
            self._prompt_shapes_seen.add(key)
        if rt.device.type == "cuda":
            dev = torch.from_numpy(host).pin_memory().to(rt.device, non_blocking=True)
        else:
            dev = torch.from_numpy(host).to(rt.device)
        ctx = context_over(dev, rt, phase, T, B, n_want, max_seq_len, max_kv_len, len(dest_rows), kv_fill)
        start = ops.launch_count()
        if picker is None:
            result = self.model.forward(ctx, self.cache)
        else:
            device_keys = None
            if keys is not None:
                device_keys = torch.tensor(keys, dtype=torch.int64).pin_memory().to(rt.device, non_blocking=True)
            result = self.model.forward_pick(ctx, self.cache, picker.temperature, picker.seed, device_keys)
        self.last_launches = ops.launch_count() - start
        return result

    def check_device_status(self) -> None:
        """Raise if a kernel recorded that it gave up on a bounded wait (reads 4 bytes back,
        so callers do it where they synchronize anyway)."""
        from ..kernels import gemm_dispatch
        try:
            gemm_dispatch.check_status()
        except Exception:
            self.poisoned = True
            raise

    # -- decode, host side in a few array operations -----------------------------------
    def _prepare_decode(self, slots: np.ndarray, tokens: np.ndarray):
        """Checks and bookkeeping of a decode step for `slots` (one token each): returns the
        packed host buffer and the lengths before the step, or None when the general path has
        to take over (a slot that is not open, a sequence at its first token, a window).
        Pages are taken here; the caller commits the lengths after launching."""
        cache, batch = self.cache, len(slots)
        if slots.min() < 0 or slots.max() >= cache.max_slots or not cache.open_mask[slots].all():
            return None  # the general path names the slot that is not open
        if len(np.unique(slots)) != batch:
            raise InvalidError("a slot appears twice in one step")
        if tokens.min() < 0 or tokens.max() >= self.model.plan.vocab_size:
            raise InvalidError("token outside vocabulary")
        if (cache.lengths[slots] == 0).any():
            return None  # a sequence at its first token: a prefill step, or a mixed one to refuse
        grown = cache.grow_by_one(slots)
        if grown is None:
            return None
        before, dest_rows = grown
        cache.sync()
        groups = len(dest_rows)
        host = np.empty((8 + groups) * batch + 1, dtype=np.int32)
        order = np.arange(batch + 1, dtype=np.int32)
        host[0:batch] = tokens
        host[batch:2 * batch] = before
        host[2 * batch:3 * batch] = order[:batch]
        host[3 * batch:4 * batch + 1] = order
        host[4 * batch + 1:5 * batch + 1] = slots
        host[5 * batch + 1:6 * batch + 1] = before + 1
        host[6 * batch + 1:7 * batch + 1] = np.argsort(-before, kind="stable")
        host[7 * batch + 1:8 * batch + 1] = order[:batch]
        for g, rows in enumerate(dest_rows):
            host[(8 + g) * batch + 1:(9 + g) * batch + 1] = rows
        return host, before

    def _decode_vectorized(self, entries: List[StepEntry], borrow: bool) -> Optional[torch.Tensor]:
        """The decode step for sequences that each bring one token, with the same checks and
        the same effects as the general path, but without a Python loop per sequence. Returns
        None when the general path has to take over."""
        batch = len(entries)
        slots = np.fromiter((e.slot for e in entries), dtype=np.int64, count=batch)
        tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=batch)
        wanted = []
        for b, e in enumerate(entries):
            for place in e.want:
                if int(place) != 0:
                    raise InvalidError(f"wanted place {place} is outside the 1 tokens of the entry")
                wanted.append(b)
        prepared = self._prepare_decode(slots, tokens)
        if prepared is None:
            return None
        host, before = prepared
        try:
            logits = self._replay(host, batch, int(before.max()) + 1, wanted, borrow, fill_class(before + 1))
        except Exception:
            self.poisoned = True
            raise
        self.cache.commit_lengths(slots, before + 1)
        self.steps_run += 1
        return logits

    # -- decode that does not wait for its own result -------------------------------------
    @property
    def can_decode_ahead(self) -> bool:
        """True when decode steps can take their tokens from the device (CUDA graphs on)."""
        return self.use_graphs

    @property
    def can_rewind(self) -> bool:
        """True when the last decode step of some sequences can be taken back: keys and values
        are simply written again, fixed-size state cannot be un-updated."""
        return not self.cache.state_groups

    def rewind(self, slots: Sequence[int], tokens: int = 1) -> None:
        """Forget the last `tokens` tokens of started sequences (their cache rows stay where
        they are and are overwritten when the positions are fed again)."""
        if not self.can_rewind:
            raise UnsupportedError("sequences with fixed-size state cannot be rewound")
        self.cache.shorten(slots, tokens)

    def decode_ahead(self, slots: Sequence[int], tokens: Optional[Sequence[int]], previous,
                     picker) -> "PendingPicks":
        """Enqueue one decode step for `slots` and the choice of their next tokens; do not wait.

        The step's input tokens are `tokens` (host ids), or, when `tokens` is None, the ids
        that `previous` (the PendingPicks of the step before, for the same slots in the same
        order) chose on the device: the host then need not have seen them yet. `picker` maps
        the step's logits to an int32 [B] device tensor of chosen ids. The returned object
        gives the ids on the host when asked (it waits for this step only).
        """
        if self.poisoned:
            raise PoisonedError("a device error poisoned this session; reset it")
        batch = len(slots)
        slot_array = np.asarray(slots, dtype=np.int64)
        token_array = np.zeros(batch, dtype=np.int64) if tokens is None else np.asarray(tokens, dtype=np.int64)
        prepared = self._prepare_decode(slot_array, token_array)
        if prepared is None:
            raise UnsupportedError("decode_ahead needs open, started sequences")
        host, before = prepared
        try:
            choice = (picker.temperature, picker.seed) if hasattr(picker, "temperature") else None
            graph = self._graph_for(batch, int(before.max()) + 1, choice, fill_class(before + 1))
            graph.upload(host, picker.keys if choice is not None and picker.temperature is not None else None)
            if tokens is None:
                graph.static[:batch].copy_(previous.device_ids)  # the ids chosen by the step before
            self._launch(graph)
            device_ids = graph.ids if choice is not None else picker(graph.logits)
            pending = self._pending_slot()
            pending.launch(device_ids, batch)
        except Exception:
            self.poisoned = True
            raise
        self.cache.commit_lengths(slot_array, before + 1)
        self.steps_run += 1
        return pending

    def _pending_slot(self) -> "PendingPicks":
        if not self._pending_ring:
            self._pending_ring = [PendingPicks(self.cache.max_slots) for _ in range(4)]
        slot = self._pending_ring[self._pending_turn % 4]
        self._pending_turn += 1
        return slot

    # -- decode through a captured graph ---------------------------------------------
    def _decode_with_graph(self, entries: List[StepEntry], before: List[int], borrow: bool,
                           dest_rows) -> torch.Tensor:
        batch = len(entries)
        all_rows = [StepEntry(e.slot, e.tokens, (0,)) for e in entries]
        host, _, _, _, _, max_kv_len = pack_host(all_rows, before, dest_rows)
        wanted = [b for b, e in enumerate(entries) for _ in e.want]
        return self._replay(host, batch, max_kv_len, wanted, borrow, fill_class([b + 1 for b in before]))

    def _replay(self, host: np.ndarray, batch: int, max_kv_len: int, wanted: List[int],
                borrow: bool, kv_fill: int = 4) -> torch.Tensor:
        graph = self._graph_for(batch, max_kv_len, None, kv_fill)
        graph.upload(host)
        self._launch(graph)
        logits = graph.logits
        if wanted != list(range(batch)):
            index = torch.tensor(wanted, dtype=torch.long, device=logits.device)
            return logits.index_select(0, index)
        return logits if borrow else logits.clone()

    def _graph_for(self, batch: int, max_kv_len: int, choice=None, kv_fill: int = 4) -> _StepGraph:
        bucket = length_bucket(max_kv_len)
        return self._graph_of(("decode", batch, batch, batch, 1, bucket, choice, kv_fill))

    def _graph_of(self, key: Tuple) -> _StepGraph:
        """The captured step of geometry `key` = (phase, tokens, sequences, wanted rows, longest
        portion, longest sequence, how tokens are chosen, how unequal the sequences are); made on
        first use."""
        graph = self._graphs.get(key)
        if graph is None:
            graph = self._graphs[key] = _StepGraph(self, *key)
            while len(self._graphs) > self.max_graphs:
                self._graphs.popitem(last=False)  # the least recently used one and its buffers
        else:
            self._graphs.move_to_end(key)
        return graph

    def _launch(self, graph: _StepGraph) -> None:
        from ..kernels import gemm_dispatch
        if graph.graph is None:
            self._capture(graph)
        graph.graph.replay()
        self.last_launches = graph.launches
        if graph.reports_status:
            # a replay launches kernels with bounded waits without passing through their Python
            # wrappers: say here that the status word has to be read at the next check
            gemm_dispatch.mark_status_dirty()

    def _capture(self, graph: _StepGraph) -> None:
        # One eager run first: it loads every kernel the step needs and writes
        # exactly what the replay will write again, so it changes no result.
        def run():
            if graph.choice is None:
                return self.model.forward(graph.ctx, self.cache)
            temperature, seed = graph.choice
            return self.model.forward_pick(graph.ctx, self.cache, temperature, seed,
                                           graph.keys if temperature is not None else None)
        run()
        torch.cuda.current_stream().synchronize()
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        from ..kernels import gemm_dispatch
        captured = torch.cuda.CUDAGraph()
        start = ops.launch_count()
        status_launches = gemm_dispatch.status_launch_count()
        with torch.cuda.graph(captured, pool=self._pool):
            if graph.choice is not None:
                graph.ids = run()
            else:
                graph.logits = run()
                # the greedy pick rides along (two small kernels): a sampler that wants it finds it
                # as `logits.greedy_ids` and needs no launch of its own
                graph.greedy = ops.argmax_rows(graph.logits)
                graph.logits.greedy_ids = graph.greedy
        graph.launches = ops.launch_count() - start  # the pick's two kernels included
        graph.reports_status = gemm_dispatch.status_launch_count() > status_launches
        graph.graph = captured
