"""A decoder put together from a plan: embedding, scheduled blocks, final norm, head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..errors import InvalidError
from ..kernels import ops
from ..parts.base import Block, ModelPlan, PartSpec
from ..parts.linear import LinearWeight
from ..registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, build_part

FAMILIES = {"mixer": (MIXERS, "mixer"), "feed_forward": (FEED_FORWARDS, "feed-forward"), "norm": (NORMS, "norm")}
from ..runtime import Runtime
from ..weights.loader import TensorSpec


def _full_names(spec: PartSpec, part) -> Dict[str, str]:
    """own tensor name -> checkpoint name, for one part."""
    return {own: spec.names.get(own, spec.prefix + own) for own in part.tensors()}


class DecoderModel:
    """Owns the parts of one model and runs them over a step's packed tokens.

    It knows nothing of Llama: which parts there are, their sizes, their tensor
    names and the order of layers all come from the plan.
    """

    def __init__(self, plan: ModelPlan, runtime: Runtime):
        self.plan, self.runtime = plan, runtime
        self.blocks: List[Block] = []
        self._names: List[Dict[str, Dict[str, str]]] = []
        for layer in plan.layers:
            if layer.block not in BLOCKS:
                raise InvalidError(f"block kind {layer.block!r} is not registered")
            block_class = BLOCKS[layer.block]
            # the block says which roles a layer of its kind has, and of which family each is
            parts = {}
            for role, family in block_class.roles.items():
                if role not in layer.parts:
                    raise InvalidError(f"a {layer.block!r} layer needs a part for the role {role!r}")
                if family not in FAMILIES:
                    raise InvalidError(f"block {layer.block!r}: role {role!r} has unknown family {family!r}")
                table, label = FAMILIES[family]
                parts[role] = build_part(table, layer.parts[role], label)
            unknown = sorted(set(layer.parts) - set(parts))
            if unknown:
                raise InvalidError(f"a {layer.block!r} layer has no role {', '.join(unknown)}")
            self.blocks.append(block_class(**parts))
            self._names.append({role: _full_names(layer.parts[role], part) for role, part in parts.items()})
        self.final_norm = build_part(NORMS, plan.final_norm, "norm")
        self._final_names = _full_names(plan.final_norm, self.final_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[LinearWeight] = None
        self.unexpected_tensors: tuple = ()  # stored names the loader skipped (set by the loader's caller)
        self._check_schedule()

    # -- schedule and cache --------------------------------------------------------
    def _check_schedule(self) -> None:
        writers = {}
        for position, entry in enumerate(self.plan.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise InvalidError(f"schedule names layer {entry.layer}, the model has {len(self.blocks)}")
            if entry.writes_cache:
                if entry.cache in writers:
                    raise InvalidError(f"cache entry {entry.cache} is written by two schedule entries")
                writers[entry.cache] = position
            elif entry.cache not in writers:
                raise InvalidError(f"schedule entry {position} reads cache entry {entry.cache} before it is written")
        if sorted(writers) != list(range(len(writers))):
            raise InvalidError("cache entries must be numbered 0..n-1")

    def cache_requests(self) -> list:
        """What each cache entry's writing layer asks of the cache (index = cache entry)."""
        out = {}
        for entry in self.plan.schedule:
            if entry.writes_cache:
                out[entry.cache] = self.blocks[entry.layer].cache_request()
        return [out[i] for i in range(len(out))]

    @property
    def graph_safe(self) -> bool:
        """True when every part only enqueues device work, so a decode step can be a CUDA graph."""
        parts = [self.final_norm]
        for block in self.blocks:
            parts += [block, *block.parts.values()]
        return all(p.graph_safe for p in parts)

    # -- weights ---------------------------------------------------------------------
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        plan = self.plan
        specs = {plan.embedding_name: TensorSpec((plan.vocab_size, plan.hidden_size))}
        if plan.head_name is not None:
            specs[plan.head_name] = TensorSpec((plan.vocab_size, plan.hidden_size))
        for block, names in zip(self.blocks, self._names):
            for role, mapping in names.items():
                part_specs = getattr(block, role).tensors()
                for own, full in mapping.items():
                    specs[full] = part_specs[own]
        for own, full in self._final_names.items():
            specs[full] = self.final_norm.tensors()[own]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand every part its tensors (already on the device, in their kept precision)."""
        rt = self.runtime
        self.embedding = tensors[self.plan.embedding_name].contiguous()
        head = self.embedding if self.plan.head_name is None else tensors[self.plan.head_name]
        self.head = LinearWeight(head)
        for block, names in zip(self.blocks, self._names):
            for role, mapping in names.items():
                getattr(block, role).bind({own: tensors[full] for own, full in mapping.items()}, rt)
        self.final_norm.bind({own: tensors[full] for own, full in self._final_names.items()}, rt)

    # -- forward ---------------------------------------------------------------------
    def forward(self, ctx, cache) -> torch.Tensor:
        """float32 logits [len(ctx.wanted_rows), vocab] for one step."""
        x = self._hidden_of_wanted_rows(ctx, cache)
        if x is None:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=self.runtime.device)
        logits = self.head(x, out_dtype=torch.float32)
        if self.plan.logit_scale is not None:
            ops.scale_(logits, self.plan.logit_scale)
        return logits

    def forward_pick(self, ctx, cache, temperature=None, seed: int = 0, keys=None) -> torch.Tensor:
        """int32 [len(ctx.wanted_rows)]: the token chosen at each wanted place, for a caller that
        wants no logits (generation): greedy when `temperature` is None, else a draw from
        softmax(logits / temperature) keyed per row by `keys` (int64). The head product chooses in
        its epilogue where a kernel can (crates/model-runtime/src/execute.rs:238-247 pairs the head
        with the GPU argmax the same way). -1 marks a row with a non-finite logit."""
        x = self._hidden_of_wanted_rows(ctx, cache)
        if x is None:
            return torch.empty((0,), dtype=torch.int32, device=self.runtime.device)
        scale = self.plan.logit_scale
        if scale is not None and scale <= 0:
            logits = ops.scale_(self.head(x, out_dtype=torch.float32), scale)
            return ops.argmax_rows(logits) if temperature is None else \
                ops.sample_gumbel_rows(logits, temperature, seed, keys)
        if temperature is not None and scale is not None:
            temperature = temperature / scale  # (s z) / T = z / (T / s)
        return self.head.pick(x, temperature, seed, keys)

    def _hidden_of_wanted_rows(self, ctx, cache) -> Optional[torch.Tensor]:
        """Embedding, the scheduled blocks and the final norm on the wanted rows; None when no
        row is wanted (the cache is filled all the same)."""
        plan = self.plan
        # what dispatchers kept belongs to one run of the step: a context that runs again (a
        # captured step, once before and once under capture) must compute it again from its arrays
        ctx.scratch.clear()
        ctx.fresh_kv.clear()
        hidden = ops.embed_rows(self.embedding, ctx.token_ids, plan.embedding_scale)
        wanted = ctx.wanted_rows.numel() > 0
        schedule = plan.schedule
        for i, entry in enumerate(schedule):
            ctx.entry = entry
            view = cache.view(entry.cache) if cache is not None else None
            # may this block's last product leave its K slices for the next reader of the stream?
            if i + 1 < len(schedule):
                ctx.next_folds_pending = self.blocks[schedule[i + 1].layer].folds_pending_on_entry
            else:
                ctx.next_folds_pending = wanted and self.final_norm.folds_pending
            hidden = self.blocks[entry.layer].forward(hidden, ctx, view)
            if ctx.pending is not None and not ctx.next_folds_pending:
                ctx.settle(hidden)  # a block left sums its successor cannot add itself
        ctx.entry = None
        ctx.next_folds_pending = False
        if not wanted:
            ctx.take_pending()
            return None
        # the head runs only on the rows whose logits are wanted
        # (crates/model-runtime/src/execute.rs:238-247 does it for the last row)
        return self.final_norm.forward(hidden, ctx, rows=ctx.wanted_rows)
