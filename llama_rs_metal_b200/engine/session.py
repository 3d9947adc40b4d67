"""Engine -> Model -> Session: the public entry point, after the reference's facade.

    engine = Engine()                                  # crates/llama-rs/src/engine.rs:27
    model = engine.load(folder, dtype="bfloat16")      # engine.rs:58 (float_weights_f32 ~ dtype="float32")
    session = model.session(context=4096, max_batch=8) # crates/llama-rs/src/model.rs:18
    results = session.generate(prompts, GenerationOptions(max_tokens=32, sampling=Sampling(temperature=0)))

Where the reference's Session is one sequence, this one holds a cache for
`max_batch` sequences; prefill/decode/reset/tokens/logits keep their meaning
for the session's own single sequence, and `generate` takes many prompts.
Text, tokenizers and chat templates are outside the library: prompts and
results are token ids.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional, Sequence

import torch

from ..cache import PAGE_SIZE, Cache
from ..config.base import read_config_json, read_generation_eos
from ..errors import (CancelledError, ContextError, InvalidError, KernelUnavailableError, CacheMemoryError,
                      OptionsError)
from ..registry import find_architecture
from ..runtime import Runtime, parse_dtype
from ..sampling.device import BatchSampler
from ..sampling.options import GenerationOptions
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors, write_model_folder
from .batch import StepEntry
from .generate import GenerationResult, generate
from .model import DecoderModel
from .step import StepRunner


@dataclass
class MemoryEstimate:
    """Bytes a model and a session need (crates/model-runtime/src/memory.rs:3-49)."""

    weights: int
    cache: int

    @property
    def session(self) -> int:
        return self.cache


class Engine:
    """One GPU. There is no CPU device: constructing an Engine without CUDA raises."""

    def __init__(self, device: int = 0, memory_limit: Optional[int] = None):
        if not torch.cuda.is_available():
            raise KernelUnavailableError("no CUDA device: this library has no CPU path")
        self.device = torch.device("cuda", device)
        self.memory_limit = memory_limit
        from ..kernels import library
        library.load()  # fail now, loudly, if the kernels cannot be built or loaded

    def device_name(self) -> str:
        return torch.cuda.get_device_name(self.device)

    def load(self, model_dir: str, dtype="bfloat16") -> "Model":
        return Model(self, model_dir, parse_dtype(dtype))

    def random(self, config: dict, seed: int = 0, std: float = 0.02, norm_mean: float = 1.0,
               norm_std: float = 0.0, dtype="bfloat16") -> "Model":
        """A model of the architecture `config` (a config.json dict) names with random weights drawn
        on the device: no folder, no file, seconds even for billions of weights. For measurements
        at sizes whose folder would take minutes to write; write_random_model() is the mode that
        leaves a loadable folder."""
        return Model(self, None, parse_dtype(dtype), random=dict(config=config, seed=seed, std=std,
                                                                norm_mean=norm_mean, norm_std=norm_std))


def build_model(model_dir: str, runtime: Runtime):
    """(config, plan, model with weights bound, bytes of weights) for a model folder. Stored
    tensors the model has no use for are skipped; their names are in `model.unexpected_tensors`."""
    root = read_config_json(model_dir)
    arch = find_architecture(root)
    config = arch.config_class.from_dict(root)
    plan = arch.plan(config)
    model = DecoderModel(plan, runtime)
    tensors = load_tensors(model_dir, model.tensor_specs(), ignored=plan.ignored_names,
                           float32=runtime.float32, device=runtime.device)
    model.bind(tensors)
    model.unexpected_tensors = tuple(tensors.unexpected)
    weight_bytes = sum(t.numel() * t.element_size() for t in tensors.values())
    return config, plan, model, weight_bytes


def build_random_model(spec: dict, runtime: Runtime):
    """build_model() for weights drawn on the device instead of read from a folder."""
    arch = find_architecture(spec["config"])
    config = arch.config_class.from_dict(spec["config"])
    plan = arch.plan(config)
    model = DecoderModel(plan, runtime)
    tensors = random_tensors(model.tensor_specs(), spec["seed"], std=spec["std"], vector_mean=spec["norm_mean"],
                             vector_std=spec["norm_std"],
                             dtype=torch.float32 if runtime.float32 else torch.bfloat16, device=runtime.device)
    model.bind(tensors)
    return config, plan, model, sum(t.numel() * t.element_size() for t in tensors.values())


class Model:
    def __init__(self, engine: Engine, model_dir: Optional[str], dtype: torch.dtype, random: Optional[dict] = None):
        self.engine = engine
        self.model_dir = model_dir
        self.runtime = Runtime(engine.device, dtype)
        if random is not None:
            self.config, self.plan, self.decoder, self.weight_bytes = build_random_model(random, self.runtime)
        else:
            self.config, self.plan, self.decoder, self.weight_bytes = build_model(model_dir, self.runtime)
        # stored tensors no part asked for: skipped, as the reference skips unknown names
        # (crates/model-format/src/mlx/mod.rs:41-43)
        self.unexpected_tensors = self.decoder.unexpected_tensors
        stops = set(self.plan.stop_token_ids) | set(read_generation_eos(model_dir) if model_dir else ())
        self.stop_token_ids = tuple(sorted(stops))

    def memory(self, context: int, max_batch: int = 1) -> MemoryEstimate:
        if context <= 0 or context > self.plan.max_positions:
            raise ContextError(self.plan.max_positions, context)
        elem = 4 if self.runtime.float32 else 2
        pages = max_batch * -(-context // PAGE_SIZE)
        cache = 0
        for request in self.decoder.cache_requests():
            if hasattr(request, "kv_heads"):
                cache += 2 * pages * PAGE_SIZE * request.kv_heads * request.head_dim * elem
            elif request is not None:
                n = 1
                for s in request.shape:
                    n *= s
                cache += max_batch * n * torch.empty((), dtype=request.dtype).element_size()
        return MemoryEstimate(self.weight_bytes, cache)

    def session(self, context: int = 0, max_batch: int = 1, max_tokens: Optional[int] = None) -> "Session":
        """`context` 0 selects min(8192, the model's limit) (crates/llama-rs/src/model.rs:19-23)."""
        if context == 0:
            context = min(8192, self.plan.max_positions)
        estimate = self.memory(context, max_batch)
        limit = self.engine.memory_limit
        if limit is not None and estimate.weights + estimate.cache > limit:
            raise CacheMemoryError(f"model and session need {estimate.weights + estimate.cache} bytes, "
                                   f"the engine's limit is {limit}")
        return Session(self, context, max_batch, max_tokens)


class Session:
    def __init__(self, model: Model, context: int, max_batch: int, max_tokens: Optional[int] = None):
        self.model, self.context, self.max_batch = model, context, max_batch
        pages_per_seq = -(-context // PAGE_SIZE)
        self.token_budget = max_tokens if max_tokens is not None else max_batch * pages_per_seq * PAGE_SIZE
        self.cache = Cache(model.decoder.cache_requests(), model.runtime.dtype, model.runtime.device,
                           max_tokens=self.token_budget, max_slots=max_batch, max_sequence=context)
        self.runner = StepRunner(model.decoder, self.cache, model.runtime)
        self._cancel = False
        self._own_slot: Optional[int] = None
        self._own_tokens: List[int] = []
        self._last_logits: Optional[torch.Tensor] = None

    # -- the stepper interface the generation loop drives ------------------------------
    def open_slot(self) -> int:
        return self.cache.open_slot()

    def close_slot(self, slot: int) -> None:
        self.cache.close_slot(slot)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """For the generation loop: the logits are sampled from at once, so they may live in a
        buffer that the next step overwrites."""
        return self.runner.step(entries, borrow=True)

    def step_pick(self, entries: Sequence[StepEntry], picker):
        """For the generation loop when only tokens are wanted: chosen on the device, no logits."""
        return self.runner.step_pick(entries, picker)

    def check_device_status(self) -> None:
        self.runner.check_device_status()

    @property
    def can_decode_ahead(self) -> bool:
        return self.runner.can_decode_ahead

    def decode_ahead(self, slots, tokens, previous, picker):
        return self.runner.decode_ahead(slots, tokens, previous, picker)

    @property
    def can_rewind(self) -> bool:
        return self.runner.can_rewind

    def rewind(self, slots, tokens: int = 1) -> None:
        self.runner.rewind(slots, tokens)

    # -- many sequences -------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], options: Optional[GenerationOptions] = None,
                 stop_token_ids: Optional[Iterable[int]] = None,
                 on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
        """Token ids in, token ids out, one result per prompt (crates/llama-rs/src/session.rs:78-109)."""
        options = options or GenerationOptions()
        options.validate()
        if self._own_slot is not None:
            raise InvalidError("generate() needs the whole cache: reset() the session's own sequence first")
        stops = self.model.stop_token_ids if stop_token_ids is None else tuple(stop_token_ids)
        sampler = BatchSampler(options.sampling)
        self._cancel = False
        return generate(self, sampler, prompts, options, stops, max_batch=self.max_batch,
                        context=self.context, token_budget=self.token_budget, page_size=PAGE_SIZE,
                        cancelled=lambda: self._cancel, on_token=on_token)

    def cancel(self) -> None:
        """Checked between steps (the reference's cancellation handle, session.rs:3-6)."""
        self._cancel = True

    # -- the session's own single sequence (the reference's Session surface) ----------
    def tokens(self) -> List[int]:
        return list(self._own_tokens)

    def logits(self) -> Optional[torch.Tensor]:
        """float32 [vocab] logits after the last prefill/decode, on the device."""
        return self._last_logits

    def prefill(self, tokens: Sequence[int]) -> torch.Tensor:
        """Feed tokens to the session's own sequence; logits of the last one.

        The tokens run as one step whatever the sequence already holds: on an empty
        sequence as a prompt, on a started one as a portion that attends to the cache
        (crates/model-runtime/src/session.rs:105-164 appends to a session's history the
        same way, in chunks of 32). A kernel that gave up on a bounded wait poisons the
        session here, before any logits are handed out.
        """
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise OptionsError("prompt must contain at least one token")
        if len(self._own_tokens) + len(tokens) > self.context:
            raise ContextError(self.context, len(self._own_tokens) + len(tokens))
        if self._cancel:
            raise CancelledError("cancelled")
        if self._own_slot is None:
            self._own_slot = self.cache.open_slot()
        out = self.runner.step([StepEntry(self._own_slot, tokens, [len(tokens) - 1])])
        self._own_tokens.extend(tokens)
        self.runner.check_device_status()  # reads 4 bytes back when a kernel with bounded waits ran
        self._last_logits = out[0]
        return self._last_logits

    def synchronize_prompt(self, tokens: Sequence[int]) -> torch.Tensor:
        """Make the session's own sequence equal `tokens` with as little work as possible: if
        they go on from what the sequence holds only the new tokens are fed, otherwise the
        sequence starts over (crates/llama-rs/src/session.rs:47-77). Logits of the last token."""
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise OptionsError("prompt must contain at least one token")
        if len(tokens) > self.context:
            raise ContextError(self.context, len(tokens))
        if any(not 0 <= t < self.model.plan.vocab_size for t in tokens):
            raise OptionsError("token outside vocabulary")
        held = self._own_tokens
        if tokens[:len(held)] != held:
            self.reset()
            held = self._own_tokens
        suffix = tokens[len(held):]
        if suffix:
            return self.prefill(suffix)
        if self._last_logits is None:
            raise OptionsError("prompt must contain at least one token")
        return self._last_logits

    def decode(self, token: int) -> torch.Tensor:
        """decode(token) = prefill([token]) (crates/model-runtime/src/session.rs:165-167)."""
        return self.prefill([token])

    def reset(self) -> None:
        if self._own_slot is not None:
            self.cache.close_slot(self._own_slot)
        self._own_slot, self._own_tokens, self._last_logits = None, [], None
        self._cancel = False
        self.runner.poisoned = False
        from ..kernels import ops
        ops.reset_pick_scratch()  # a step that failed half-way may have left its running bests behind

    def snapshot(self, entry: int):
        if self._own_slot is None:
            raise InvalidError("the session's own sequence is empty")
        return self.cache.snapshot(self._own_slot, entry)


def write_random_model(model_dir: str, config_dict: dict, seed: int, std: float = 0.02,
                       norm_mean: float = 1.0, norm_std: float = 0.0,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Random-weights mode: a loadable model folder from a config.json dict and a seed.

    The tensor list comes from the architecture's own plan, so it is right for
    any registered architecture. Needs no GPU.
    """
    arch = find_architecture(config_dict)
    config = arch.config_class.from_dict(config_dict)
    plan = arch.plan(config)
    model = DecoderModel(plan, Runtime(torch.device("cpu"), torch.float32))
    tensors = random_tensors(model.tensor_specs(), seed, std=std, vector_mean=norm_mean,
                             vector_std=norm_std, dtype=dtype)
    out = config.to_dict() if hasattr(config, "to_dict") else dict(config_dict)
    return write_model_folder(model_dir, out, tensors, seed)
