"""Weights by tensor name, with one error that lists everything wrong.

A model says which tensors it wants (name -> TensorSpec) and which stored names
it ignores on purpose (a saved `lm_head.weight` beside tied embeddings,
crates/model-format/src/mlx/mod.rs:44-48). The loader checks names and shapes
for all of them before it copies anything
(crates/model-runtime/src/loader.rs:2-13 has the two messages). A missing or
wrongly shaped tensor is an error, and the error also lists the stored names
nobody asked for (a misnamed tensor shows up as one missing and one unexpected).
Stored names nobody asked for are by themselves no error: they are skipped, as
the reference skips names it does not know (mlx/mod.rs:41-43, e.g. the vision
tower of a multimodal export), and reported in `LoadedTensors.unexpected`;
`strict=True` makes them an error too.

Storage precision is kept: bfloat16 stays bfloat16, a tensor stored in 32-bit
stays 32-bit, integer tables become int32. float16 has no kernels of its own
and is rounded to bfloat16. With `float32=True` every floating tensor is
widened to float32 (the reference's --float-weights-f32,
crates/model-format/src/checkpoint.rs:252-265).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Tuple

import torch

from ..errors import UnsupportedError, WeightError
from .safetensors_io import TensorEntry, open_checkpoint

PREFIXES = ("model.language_model.", "language_model.")  # mlx/names.rs:3-8


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects of one tensor."""

    shape: Tuple[int, ...]
    kind: str = "float"  # "float" | "integer"


def canonical_name(name: str) -> str:
    """Strip the wrappers some exporters put around the language model's names."""
    if name.startswith("model.language_model."):
        return "model." + name[len("model.language_model."):]
    if name.startswith("language_model."):
        return name[len("language_model."):]
    return name


class LoadedTensors(dict):
    """name -> tensor, plus the stored names that were skipped because nobody asked for them."""

    unexpected: Tuple[str, ...] = ()


def check_names_and_shapes(found: Mapping[str, Tuple[int, ...]], wanted: Mapping[str, TensorSpec],
                           ignored: Iterable[str] = (), strict: bool = False) -> Tuple[str, ...]:
    """Raise one WeightError naming missing, unexpected and wrongly shaped tensors when a tensor
    is missing or has the wrong shape (or, with `strict`, when one is unexpected). Returns the
    unexpected names otherwise."""
    ignored = set(ignored)
    missing = [n for n in wanted if n not in found]
    unexpected = [n for n in found if n not in wanted and n not in ignored]
    wrong = [(n, wanted[n].shape, found[n]) for n in wanted
             if n in found and tuple(found[n]) != tuple(wanted[n].shape)]
    if missing or wrong or (strict and unexpected):
        raise WeightError(missing=missing, unexpected=unexpected, wrong_shape=wrong)
    return tuple(sorted(unexpected))


def stored_dtype_policy(dtype: torch.dtype, kind: str, float32: bool) -> torch.dtype:
    if kind == "integer" or not dtype.is_floating_point:
        if dtype.is_floating_point:
            raise UnsupportedError("integer table stored as a floating tensor")
        return torch.int32
    if float32:
        return torch.float32
    if dtype in (torch.float32, torch.float64):
        return torch.float32
    if dtype in (torch.bfloat16, torch.float16):
        return torch.bfloat16
    raise UnsupportedError(f"unsupported weight dtype {dtype}")


def load_tensors(model_dir: str, wanted: Mapping[str, TensorSpec], ignored: Iterable[str] = (),
                 float32: bool = False, device: str = "cpu", strict: bool = False) -> LoadedTensors:
    """Load exactly the wanted tensors onto `device` under the storage-precision policy."""
    entries: Dict[str, TensorEntry] = {}
    for name, entry in open_checkpoint(model_dir).items():
        canon = canonical_name(name)
        if canon in entries:
            raise WeightError(other=[f"duplicate tensor {canon}"])
        entries[canon] = entry
    for name, entry in entries.items():
        if name in wanted and wanted[name].kind == "float" and not entry.dtype.is_floating_point:
            raise WeightError(other=[f"{name}: stored as {entry.dtype}, a floating tensor is expected"])
    unexpected = check_names_and_shapes({n: e.shape for n, e in entries.items()}, wanted, ignored, strict)
    out = LoadedTensors()
    out.unexpected = unexpected
    for name, spec in wanted.items():
        entry = entries[name]
        target = stored_dtype_policy(entry.dtype, spec.kind, float32)
        out[name] = entry.load().to(device=device, dtype=target, copy=True)
    return out
