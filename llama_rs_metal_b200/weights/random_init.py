"""Random-weights mode: write a model folder from a configuration and a seed.

The reference has random weights only in test fixtures
(crates/llama-rs/tests/common/mod.rs:86-100); here it is a first-class mode
because benchmarks and tests run without checkpoints. Every tensor has its own
generator keyed by (seed, tensor name), so a tensor's values do not depend on
which other tensors exist or in which order they are made.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Callable, Dict, Mapping

import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return torch.Generator(device=device).manual_seed(int.from_bytes(digest[:8], "little") >> 1)


def random_tensors(wanted: Mapping[str, TensorSpec], seed: int, std: float = 0.02,
                   vector_mean: float = 1.0, vector_std: float = 0.0,
                   dtype: torch.dtype = torch.bfloat16,
                   is_vector: Callable[[str, TensorSpec], bool] = None, device="cpu") -> Dict[str, torch.Tensor]:
    """N(0, std) for matrices; N(vector_mean, vector_std) for 1-D scale vectors (norm weights).

    With a CUDA `device` the numbers are drawn there (large models in seconds, no folder in
    between); the device's generator draws other numbers than the CPU's for the same seed, so a
    folder written on the CPU and a model drawn on the device are different random models."""
    out = {}
    for name, spec in wanted.items():
        gen = _generator(seed, name, device)
        vector = is_vector(name, spec) if is_vector else len(spec.shape) == 1
        if spec.kind == "integer":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif vector:
            t = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * vector_std + vector_mean
            out[name] = t.to(dtype)
        else:
            t = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
            out[name] = t.mul_(std).to(dtype)
            del t
    return out


def write_model_folder(model_dir: str, config_dict: dict, tensors: Mapping[str, torch.Tensor],
                       seed: int = None) -> str:
    """config.json + model.safetensors in `model_dir` (created if needed)."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config_dict, handle, indent=1)
    meta = {"format": "pt"}
    if seed is not None:
        meta["seed"] = str(seed)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), dict(tensors), meta)
    return model_dir
