"""Random-weights mode: from a configuration and a seed to a model folder, or to tensors
on a device.

Matrices and tables are N(0, sigma); every norm gain is 1 + N(0, gain_sigma). Each tensor
has its own generator, seeded from (seed, tensor name), so a tensor's values depend on
neither the order nor the presence of the others. Values are drawn in float32 and rounded
once to the storage type. (The reference's tests build their checkpoints the same way,
from the model's own weight table: fixture_test.go:78-212.)
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterable

import torch

from .binder import WeightSpec
from .safetensors import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}\0{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(spec: WeightSpec, seed: int, sigma: float, gain_sigma: float,
                  dtype: torch.dtype, device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, spec.name))
    t = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
    if spec.role == "gain":
        t = 1.0 + gain_sigma * t
    else:
        t = sigma * t
    return t.to(dtype)


def random_weights(specs: Iterable[WeightSpec], seed: int, sigma: float = 0.02,
                   gain_sigma: float = 0.1, dtype: torch.dtype = torch.bfloat16,
                   device="cpu") -> Dict[str, torch.Tensor]:
    return {s.name: random_tensor(s, seed, sigma, gain_sigma, dtype, device) for s in specs}


def write_random_model(model_dir: str, config: dict, seed: int, sigma: float = 0.02,
                       gain_sigma: float = 0.1, dtype: torch.dtype = torch.bfloat16) -> None:
    """Write config.json and model.safetensors for `config` (a config.json as a dict)."""
    from ..engine.model import Model
    from ..registry import model_spec_from_config
    spec = model_spec_from_config(config)
    model = Model(spec, torch.float32, "cpu")
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    tensors = random_weights(model.weight_specs(), seed, sigma, gain_sigma, dtype)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors)
