"""Random-weights mode: from a configuration and a seed to a model folder, or to tensors
on a device.

Matrices and tables are N(0, sigma); every norm gain is 1 + N(0, gain_sigma). Each tensor
has its own stream, seeded from (seed, tensor name), so a tensor's values depend on
neither the order nor the presence of the others, and the stream is made from integer
hashes and single float32 operations, so one seed gives the same model whether the values
are made on the CPU (a model folder) or on the GPU (`open_random`). Values are float32,
rounded once to the storage type. (The reference's tests build their checkpoints the same way,
from the model's own weight table: fixture_test.go:78-212.)
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from typing import Dict, Iterable

import torch

from .binder import WeightSpec
from .safetensors import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}\0{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


_QUANTILES = None
_CHUNK = 1 << 24


def _quantile_table() -> torch.Tensor:
    """The standard normal's quantile function at 65537 evenly spaced probabilities, float32,
    made once on the CPU in float64 (so it is the same table wherever the values are made)."""
    global _QUANTILES
    if _QUANTILES is None:
        p = (torch.arange(65537, dtype=torch.float64) + 0.5) / 65537.0
        _QUANTILES = (math.sqrt(2.0) * torch.erfinv(2.0 * p - 1.0)).to(torch.float32)
    return _QUANTILES


def seeded_normal(n: int, seed: int, device="cpu") -> torch.Tensor:
    """n float32 draws from (very nearly) N(0, 1) that are the same bits on every device.

    Element i takes 32 bits from a SplitMix64 hash of (seed, i), made with integer
    operations alone; 16 of them pick a cell of the quantile table and 16 a place inside
    it, where the quantile is interpolated with one float32 subtraction, one multiplication
    and one addition. Integer arithmetic and single IEEE operations give the same result
    on the CPU and on a GPU, which a library's normal generator does not promise. (The
    values lie within 4.3 standard deviations.)"""
    table = _quantile_table().to(device)
    out = torch.empty(n, dtype=torch.float32, device=device)
    mask = (1 << 64) - 1

    def wrap(v: int) -> int:            # a 64-bit constant as the int64 with the same bits
        v &= mask
        return v - (1 << 64) if v >= (1 << 63) else v
    start = wrap(seed * 0x9E3779B97F4A7C15)
    for at in range(0, n, _CHUNK):
        m = min(_CHUNK, n - at)
        z = torch.arange(at, at + m, dtype=torch.int64, device=device) * wrap(0x9E3779B97F4A7C15)
        z = z + start
        z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * wrap(0xBF58476D1CE4E5B9)
        z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * wrap(0x94D049BB133111EB)
        z = z ^ ((z >> 31) & ((1 << 33) - 1))
        cell = (z >> 48) & 0xFFFF
        frac = ((z >> 32) & 0xFFFF).to(torch.float32) / 65536.0
        lo, hi = table[cell], table[cell + 1]
        out[at:at + m] = lo + (hi - lo) * frac
    return out


def random_tensor(spec: WeightSpec, seed: int, sigma: float, gain_sigma: float,
                  dtype: torch.dtype, device="cpu") -> torch.Tensor:
    n = 1
    for s in spec.shape:
        n *= int(s)
    t = seeded_normal(n, _tensor_seed(seed, spec.name), device).view(spec.shape)
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
