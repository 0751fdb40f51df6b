"""The library entry point: open a model folder, get sessions and schedulers from it.

    model = tgo_b200.open(model_dir, dtype="bfloat16")
    session = model.new_session(context=4096)
    for token in session.complete(prompt_ids, Policy(max_tokens=32)): ...
    sched = model.new_scheduler(slots=8, chunk=512, reserve=256)

The names follow the reference's Open / NewSession / NewScheduler (model.go:199,
session.go:124, scheduler.go:72). Text is outside this engine: prompts and results are
token ids.
"""
from __future__ import annotations

import builtins
import json
import os
import sys
from typing import Optional

import torch

from .engine.model import Model
from .registry import model_spec_from_config
from .weights.binder import load_weights
from .weights.random_init import random_weights
from .weights.safetensors import SafetensorsRepo

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name}; bfloat16 or float32")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r}; bfloat16 or float32") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"tgo_b200 runs on a CUDA device only, not on {device}")
    if not torch.cuda.is_available():
        raise RuntimeError("tgo_b200 needs a CUDA device and torch sees none; there is no "
                           "CPU path")
    return device


class LoadedModel:
    """A model with its weights on the device (the reference's `Model`, model.go:129-177)."""

    def __init__(self, model: Model, config: dict, source: str):
        self.model = model
        self.config = config
        self.source = source

    @property
    def spec(self):
        return self.model.spec

    @property
    def info(self) -> dict:
        s = self.model.spec
        return {"architecture": s.architecture, "layers": len(s.layers),
                "calls": len(s.run_order), "hidden_size": s.hidden_size,
                "vocab_size": s.vocab_size, "dtype": str(self.model.dtype).replace("torch.", ""),
                "weight_bytes": self.model.weight_bytes(),
                "cache_bytes_per_token": self.model.cache_bytes_per_token(),
                "source": self.source}

    def new_engine(self, page_size: int = 16, max_tokens: Optional[int] = None,
                   num_pages: Optional[int] = None, num_slots: int = 4):
        from .engine.step import Engine
        return Engine(self.model, page_size, max_tokens, num_pages, num_slots)

    def new_scheduler(self, slots: int, chunk: int = 0, reserve: int = 512, **kw):
        from .engine.scheduler import Scheduler
        return Scheduler(self, slots, chunk=chunk, reserve=reserve, **kw)

    def new_session(self, context: int = 4096, **kw):
        from .engine.session import Session
        return Session(self, context, **kw)


def open(model_dir: str, dtype="bfloat16", device="cuda:0", log=None) -> LoadedModel:  # noqa: A001
    """Read config.json, pick the architecture by its name, check the checkpoint against
    what the model declares, and load (model.go:199-327)."""
    device = require_cuda(device)
    dtype = parse_dtype(dtype)
    with builtins.open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    spec = model_spec_from_config(config)
    model = Model(spec, dtype, device)
    repo = SafetensorsRepo(model_dir)
    try:
        weights = load_weights(model.weight_specs(), repo, dtype, device, model.tied_alias(),
                               log or (lambda m: print(m, file=sys.stderr)))
    finally:
        repo.close()
    model.bind(weights)
    return LoadedModel(model, config, model_dir)


def open_random(config: dict, seed: int, dtype="bfloat16", device="cuda:0", sigma: float = 0.02,
                gain_sigma: float = 0.1) -> LoadedModel:
    """A model of `config` with seeded random weights made on the device, no folder."""
    device = require_cuda(device)
    dtype = parse_dtype(dtype)
    spec = model_spec_from_config(config)
    model = Model(spec, dtype, device)
    weights = {}
    for ws in model.weight_specs():
        store = torch.float32 if ws.role == "gain" else dtype
        weights.update(random_weights([ws], seed, sigma, gain_sigma, store, device))
    model.bind(weights)
    return LoadedModel(model, config, f"random(seed={seed})")
