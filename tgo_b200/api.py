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
    def stop_ids(self):
        """Token ids that end a completion without being part of it, as the model folder
        states them: `eos_token_id` (a number or a list) of generation_config.json, else of
        config.json. The reference takes them from its tokenizer's end-of-turn and
        end-of-text markers (decode.go:151-155); this engine has no tokenizer."""
        raw = None
        path = os.path.join(self.source, "generation_config.json") if self.source else ""
        if path and os.path.isfile(path):
            with builtins.open(path) as f:
                raw = json.load(f).get("eos_token_id")
        if raw is None:
            raw = self.config.get("eos_token_id")
        if raw is None:
            return []
        ids = raw if isinstance(raw, list) else [raw]
        V = self.spec.vocab_size
        return [int(i) for i in ids if isinstance(i, int) and not isinstance(i, bool) and 0 <= i < V]

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
                   num_pages: Optional[int] = None, num_slots: int = 4, graphs: bool = True):
        from .engine.step import Engine
        return Engine(self.model, page_size, max_tokens, num_pages, num_slots, graphs)

    def new_scheduler(self, slots: int, chunk: int = 0, reserve: int = 512,
                      pool_tokens: Optional[int] = None, page_size: int = 16,
                      max_batched_tokens: Optional[int] = None):
        """A continuous-batching scheduler over a pool of `pool_tokens` cache positions
        (default: every slot can hold chunk + reserve... at least 4096 positions)."""
        from .engine.scheduler import DEFAULT_CHUNK, Scheduler
        from .engine.step import Engine
        if pool_tokens is None:
            pool_tokens = slots * max(4096, (chunk or DEFAULT_CHUNK) + reserve)
        engine = Engine(self.model, page_size=page_size, max_tokens=pool_tokens, num_slots=slots)
        return Scheduler(engine, slots, chunk=chunk, reserve=reserve,
                         max_batched_tokens=max_batched_tokens)

    def new_session(self, context: int = 4096, **kw):
        from .engine.session import Session
        return Session(self, context, **kw)

    def generate(self, prompts, policy=None, slots: Optional[int] = None, chunk: int = 0,
                 pool_tokens: Optional[int] = None, page_size: int = 16, stop_ids=(),
                 max_batched_tokens: Optional[int] = None, scheduler=None,
                 reserve: Optional[int] = None):
        """Run every prompt (lists of token ids) to completion with continuous batching;
        returns the generated ids per prompt, in order. `policy` is one Policy for all or
        one per prompt; its max_tokens must be positive. The requests stay in
        `last_requests`; a policy with logprobs finds a TokenProb per generated token in its
        request's `.logprobs`."""
        from .engine.scheduler import Request, Runner
        from .sampling.policy import Policy
        from .sampling.sampler import sample_rows
        prompts = [list(map(int, p)) for p in prompts]
        policies = policy if isinstance(policy, (list, tuple)) else [policy or Policy(
            max_tokens=16)] * len(prompts)
        V = self.spec.vocab_size
        for pol in policies:
            pol.check(V)
            if pol.max_tokens <= 0:
                raise ValueError("generate: give every policy a positive max_tokens")
        slots = slots or min(len(prompts), 64)
        if scheduler is None:
            need = max(len(p) + pol.max_tokens for p, pol in zip(prompts, policies))
            if pool_tokens is None:
                pool_tokens = slots * ((need + 63) // 64 * 64)
            scheduler = self.new_scheduler(slots, chunk=chunk, reserve=reserve or max(
                pol.max_tokens for pol in policies), pool_tokens=pool_tokens,
                page_size=page_size, max_batched_tokens=max_batched_tokens)
        runner = Runner(scheduler, sample_rows, stop_ids)
        requests = [Request(p, pol, request_id=i) for i, (p, pol) in
                    enumerate(zip(prompts, policies))]
        for r in requests:
            runner.submit(r)
        runner.run()
        self.last_runner = runner
        self.last_requests = requests        # each with .logprobs, for policies that ask
        return [r.output for r in requests]


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
