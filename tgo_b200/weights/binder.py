"""From tensor names in a checkpoint to tensors on the device.

The parts of a model declare what they need as WeightSpec records; the checkpoint
must hold exactly those names in those shapes. Whatever is wrong is reported once,
in one error that lists missing tensors, unexpected tensors and wrong shapes
(model/weights.go:158-276). A tied head that the checkpoint ships anyway is
accepted only if its bytes equal the embedding's (model.go:403-439).

Storage rule: a tensor keeps the width it is stored in unless the engine's
compute dtype asks otherwise for its role. Matrices and tables take the compute
dtype (bfloat16 stays bfloat16 in a bfloat16 engine, everything is widened in a
float32 engine); gains are widened to float32, which loses nothing; integer
tables are held as int32; a float32 tensor in a bfloat16 engine stays float32
unless its role is "matrix" or "table", and then the narrowing is reported.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .safetensors import SafetensorsRepo

ROLES = ("matrix", "table", "gain", "other")


@dataclass(frozen=True)
class WeightSpec:
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"          # matrix | table | gain | other


class WeightError(ValueError):
    """The checkpoint does not hold what the model declares."""


def _listing(items: List[str], limit: int = 8) -> str:
    shown = ", ".join(items[:limit])
    return shown + (f", and {len(items) - limit} more" if len(items) > limit else "")


def check_weights(expected: Iterable[WeightSpec], have: Dict[str, Tuple[str, Tuple[int, ...]]],
                  optional_alias: Optional[Tuple[str, str]] = None) -> List[str]:
    """Compare declared tensors with a checkpoint's header.

    `have` maps name -> (dtype string, shape). `optional_alias` = (alias, target):
    a tensor named `alias` may be present although the model reads `target` in its
    place (a tied head that was shipped); the caller compares the bytes.
    Returns the names present under the alias rule. Raises WeightError otherwise.
    """
    expected = list(expected)
    names = [w.name for w in expected]
    dup = sorted({n for n in names if names.count(n) > 1})
    if dup:
        raise WeightError(f"weights: declared twice: {_listing(dup)}")
    want = {w.name: w for w in expected}
    missing = sorted(n for n in want if n not in have)
    extra = sorted(n for n in have if n not in want)
    aliased = []
    if optional_alias and optional_alias[0] in extra:
        extra.remove(optional_alias[0])
        aliased.append(optional_alias[0])
    wrong = []
    for n in sorted(want):
        if n in have:
            dt, shape = have[n]
            shape, declared = tuple(shape), tuple(want[n].shape)
            if any(int(s) == 0 for s in shape) and shape != declared:
                # weights/weights.go:605-610: a tensor without elements is a broken file
                wrong.append(f"{n} is empty (shape {list(shape)})")
            elif want[n].role != "other" and len(shape) not in (1, 2):
                # weights/weights.go:756-762: a weight is a matrix or a gain vector
                wrong.append(f"{n} has rank {len(shape)} (shape {list(shape)}); a weight is a "
                             "matrix or a gain vector")
            elif want[n].role == "table" and len(shape) == 2 and len(declared) == 2 and \
                    shape[1] == declared[1] and shape[0] != declared[0]:
                # model/weights.go:224-234: the field to change is in config.json, so name it
                wrong.append(f"config: vocab_size is {declared[0]} and {n} has {shape[0]} rows; "
                             "the config and the weights are from different models")
            elif shape != declared:
                wrong.append(f"{n} is {list(shape)}, declared {list(declared)}")
            elif dt not in ("BF16", "F16", "F32") and want[n].role != "other":
                wrong.append(f"{n} is stored as {dt}; BF16, F16 or F32 is needed")
    if missing or extra or wrong:
        parts = []
        if missing:
            parts.append(f"{len(missing)} missing: {_listing(missing)}")
        if extra:
            parts.append(f"{len(extra)} unexpected (the architecture name matched and the "
                         f"weights did not): {_listing(extra)}")
        if wrong:
            parts.append(f"{len(wrong)} of the wrong shape or type: {_listing(wrong)}")
        raise WeightError("weights: " + "; ".join(parts))
    return aliased


def _place(t: torch.Tensor, role: str, compute_dtype: torch.dtype, device, name: str,
           log, narrowed=None) -> torch.Tensor:
    if not t.dtype.is_floating_point:
        return t.to(device=device, dtype=torch.int32)
    if role == "gain":
        return t.to(device=device, dtype=torch.float32)
    if role in ("matrix", "table"):
        if t.dtype == torch.float32 and compute_dtype != torch.float32 and log:
            log(f"weights: {name} is stored in 32-bit and is narrowed to {compute_dtype}")
        out = t.to(device=device, dtype=compute_dtype)
        if t.dtype == torch.float16 and compute_dtype == torch.bfloat16:
            # float16 has three mantissa bits more than bfloat16: the values are rounded.
            # What must not happen silently is a value that does not survive at all
            # (weights/weights.go:450-458 refuses a checkpoint its 16-bit type cannot hold)
            if not torch.isfinite(out).all():
                raise WeightError(f"weights: {name} holds values that are not finite in "
                                  f"{compute_dtype}")
            if narrowed is not None:
                narrowed.append(name)
        return out
    if t.dtype == torch.float32:
        return t.to(device=device)
    return t.to(device=device, dtype=compute_dtype)


def load_weights(expected: Iterable[WeightSpec], repo: SafetensorsRepo,
                 compute_dtype: torch.dtype, device,
                 tied_alias: Optional[Tuple[str, str]] = None,
                 log=lambda m: print(m, file=sys.stderr)) -> Dict[str, torch.Tensor]:
    """Check, then move every declared tensor to the device, one at a time, so the
    host never holds more than one plane beyond the file map."""
    expected = list(expected)
    have = {n: (repo.entry(n).dtype, repo.entry(n).shape) for n in repo.names()}
    aliased = check_weights(expected, have, tied_alias)
    if aliased:
        alias, target = tied_alias
        a, b = repo.tensor(alias), repo.tensor(target)
        if a.shape != b.shape or a.dtype != b.dtype or not torch.equal(
                a.view(torch.uint8), b.view(torch.uint8)):
            raise WeightError(f"weights: the config ties the head to {target} and the checkpoint "
                              f"ships a different {alias}")
    out, narrowed = {}, []
    for w in expected:
        out[w.name] = _place(repo.tensor(w.name), w.role, compute_dtype, device, w.name, log,
                             narrowed)
    if narrowed and log:
        log(f"weights: {len(narrowed)} tensors are stored as float16 and were rounded to "
            f"bfloat16 (8 significant bits instead of 11): {_listing(narrowed, 3)}")
    return out
