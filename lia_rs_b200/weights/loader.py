"""Weights by tensor name, checked against what the model declares.

A model declares `TensorSpec`s (name, shape).  `load_weights` reads exactly those from the
folder and raises ONE `WeightError` that lists every missing tensor, every unexpected one
and every wrong shape (the reference reports "missing tensor {name}" and
"invalid BF16 tensor {name}" one at a time: src/safetensors/archive.rs:65,
src/inference/huggingface/weights.rs:63-66).

Storage rule: 16-bit floating tensors are kept in bfloat16, integer tables become int32, and
a tensor stored in 32-bit floating point stays 32-bit.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .safetensors_io import Archive


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in self.wrong_shape))
        for message in self.other:
            lines.append("  " + message)
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple
    kind: str = "matrix"        # "matrix" (normal init) | "norm" (ones) | "table" (integers)
    optional: bool = False


def storage_dtype(dtype: torch.dtype) -> torch.dtype:
    if dtype in (torch.bfloat16, torch.float16):
        return torch.bfloat16
    if dtype == torch.float32:
        return torch.float32
    return torch.int32


def _check_names_and_shapes(shapes: dict, specs) -> dict:
    """`shapes`: name -> shape of what is on offer.  Raises the one WeightError; returns name -> spec."""
    names = set(shapes)
    wanted = {s.name: s for s in specs}
    missing = [n for n, s in wanted.items() if n not in names and not s.optional]
    unexpected = sorted(names - set(wanted))
    wrong = [(name, spec.shape, tuple(shapes[name])) for name, spec in wanted.items()
             if name in names and tuple(shapes[name]) != tuple(spec.shape)]
    if missing or unexpected or wrong:
        raise WeightError(sorted(missing), unexpected, wrong)
    return wanted


def _store(read, wanted: dict, names) -> dict:
    out, bad = {}, []
    for name in wanted:
        if name not in names:
            continue
        t = read(name)
        t = t.to(storage_dtype(t.dtype))
        if t.is_floating_point() and not torch.isfinite(t.float()).all():
            bad.append(f"non-finite values in {name}")
        out[name] = t
    if bad:
        raise WeightError([], [], [], bad)
    return out


def load_weights(model_dir: str, specs) -> dict:
    archive = Archive(model_dir)
    names = set(archive.names())
    wanted = _check_names_and_shapes({n: archive.entry(n).shape for n in names}, specs)
    return _store(archive.read, wanted, names)


def adopt_tensors(tensors: dict, specs) -> dict:
    """The same checks and storage rule for tensors that are already in memory (the random-weights mode
    without a folder)."""
    wanted = _check_names_and_shapes({n: t.shape for n, t in tensors.items()}, specs)
    return _store(tensors.__getitem__, wanted, set(tensors))
