"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.  Matrices are N(0, initializer_range) rounded once to bfloat16,
norm weights are 1; the folder then loads like any checkpoint."""
from __future__ import annotations

import json
import os

import torch

from .safetensors_io import write_safetensors


def random_tensors(specs, seed: int, std: float) -> dict:
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    out = {}
    for spec in specs:
        if spec.optional:
            continue
        if spec.kind == "norm":
            out[spec.name] = torch.ones(spec.shape, dtype=torch.bfloat16)
        elif spec.kind == "table":
            out[spec.name] = torch.zeros(spec.shape, dtype=torch.int32)
        else:
            # generate in pieces so that a 70k x 4k matrix needs no large fp32 temporary
            t = torch.empty(spec.shape, dtype=torch.bfloat16)
            flat = t.view(-1)
            step = 1 << 24
            for begin in range(0, flat.numel(), step):
                n = min(step, flat.numel() - begin)
                flat[begin:begin + n] = (torch.randn(n, generator=generator) * std).to(torch.bfloat16)
            out[spec.name] = t
    return out


def random_weights(config, seed: int = 0) -> dict:
    """The tensors of the model that `config` (a typed configuration of a registered architecture) describes,
    by checkpoint name: the one source of random weights, whether they are written to a folder or not."""
    from ..config import resolve_architecture

    model_spec = resolve_architecture(config.to_dict()).build(config)
    return random_tensors(model_spec.tensor_specs(), seed, float(getattr(config, "initializer_range", 0.02)))


def write_random_model(config, model_dir: str, seed: int = 0) -> str:
    """`config` is a typed configuration (any class registered with the architecture
    registry).  Returns the folder."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), random_weights(config, seed))
    return model_dir
