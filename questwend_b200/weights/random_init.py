"""Random weights from a configuration and a seed.

The reference has no such mode.  Matrices and the embedding are drawn from
N(0, 0.02) and every norm weight from 1 + U(-0.1, 0.1).  Each tensor has its
own generator, seeded by the seed and the tensor's place in the manifest, so
the values do not depend on the order of generation; drawn on the CPU they are
the same on every machine.
"""
from __future__ import annotations

import json
import os

import torch

from .manifest import MATRIX, NORM_WEIGHT, NORMAL, TABLE, TensorSpec
from .safetensors_io import write_safetensors

INIT_STD = 0.02
NORM_SPREAD = 0.1


def _draw(spec: TensorSpec, seed: int, index: int, device) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) * 1000003 + index * 7919 + 12345) % (2 ** 63 - 1))
    if spec.role == TABLE:
        raise ValueError(f"tensor '{spec.name}': integer tables have no random form")
    if spec.init == NORMAL:
        t = torch.empty(spec.shape, dtype=torch.float32, device=device)
        t.normal_(0.0, INIT_STD, generator=gen)
        return t
    if spec.init == NORM_WEIGHT:
        t = torch.empty(spec.shape, dtype=torch.float32, device=device)
        t.uniform_(-NORM_SPREAD, NORM_SPREAD, generator=gen)
        return t.add_(1.0)
    raise ValueError(f"tensor '{spec.name}': unknown init '{spec.init}'")


def random_tensors(manifest: list[TensorSpec], seed: int, dtype: torch.dtype,
                   device="cpu", vector_dtype: torch.dtype | None = None) -> dict[str, torch.Tensor]:
    """Draw every required tensor of the manifest.  Matrices get ``dtype``; vectors
    ``vector_dtype`` (default: ``dtype``)."""
    out = {}
    for i, spec in enumerate(manifest):
        if spec.optional or spec.ignored:
            continue
        t = _draw(spec, seed, i, device)
        out[spec.name] = t.to(dtype if spec.role == MATRIX else (vector_dtype or dtype))
    return out


def write_model_folder(out_dir: str, config, seed: int, dtype: str | torch.dtype = "bfloat16") -> str:
    """Write ``config.json`` and ``model.safetensors`` for a configuration and a seed."""
    from ..config.registry import get_architecture
    if isinstance(dtype, str):
        dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
                 "float32": torch.float32, "fp32": torch.float32}[dtype]
    arch = get_architecture(config.architecture)
    plan = arch.plan(config)
    os.makedirs(out_dir, exist_ok=True)
    tensors = random_tensors(plan.manifest(), seed, dtype, device="cpu")
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    cfg = config.to_dict()
    cfg["torch_dtype"] = "bfloat16" if dtype == torch.bfloat16 else "float32"
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return out_dir
