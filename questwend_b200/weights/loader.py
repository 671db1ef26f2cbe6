"""Loading a model's tensors by name, with one error that says everything wrong.

The reference looks tensors up by name and throws ``missing tensor: <name>`` at
the first one it cannot find (core/runtime.cpp:268-279); it never checks shapes.
Here the whole manifest is checked against the files first, and a single
``WeightsError`` lists every missing tensor, every unexpected tensor and every
wrong shape, so that a bad export is fixed in one go.
"""
from __future__ import annotations

import torch

from .manifest import MATRIX, TABLE, TensorSpec
from .safetensors_io import SafetensorsFolder


class WeightsError(ValueError):
    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"{where}: the weights do not fit the configuration"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {got}" for n, got in self.wrong_dtype))
        super().__init__("\n".join(lines))


def held_dtype(spec: TensorSpec, stored: torch.dtype, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor is held in on the device.

    Matrices take the engine's dtype.  Integer tables become int32.  Small
    vectors keep 32-bit storage when the file has it (and every vector is 32-bit
    in the 32-bit engine); a 16-bit vector stays bfloat16 in the bfloat16 engine.
    """
    if spec.role == TABLE:
        return torch.int32
    if spec.role == MATRIX:
        return compute_dtype
    if compute_dtype == torch.float32 or stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_manifest(manifest: list[TensorSpec], names_to_info: dict, where: str) -> None:
    """Raise one WeightsError for everything that does not fit."""
    by_name = {s.name: s for s in manifest}
    missing = [s.name for s in manifest if not s.optional and not s.ignored and s.name not in names_to_info]
    unexpected = [n for n in names_to_info if n not in by_name]
    wrong_shape, wrong_dtype = [], []
    for n, (dt, shape) in names_to_info.items():
        s = by_name.get(n)
        if s is None or s.ignored:
            continue
        if tuple(shape) != tuple(s.shape):
            wrong_shape.append((n, tuple(shape), tuple(s.shape)))
        floating = dt in (torch.float64, torch.float32, torch.float16, torch.bfloat16)
        if (s.role == TABLE) == floating:
            wrong_dtype.append((n, str(dt).replace("torch.", "")))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsError(where, sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)


def load_tensors(model_dir: str, manifest: list[TensorSpec], compute_dtype: torch.dtype,
                 device: torch.device | str) -> dict[str, torch.Tensor]:
    """Read every tensor of the manifest from the folder onto the device."""
    folder = SafetensorsFolder(model_dir)
    try:
        infos = {n: folder.info(n) for n in folder.names()}
        check_manifest(manifest, infos, model_dir)
        out = {}
        for spec in manifest:
            if spec.name not in infos or spec.ignored:
                continue
            t = folder.tensor(spec.name)
            held = t.to(device=device, dtype=held_dtype(spec, t.dtype, compute_dtype)).contiguous()
            if held.data_ptr() == t.data_ptr():
                held = held.clone()              # never hand out the file's own (read-only) bytes
            out[spec.name] = held
        return out
    finally:
        folder.close()
