"""Reading and writing safetensors files, by tensor name.

The format: eight bytes of little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}``, then the tensors'
raw bytes.  The reader maps the file and hands out tensors without copying the
file first; a folder with ``model.safetensors.index.json`` is read shard by
shard.  The reference reads GGUF the same way: a name -> (file, offset) map
built once, bytes fetched per tensor (core/model.cpp:444-502, 306-323), with
shards found by name (core/model.cpp:400-423).
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped .safetensors file: ``names()``, ``info(name)``, ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: truncated file ({size} bytes, no header length)")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if 8 + n > size:
            raise SafetensorsError(f"{path}: truncated file (header of {n} bytes does not fit in {size})")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + n
        self._entries = {}
        for name, info in header.items():
            dt = info.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt!r}")
            shape = tuple(int(x) for x in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=_DTYPES[dt]).element_size()
            if e - b != want:
                raise SafetensorsError(f"{path}: tensor '{name}' of shape {list(shape)} and dtype {dt} "
                                       f"needs {want} bytes, the header gives {e - b}")
            if self._base + e > size:
                raise SafetensorsError(f"{path}: truncated file (tensor '{name}' ends at byte "
                                       f"{self._base + e}, the file has {size})")
            self._entries[name] = (_DTYPES[dt], shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> list[str]:
        return list(self._entries)

    def info(self, name: str):
        dt, shape, _, _ = self._entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapped bytes (read-only memory: clone or copy before writing)."""
        dt, shape, b, e = self._entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # the buffer is not writable; we never write to it
            flat = torch.frombuffer(self._mm, dtype=torch.uint8, count=e - b, offset=self._base + b)
        return flat.view(dt).reshape(shape)

    def close(self):
        # Tensors handed out keep the map alive; it is unmapped when the last of them goes.
        self._mm = None
        self._f.close()


class SafetensorsFolder:
    """All tensors of a model folder: one ``model.safetensors`` or an index with shards."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._files: dict[str, SafetensorsFile] = {}
        self._where: dict[str, str] = {}
        if os.path.exists(index):
            with open(index) as f:
                weight_map = json.load(f)["weight_map"]
            for name, fname in weight_map.items():
                if fname not in self._files:
                    self._files[fname] = SafetensorsFile(os.path.join(model_dir, fname))
                if name not in self._files[fname]._entries:
                    raise SafetensorsError(f"{index}: tensor '{name}' is not in shard {fname}")
                self._where[name] = fname
        elif os.path.exists(single):
            self._files["model.safetensors"] = SafetensorsFile(single)
            for name in self._files["model.safetensors"].names():
                self._where[name] = "model.safetensors"
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor "
                                   f"model.safetensors.index.json is there")

    def names(self) -> list[str]:
        return list(self._where)

    def info(self, name: str):
        return self._files[self._where[name]].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)

    def close(self):
        for f in self._files.values():
            f.close()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write CPU tensors to one file; names are stored in the given order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(t)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((-len(raw)) % 8)             # keep the data 8-byte aligned
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in blobs:
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
