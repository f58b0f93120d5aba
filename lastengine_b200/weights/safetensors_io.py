"""Reading and writing safetensors files: 8 bytes of little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the raw little-endian data.

Tensors are found by name over a memory map, the way the reference finds GGUF tensors by
name over its map (src/dense.rs:66-67,84-93), and are only read when asked for.
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class WeightsError(RuntimeError):
    """A checkpoint that cannot be read, or that does not fit the model."""


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightsError(f"{path}: {e.strerror or e}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightsError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise WeightsError(f"{path}: truncated (header says {n} bytes, file has {size - 8} after the length)")
        try:
            header = json.loads(self._f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise WeightsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self.entries: dict[str, dict] = header
        self._data_start = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        for name, e in self.entries.items():
            if e.get("dtype") not in _DTYPES:
                raise WeightsError(f"{path}: tensor '{name}' has unsupported dtype {e.get('dtype')!r}")
            b, t = e["data_offsets"]
            numel = 1
            for s in e["shape"]:
                numel *= s
            if t - b != numel * torch.empty((), dtype=_DTYPES[e["dtype"]]).element_size():
                raise WeightsError(f"{path}: tensor '{name}': {t - b} bytes do not match shape {e['shape']}")
            if self._data_start + t > size:
                raise WeightsError(f"{path}: truncated (tensor '{name}' ends at byte {self._data_start + t}, "
                                   f"file has {size})")

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the map (read-only memory: copy or move before writing to it)."""
        e = self.entries[name]
        b, t = e["data_offsets"]
        dt = _DTYPES[e["dtype"]]
        if t == b:
            return torch.empty(e["shape"], dtype=dt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; the tensor is only read
            flat = torch.frombuffer(self._mm, dtype=dt, count=(t - b) // torch.empty((), dtype=dt).element_size(),
                                    offset=self._data_start + b)
        return flat.view(e["shape"])


def open_checkpoint(model_dir: str) -> dict[str, tuple[SafetensorsFile, str]]:
    """name -> (file, name) over model.safetensors, or over the shards an index file lists."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    out: dict[str, tuple[SafetensorsFile, str]] = {}
    if os.path.isfile(index):
        with open(index) as f:
            wm = json.load(f).get("weight_map", {})
        files: dict[str, SafetensorsFile] = {}
        for name, fn in wm.items():
            if fn not in files:
                files[fn] = SafetensorsFile(os.path.join(model_dir, fn))
            if name not in files[fn].entries:
                raise WeightsError(f"{index}: '{name}' is not in {fn}")
            out[name] = (files[fn], name)
        return out
    if not os.path.isfile(single):
        raise WeightsError(f"{model_dir}: no model.safetensors (and no model.safetensors.index.json)")
    sf = SafetensorsFile(single)
    return {n: (sf, n) for n in sf.names()}


def save_file(tensors: dict[str, torch.Tensor], path: str, metadata: dict[str, str] | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightsError(f"cannot store dtype {t.dtype} ('{name}')")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-(len(blob) + 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
