"""Reading and writing .safetensors files, by tensor name.

The format: an 8-byte little-endian header length, a JSON header mapping each
name to {dtype, shape, data_offsets}, then the raw data (offsets count from the
end of the header). `__metadata__` is not a tensor. The reference carries its
own reader of the same format in pulsarlm/src/pulsarlm/safetensors_file.py:14-88.
"""

from __future__ import annotations

import json
import mmap
import os
import struct

import torch

_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped file; `tensor(name)` is a view into the map (copy it or
    move it to a device before the file object goes away)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors file")
        self._file = open(path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if 8 + header_len > size:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._map[8 : 8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{path}: header is not JSON ({error})") from error
        header.pop("__metadata__", None)
        self._data_start = 8 + header_len
        self.entries: dict[str, dict] = header
        for name, entry in header.items():
            if entry.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {entry.get('dtype')!r}")
            begin, end = entry["data_offsets"]
            count = 1
            for d in entry["shape"]:
                count *= d
            width = torch.empty((), dtype=_DTYPES[entry["dtype"]]).element_size()
            if end - begin != count * width or self._data_start + end > size:
                raise SafetensorsError(f"{path}: tensor {name!r} has inconsistent offsets")

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        entry = self.entries[name]
        begin, end = entry["data_offsets"]
        dtype = _DTYPES[entry["dtype"]]
        shape = tuple(entry["shape"])
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        flat = torch.frombuffer(self._map, dtype=dtype, count=(end - begin) // dtype.itemsize,
                                offset=self._data_start + begin)
        return flat.view(shape)

    def close(self) -> None:
        # Views made by tensor() keep the map alive through the buffer protocol;
        # closing fails while any exist, which is left to the garbage collector.
        try:
            self._map.close()
        except BufferError:
            pass
        self._file.close()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Writes `tensors` (CPU or device; made contiguous) under their names."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = list(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        size = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + size]}
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())


def model_files(model_dir: str) -> list[str]:
    """The weight files of a model folder: `model.safetensors`, or the shards named
    by `model.safetensors.index.json`, or every `*.safetensors` in the folder (or
    in its `weights/` subfolder, as the reference lays folders out in
    pulsarlm/src/pulsarlm/checkpoint.py:188-203), sorted."""
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(model_dir, s) for s in shards]
    for folder in (model_dir, os.path.join(model_dir, "weights")):
        if os.path.isdir(folder):
            found = sorted(n for n in os.listdir(folder) if n.endswith(".safetensors"))
            if found:
                return [os.path.join(folder, n) for n in found]
    raise SafetensorsError(f"{model_dir}: no .safetensors file")
