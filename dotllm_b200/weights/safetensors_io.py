"""Reader and writer for the safetensors container: 8-byte little-endian header
length, a JSON header ``{name: {dtype, shape, data_offsets}}``, then raw bytes.

The reference reads GGUF only (src/DotLLM.Models/ModelLoader.cs:21-28) and has
no safetensors path; this file plays the role of its ``GgufFile`` reader
(src/DotLLM.Models/Gguf/): memory-map, index tensors by name, hand out views.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

from ..errors import WeightsError

# safetensors dtype tag -> (torch dtype used to view the bytes, bytes per element)
_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_TAGS = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One memory-mapped .safetensors file; tensors are views into the mapping."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise WeightsError(f"no such file: {self.path}")
        self._fh = open(self.path, "rb")
        size = self.path.stat().st_size
        if size < 8:
            raise WeightsError(f"{self.path}: too short to be a safetensors file")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)   # private, never written
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len <= 0 or 8 + header_len > size:
            raise WeightsError(f"{self.path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise WeightsError(f"{self.path}: header is not valid JSON ({exc})") from exc
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + header_len
        self.entries = {}
        for name, meta in header.items():
            tag = meta.get("dtype")
            if tag not in _DTYPES:
                raise WeightsError(f"{self.path}: tensor {name!r} has unsupported dtype {tag!r}")
            shape = tuple(int(s) for s in meta["shape"])
            lo, hi = (int(v) for v in meta["data_offsets"])
            count = 1
            for s in shape:
                count *= s
            if lo < 0 or hi < lo or self._base + hi > size or hi - lo != count * _DTYPES[tag][1]:
                raise WeightsError(f"{self.path}: tensor {name!r} has offsets [{lo}, {hi}) that do not "
                                   f"fit shape {shape} of {tag} in a file of {size} bytes")
            self.entries[name] = (tag, shape, lo, hi)

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return self.entries[name][1]

    def dtype_tag(self, name):
        return self.entries[name][0]

    def tensor(self, name):
        """A CPU tensor that views the mapped bytes: move or clone it before the file is closed."""
        tag, shape, lo, hi = self.entries[name]
        dtype, _ = _DTYPES[tag]
        if hi == lo:
            return torch.empty(shape, dtype=dtype)
        flat = torch.frombuffer(self._map, dtype=dtype, count=(hi - lo) // _DTYPES[tag][1],
                                offset=self._base + lo)
        return flat.view(shape)

    def close(self):
        try:
            self._map.close()
        except BufferError:
            pass          # views still alive; the mapping is released with them
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def save_safetensors(path, tensors, metadata=None):
    """Write ``{name: tensor}`` to one safetensors file, names sorted, data 8-byte aligned."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    chunks = []
    for name in sorted(tensors):
        t = tensors[name].detach().to("cpu").contiguous()
        if t.dtype not in _TAGS:
            raise WeightsError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _TAGS[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        chunks.append(raw)
        offset += len(raw)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((-len(blob)) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for raw in chunks:
            fh.write(raw)


def open_model_files(folder):
    """The safetensors files of a model folder: ``model.safetensors``, or the shards
    that ``model.safetensors.index.json`` names."""
    folder = Path(folder)
    single = folder / "model.safetensors"
    index = folder / "model.safetensors.index.json"
    if single.is_file():
        return [SafetensorsFile(single)]
    if index.is_file():
        try:
            weight_map = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError) as exc:
            raise WeightsError(f"{index}: not a safetensors index ({exc})") from exc
        return [SafetensorsFile(folder / shard) for shard in sorted(set(weight_map.values()))]
    raise WeightsError(f"no model.safetensors (or model.safetensors.index.json) in {folder}")
