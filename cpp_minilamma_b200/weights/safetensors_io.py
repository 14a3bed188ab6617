"""Reader and writer of the safetensors container, by tensor name.

Layout: 8-byte little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`,
then the raw little-endian tensor bytes.  A folder holds either `model.safetensors` or
shards listed in `model.safetensors.index.json` (`weight_map`: name -> file).

The reference reads a JSON manifest plus one raw float32 file and checks dtype, byte
size, overlap and trailing bytes (src/load.cc:185-314, 407-459, 545-566); the same
checks are made here on the safetensors header.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch


class WeightFileError(ValueError):
    """The container itself is damaged (truncated, overlapping, bad header)."""


_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    file: Path
    begin: int  # absolute byte offsets in the file
    end: int


class SafetensorsFile:
    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        with open(self.path, "rb") as fh:
            head = fh.read(8)
            if len(head) != 8:
                raise WeightFileError(f"{self.path}: shorter than the 8-byte header length")
            (header_len,) = struct.unpack("<Q", head)
            if header_len > size - 8:
                raise WeightFileError(f"{self.path}: header length {header_len} exceeds the file size {size}")
            try:
                header = json.loads(fh.read(header_len).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as exc:
                raise WeightFileError(f"{self.path}: header is not valid JSON ({exc})") from None
        if not isinstance(header, dict):
            raise WeightFileError(f"{self.path}: header must be a JSON object")
        base = 8 + header_len
        self.entries: Dict[str, TensorEntry] = {}
        spans: List[Tuple[int, int, str]] = []
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype_name, shape, (begin, end) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise WeightFileError(f"{self.path}: entry {name!r} lacks dtype/shape/data_offsets") from None
            if dtype_name not in _DTYPES:
                raise WeightFileError(f"{self.path}: tensor {name!r} has unsupported dtype {dtype_name!r}")
            dtype, width = _DTYPES[dtype_name]
            count = 1
            for dim in shape:
                if not isinstance(dim, int) or dim < 0:
                    raise WeightFileError(f"{self.path}: tensor {name!r} has a bad shape {shape}")
                count *= dim
            if end - begin != count * width:
                raise WeightFileError(
                    f"{self.path}: tensor {name!r} spans {end - begin} bytes, shape {shape} of {dtype_name} "
                    f"needs {count * width}")
            if begin < 0 or base + end > size:
                raise WeightFileError(f"{self.path}: tensor {name!r} lies beyond the end of the file")
            spans.append((begin, end, name))
            self.entries[name] = TensorEntry(name, dtype, shape, self.path, base + begin, base + end)
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise WeightFileError(f"{self.path}: tensors {n0!r} and {n1!r} overlap")
        if spans and base + spans[-1][1] != size:
            raise WeightFileError(f"{self.path}: {size - base - spans[-1][1]} trailing bytes after the last tensor")
        self._map = None

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a CPU torch tensor that owns its memory."""
        entry = self.entries[name]
        if self._map is None:
            with open(self.path, "rb") as fh:
                self._map = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=entry.end - entry.begin, offset=entry.begin)
        flat = torch.from_numpy(raw.copy())
        return flat.view(entry.dtype).reshape(entry.shape)

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None


class ModelFiles:
    """All tensors of a model folder, whichever shard they are in."""

    def __init__(self, folder):
        folder = Path(folder)
        index = folder / "model.safetensors.index.json"
        single = folder / "model.safetensors"
        self.files: List[SafetensorsFile] = []
        self.entries: Dict[str, TensorEntry] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        if index.is_file():
            try:
                weight_map = json.loads(index.read_text())["weight_map"]
            except (json.JSONDecodeError, KeyError) as exc:
                raise WeightFileError(f"{index}: not a shard index ({exc})") from None
            for shard in sorted(set(weight_map.values())):
                self._add(SafetensorsFile(folder / shard))
        elif single.is_file():
            self._add(SafetensorsFile(single))
        else:
            raise WeightFileError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")

    def _add(self, file: SafetensorsFile) -> None:
        self.files.append(file)
        for name, entry in file.entries.items():
            if name in self.entries:
                raise WeightFileError(f"tensor {name!r} appears in {self.entries[name].file} and {file.path}")
            self.entries[name] = entry
            self._owner[name] = file

    def read(self, name: str) -> torch.Tensor:
        return self._owner[name].read(name)

    def close(self):
        for f in self.files:
            f.close()


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write CPU tensors under their names, in the given order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    blobs = []
    for name, tensor in tensors.items():
        t = tensor.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightFileError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * ((8 - len(encoded) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(encoded)))
        fh.write(encoded)
        for raw in blobs:
            fh.write(raw)
