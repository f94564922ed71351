"""Reading and writing of safetensors files, by tensor name.

The format: 8 bytes little-endian header length ``n``, ``n`` bytes of JSON mapping
each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header; the key ``__metadata__`` is free-form), then the
raw little-endian bytes.  The reference reads a positional float32 dump instead
(src/io/checkpoint.cpp:106-317); lookup by name has no counterpart there.

A folder may hold ``model.safetensors`` or, for models cut into several files,
``model.safetensors.index.json`` whose ``weight_map`` names the file of each tensor.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Tuple

import torch

from ..errors import ErrorCode, PhotonError

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape, self.begin, self.end, self.file = name, dtype, shape, begin, end, file


class SafetensorsFile:
    """One file, memory-mapped; tensors are materialised one at a time."""

    def __init__(self, path: str):
        self.path = path
        if not os.path.isfile(path):
            raise PhotonError(ErrorCode.FILE_NOT_FOUND, f"no weights file at {path}")
        size = os.path.getsize(path)
        if size < 8:
            raise PhotonError(ErrorCode.INVALID_FILE, f"{path}: too short for a safetensors header")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise PhotonError(ErrorCode.INVALID_FILE, f"{path}: header length {n} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise PhotonError(ErrorCode.INVALID_FILE, f"{path}: header is not valid JSON: {e}") from None
        self.data_start = 8 + n
        self.entries: Dict[str, TensorEntry] = {}
        data_len = size - self.data_start
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(x) for x in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise PhotonError(ErrorCode.INVALID_FILE, f"{path}: malformed entry for tensor {name!r}") from None
            if dt not in _DTYPES:
                raise PhotonError(ErrorCode.INVALID_FILE, f"{path}: tensor {name!r} has unsupported dtype {dt}")
            count = 1
            for s in shape:
                count *= s
            nbytes = count * torch.empty((), dtype=_DTYPES[dt]).element_size()
            if not (0 <= b <= e <= data_len) or e - b != nbytes:
                raise PhotonError(ErrorCode.INVALID_FILE,
                                  f"{path}: tensor {name!r} has offsets [{b}, {e}) that do not fit its shape "
                                  f"{shape} ({nbytes} bytes) or the file ({data_len} data bytes)")
            self.entries[name] = TensorEntry(name, _DTYPES[dt], shape, b, e, self)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def read(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        buf = memoryview(self._mm)[self.data_start + e.begin: self.data_start + e.end]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        # a private copy of the bytes: the tensor outlives the map and may be written to
        return torch.frombuffer(bytearray(buf), dtype=e.dtype).reshape(e.shape)

    def close(self) -> None:
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass
        self._f.close()


def open_model_files(folder: str) -> Tuple[Dict[str, TensorEntry], List[SafetensorsFile]]:
    """All tensors of a model folder by name."""
    index = os.path.join(folder, "model.safetensors.index.json")
    single = os.path.join(folder, "model.safetensors")
    files: List[SafetensorsFile] = []
    entries: Dict[str, TensorEntry] = {}
    if os.path.isfile(single):
        names = ["model.safetensors"]
    elif os.path.isfile(index):
        with open(index) as f:
            try:
                wm = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError):
                raise PhotonError(ErrorCode.INVALID_FILE, f"{index}: no weight_map") from None
        names = sorted(set(wm.values()))
    else:
        raise PhotonError(ErrorCode.FILE_NOT_FOUND, f"{folder}: neither model.safetensors nor model.safetensors.index.json")
    for n in names:
        sf = SafetensorsFile(os.path.join(folder, n))
        files.append(sf)
        for name, e in sf.entries.items():
            if name in entries:
                raise PhotonError(ErrorCode.INVALID_FILE, f"tensor {name!r} appears in more than one file of {folder}")
            entries[name] = e
    return entries, files


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"cannot store dtype {t.dtype}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
