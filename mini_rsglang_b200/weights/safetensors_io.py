"""Reader and writer for the safetensors container: 8 bytes of little-endian header length,
a JSON header {name: {dtype, shape, data_offsets}}, then the raw little-endian data.  The
reference reads the same files through the `safetensors` crate
(crates/models/src/weights.rs:40-44); its range checks are restated here
(crates/models/src/checkpoint.rs:73-126)."""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch

from ..errors import InvalidRequest

# safetensors dtype name -> (numpy dtype that carries the bits, torch dtype it is viewed as)
_DTYPES = {
    "F64": (np.float64, torch.float64),
    "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16),
    "BF16": (np.uint16, torch.bfloat16),
    "I64": (np.int64, torch.int64),
    "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16),
    "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8),
    "BOOL": (np.bool_, torch.bool),
}
_NAMES = {torch_dtype: name for name, (_, torch_dtype) in _DTYPES.items()}


@dataclass
class StoredTensor:
    """One entry of a file's header; `read()` copies the bytes out of the mapping."""

    name: str
    dtype: str
    shape: tuple[int, ...]
    file: "SafetensorsFile"
    begin: int
    end: int

    def read(self) -> torch.Tensor:
        if self.dtype not in _DTYPES:
            raise InvalidRequest(f"{self.name}: unsupported weight dtype {self.dtype}")
        np_dtype, torch_dtype = _DTYPES[self.dtype]
        count = int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1
        array = np.frombuffer(self.file.data, dtype=np_dtype, count=count, offset=self.begin)
        tensor = torch.from_numpy(array.copy())
        if torch_dtype is torch.bfloat16:
            tensor = tensor.view(torch.bfloat16)
        return tensor.reshape(self.shape)


class SafetensorsFile:
    """A mapped file and its parsed, checked header."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise InvalidRequest(f"{path}: too short for a safetensors header")
        self._handle = open(path, "rb")
        mapped = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", mapped[:8])
        if header_len > size - 8:
            raise InvalidRequest(f"{path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(bytes(mapped[8:8 + header_len]).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise InvalidRequest(f"{path}: header is not JSON: {e}") from None
        if not isinstance(header, dict):
            raise InvalidRequest(f"{path}: header is not a JSON object")
        self.data = memoryview(mapped)[8 + header_len:]
        self.metadata = header.pop("__metadata__", None)
        self.tensors: dict[str, StoredTensor] = {}
        for name, entry in header.items():
            try:
                dtype, shape = entry["dtype"], tuple(int(s) for s in entry["shape"])
                begin, end = (int(v) for v in entry["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise InvalidRequest(f"{path}: malformed header entry for {name}") from None
            if begin > end or end > len(self.data):
                raise InvalidRequest(f"{path}: {name}: byte range {begin}..{end} outside the data "
                                     f"section of {len(self.data)} bytes")
            if dtype in _DTYPES:
                width = np.dtype(_DTYPES[dtype][0]).itemsize
                count = int(np.prod(shape, dtype=np.int64)) if shape else 1
                if count * width != end - begin:
                    raise InvalidRequest(f"{path}: {name}: shape {list(shape)} of {dtype} needs "
                                         f"{count * width} bytes, the file gives {end - begin}")
            self.tensors[name] = StoredTensor(name, dtype, shape, self, begin, end)


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write tensors (on the host, any of the dtypes above) as one safetensors file."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    chunks = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise InvalidRequest(f"{name}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint16).numpy().tobytes() if t.dtype is torch.bfloat16 else t.numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        chunks.append(raw)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for raw in chunks:
            f.write(raw)
