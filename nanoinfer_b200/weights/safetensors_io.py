"""Reading and writing the safetensors container, by tensor name.

File layout: 8 bytes little-endian header length N, N bytes of JSON mapping each
tensor name to {"dtype", "shape", "data_offsets": [begin, end)} (offsets relative to
the first byte after the header), then the raw little-endian tensor bytes.

The reference reads no such file: it memory-maps one positional binary
(src/model/model.cpp:54-125) whose order is fixed by its exporter.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# safetensors dtype tag -> (numpy dtype used to map the bytes, torch dtype of the view)
_DTYPES = {
    "F32": (np.dtype("<f4"), torch.float32),
    "BF16": (np.dtype("<u2"), torch.bfloat16),
    "F16": (np.dtype("<f2"), torch.float16),
    "I32": (np.dtype("<i4"), torch.int32),
    "I64": (np.dtype("<i8"), torch.int64),
}
_TAG_OF = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
           torch.int32: "I32", torch.int64: "I64"}


class TensorEntry:
    __slots__ = ("name", "dtype_tag", "shape", "begin", "end", "path", "data_start")

    def __init__(self, name, dtype_tag, shape, begin, end, path, data_start):
        self.name, self.dtype_tag, self.shape = name, dtype_tag, tuple(shape)
        self.begin, self.end, self.path, self.data_start = begin, end, path, data_start


def read_header(path: str) -> Dict[str, TensorEntry]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte header length")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            meta = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
    data_start = 8 + n
    entries: Dict[str, TensorEntry] = {}
    for name, info in meta.items():
        if name == "__metadata__":
            continue
        try:
            tag, shape, (b, e) = info["dtype"], info["shape"], info["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: malformed entry for tensor '{name}'") from None
        if tag not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {tag}")
        numel = 1
        for s in shape:
            numel *= int(s)
        if e - b != numel * _DTYPES[tag][0].itemsize:
            raise SafetensorsError(f"{path}: tensor '{name}' of shape {shape} and dtype {tag} "
                                   f"does not match its {e - b} bytes")
        if b < 0 or data_start + e > size:
            raise SafetensorsError(f"{path}: tensor '{name}' reaches beyond the end of the file "
                                   f"(truncated?)")
        entries[name] = TensorEntry(name, tag, shape, b, e, path, data_start)
    return entries


def read_tensor(entry: TensorEntry) -> torch.Tensor:
    """Read one tensor into host memory with the dtype it is stored in."""
    np_dtype, torch_dtype = _DTYPES[entry.dtype_tag]
    count = (entry.end - entry.begin) // np_dtype.itemsize
    arr = np.fromfile(entry.path, dtype=np_dtype, count=count,
                      offset=entry.data_start + entry.begin)
    if arr.size != count:
        raise SafetensorsError(f"{entry.path}: short read of tensor '{entry.name}'")
    t = torch.from_numpy(arr)
    if torch_dtype == torch.bfloat16:
        t = t.view(torch.bfloat16)
    return t.reshape(entry.shape)


def list_files(model_dir: str) -> List[str]:
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    return [os.path.join(model_dir, f) for f in files]


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write (name, tensor) pairs; each tensor is stored in its own dtype."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    meta = {}
    offset = 0
    for name, t in items:
        if t.dtype not in _TAG_OF:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        meta[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape),
                      "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    header = json.dumps(meta, separators=(",", ":")).encode("utf-8")
    header += b" " * ((8 - len(header) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        for _, t in items:
            if t.dtype == torch.bfloat16:
                f.write(t.view(torch.int16).numpy().tobytes())
            else:
                f.write(t.numpy().tobytes())
