"""Reader of ``.safetensors`` checkpoints (no third-party dependency).

File layout: an 8-byte little-endian header length, that many bytes of JSON mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the header), then the raw
little-endian tensor data.  Tensors are returned as CPU torch tensors that view one read of the file.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
    "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "I16": (torch.int16, 2), "I32": (torch.int32, 4), "I64": (torch.int64, 8),
    "BOOL": (torch.bool, 1),
}


def read_header(path: str | Path) -> tuple[dict, int]:
    """``(name -> entry, offset of the data section)``; the ``__metadata__`` entry is dropped."""
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: not a safetensors file (too short)")
        (n,) = struct.unpack("<Q", raw)
        if n <= 0 or n > (1 << 31):
            raise ValueError(f"{path}: implausible header length {n}")
        header = json.loads(f.read(n).decode("utf-8"))
    header.pop("__metadata__", None)
    return header, 8 + n


def load_safetensors(path: str | Path) -> dict[str, torch.Tensor]:
    header, base = read_header(path)
    data = torch.from_numpy(np.fromfile(path, dtype=np.uint8, offset=base))
    out: dict[str, torch.Tensor] = {}
    for name, ent in header.items():
        if ent["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {ent['dtype']}")
        dtype, size = _DTYPES[ent["dtype"]]
        begin, end = ent["data_offsets"]
        shape = tuple(int(s) for s in ent["shape"])
        count = int(np.prod(shape)) if shape else 1
        if end - begin != count * size or end > data.numel():
            raise ValueError(f"{path}: tensor {name!r} has inconsistent offsets")
        raw = data[begin:end]
        if begin % size:                                        # a view needs the element's alignment
            raw = raw.clone()
        out[name] = raw.view(dtype).reshape(shape)
    return out


def save_safetensors(path: str | Path, tensors: dict[str, torch.Tensor]) -> None:
    """Writer of the same format (used to export synthetic models)."""
    names = {v: k for k, v in ((k, v[0]) for k, v in _DTYPES.items())}
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
