"""Reader for safetensors checkpoints: an 8-byte little-endian header length, that many bytes of JSON (tensor name -> dtype, shape,
data_offsets into the rest of the file), then the raw little-endian data.  The reference loads its unquantised models through the
safetensors crate (src/openai/models/mod.rs, `VarBuilder::from_mmaped_safetensors`); this is the same format read
with numpy's memory map, one tensor at a time, so a checkpoint larger than host memory can stream to the device."""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterator, Tuple

import numpy as np
import torch

from ._lib import BackendError

_NP = {"F32": (np.float32, torch.float32), "F16": (np.float16, torch.float16), "BF16": (np.uint16, torch.bfloat16), "I32": (np.int32, torch.int32),
       "I64": (np.int64, torch.int64), "U8": (np.uint8, torch.uint8), "F64": (np.float64, torch.float64)}


def read_header(path: str) -> Tuple[dict, int]:
    """-> (name -> {dtype, shape, data_offsets}, offset of the data section)"""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise BackendError(f"{path}: not a safetensors file")
        n = struct.unpack("<Q", head)[0]
        if n <= 0 or 8 + n > size:
            raise BackendError(f"{path}: header length {n} does not fit the file")
        meta = json.loads(f.read(n).decode("utf-8"))
    meta.pop("__metadata__", None)
    for name, d in meta.items():
        a, b = d["data_offsets"]
        if d["dtype"] not in _NP:
            raise BackendError(f"{path}: tensor {name} has unsupported dtype {d['dtype']}")
        want = int(np.prod(d["shape"], dtype=np.int64)) * np.dtype(_NP[d["dtype"]][0]).itemsize
        if b - a != want or a < 0 or 8 + n + b > size:
            raise BackendError(f"{path}: tensor {name} has inconsistent offsets")
    return meta, 8 + n


def iter_tensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields (name, host tensor) in file order; bf16 comes back as torch.bfloat16 (bit copy)."""
    meta, base = read_header(path)
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    for name, d in sorted(meta.items(), key=lambda kv: kv[1]["data_offsets"][0]):
        npdt, tdt = _NP[d["dtype"]]
        a, b = d["data_offsets"]
        arr = np.frombuffer(mm[base + a: base + b].tobytes(), dtype=npdt).reshape(d["shape"])
        t = torch.from_numpy(arr.copy())
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        yield name, t


def load_file(path: str) -> Dict[str, torch.Tensor]:
    return dict(iter_tensors(path))


def save_file(tensors: Dict[str, torch.Tensor], path: str) -> None:
    """Writer for the same format (tests and synthetic checkpoints)."""
    rev = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int32: "I32", torch.int64: "I64", torch.uint8: "U8"}
    meta, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        meta[name] = {"dtype": rev[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(meta, separators=(",", ":")).encode("utf-8")
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
