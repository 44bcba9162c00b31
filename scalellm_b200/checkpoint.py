"""Reading a model folder: config.json and model.safetensors.

A safetensors file is an 8-byte little-endian header length, that many bytes of JSON
(name -> dtype, shape, data_offsets) and the tensors' bytes.  The file is memory-mapped and each
tensor is copied to the device once; nothing else of the file is kept.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Tuple

import numpy as np
import torch

_DTYPES = {"BF16": (np.int16, torch.bfloat16), "F16": (np.float16, None), "F32": (np.float32, None),
           "F64": (np.float64, None), "I32": (np.int32, None), "I64": (np.int64, None),
           "I16": (np.int16, None), "I8": (np.int8, None), "U8": (np.uint8, None), "BOOL": (np.bool_, None)}


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def safetensors_header(path: str) -> Tuple[dict, int]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
    header.pop("__metadata__", None)
    return header, 8 + n


def read_safetensors(path: str, device="cpu") -> Dict[str, torch.Tensor]:
    """All tensors of the file, in their stored dtypes, on `device`."""
    header, base = safetensors_header(path)
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            for name, meta in header.items():
                np_dt, view = _DTYPES[meta["dtype"]]
                lo, hi = meta["data_offsets"]
                count = (hi - lo) // np.dtype(np_dt).itemsize
                arr = np.frombuffer(mm, dtype=np_dt, count=count, offset=base + lo).copy()
                t = torch.from_numpy(arr)
                if view is not None:
                    t = t.view(view)
                out[name] = t.reshape(meta["shape"]).to(device)
        finally:
            mm.close()
    return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """The inverse, for tools and tests that make a model folder (floating tensors as given, ints as int32)."""
    names = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32", torch.int32: "I32",
             torch.int64: "I64"}
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
