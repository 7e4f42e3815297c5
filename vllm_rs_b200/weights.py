"""Checkpoint reading: the safetensors container (8-byte little-endian header length, a JSON header mapping tensor
name -> dtype / shape / data_offsets, then the raw little-endian data) into torch tensors, and config.json."""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import numpy as np
import torch

_DTYPES = {"BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
           "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
           "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1)}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Every tensor of one .safetensors file, on the CPU, in its stored dtype (the file is memory-mapped and copied
    tensor by tensor, so the result does not keep the mapping alive)."""
    out = {}
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            (n,) = struct.unpack("<Q", mm[:8])
            header = json.loads(mm[8:8 + n].decode("utf-8"))
            base = 8 + n
            for name, info in header.items():
                if name == "__metadata__":
                    continue
                if info["dtype"] not in _DTYPES:
                    raise ValueError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
                dt, size = _DTYPES[info["dtype"]]
                lo, hi = info["data_offsets"]
                count = int(np.prod(info["shape"])) if info["shape"] else 1
                if hi - lo != count * size:
                    raise ValueError(f"{path}: tensor {name} has {hi - lo} bytes for shape {info['shape']}")
                raw = torch.frombuffer(bytearray(mm[base + lo:base + hi]), dtype=torch.uint8)
                out[name] = raw.view(dt).reshape(info["shape"]).clone() if count else torch.empty(info["shape"], dtype=dt)
        finally:
            mm.close()
    return out


def read_model_dir(model_dir) -> tuple[dict, dict[str, torch.Tensor]]:
    """(config.json as a dict, all tensors of the *.safetensors files of a model folder)."""
    d = Path(model_dir)
    with open(d / "config.json") as f:
        cfg = json.load(f)
    tensors: dict[str, torch.Tensor] = {}
    files = sorted(d.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors file in {d}")
    for p in files:
        tensors.update(read_safetensors(p))
    return cfg, tensors
