"""Reader and writer of the tensor dump format of the reference's prototypes.

A ``.bin`` file is ``int32 M, int32 N`` followed by ``M * N`` binary32 values in row-major
order, native little-endian (the reference reads it with three ``fread`` calls:
mor/csrc/cuda/jatin/V3/cpu_computation.cpp:18-32).  Captured tensors in that format can be
replayed through the operators and through ``bench.py --suite-bin``.
"""
from __future__ import annotations

import os
import struct

import numpy as np
import torch


def read_bin(path: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Returns the ``[M, N]`` tensor of a ``.bin`` file (float32, or rounded to ``dtype``)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: shorter than the 8-byte header")
        m, n = struct.unpack("<ii", head)
        if m <= 0 or n <= 0:
            raise ValueError(f"{path}: bad dimensions {m} x {n}")
        if size != 8 + 4 * m * n:
            raise ValueError(f"{path}: {size} bytes, expected {8 + 4 * m * n} for {m} x {n} float32")
        data = np.fromfile(f, dtype="<f4", count=m * n)
    t = torch.from_numpy(data.reshape(m, n).copy())
    return t if dtype == torch.float32 else t.to(dtype)


def write_bin(path: str, t: torch.Tensor) -> None:
    """Writes a 2-D tensor in the same format (values widened to float32)."""
    if t.dim() != 2:
        raise ValueError("a .bin file holds one 2-D tensor")
    a = t.detach().to("cpu", torch.float32).contiguous().numpy()
    with open(path, "wb") as f:
        f.write(struct.pack("<ii", a.shape[0], a.shape[1]))
        a.astype("<f4", copy=False).tofile(f)
