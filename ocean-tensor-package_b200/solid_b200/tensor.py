"""Device tensors as Ocean describes them: a dtype, sizes, byte strides, a byte
order flag and a pointer into a storage, column-major by default
(docs/design_choices.md:25-27 of the reference).  torch only owns the device
memory and the stream; every computation goes through the C-ABI library.
"""
from __future__ import annotations

import numpy as np

from . import dtypes as dt


def _torch():
    import torch
    return torch


class Tensor:
    """A view into device storage.

    storage      torch.uint8 CUDA tensor that owns the bytes
    offset       byte offset of element (0,...,0)
    size/strides per dimension, strides in bytes (0 broadcasts, negative allowed)
    byteswapped  stored bytes of each real component are reversed
    """

    def __init__(self, storage, dtype: str, size, strides=None, offset: int = 0, byteswapped: bool = False):
        self.storage, self.dtype, self.size = storage, dtype, [int(s) for s in size]
        if strides is None:
            strides, step = [], dt.SIZE[dtype]
            for s in self.size:
                strides.append(step)
                step *= s
        self.strides = [int(s) for s in strides]
        self.offset, self.byteswapped = int(offset), bool(byteswapped)

    # -- construction ------------------------------------------------------------
    @staticmethod
    def empty(size, dtype: str, device=None) -> "Tensor":
        torch = _torch()
        n = 1
        for s in size:
            n *= int(s)
        storage = torch.empty(max(n * dt.SIZE[dtype], 16), dtype=torch.uint8, device=device or "cuda")
        return Tensor(storage, dtype, size)

    @staticmethod
    def from_numpy(array: np.ndarray, dtype: str | None = None, device=None) -> "Tensor":
        """Upload a numpy array (its Fortran-order element sequence becomes the column-major tensor)."""
        torch = _torch()
        if dtype is None:
            dtype = {np.dtype(np.float32): "float", np.dtype(np.float64): "double", np.dtype(np.float16): "half",
                     np.dtype(np.complex64): "cfloat", np.dtype(np.complex128): "cdouble",
                     np.dtype(np.bool_): "bool"}.get(array.dtype) or \
                    next(n for n in dt.NAMES if n not in ("bool", "half", "chalf") and dt.NUMPY[n] == array.dtype)
        flat = np.asfortranarray(array).reshape(-1, order="F")
        raw = np.ascontiguousarray(flat).view(np.uint8)
        storage = torch.from_numpy(raw.copy()).to(device or "cuda")
        if storage.numel() < 16:
            storage = torch.cat([storage, torch.zeros(16 - storage.numel(), dtype=torch.uint8, device=storage.device)])
        return Tensor(storage, dtype, array.shape)

    # -- properties ---------------------------------------------------------------
    @property
    def ptr(self) -> int:
        return self.storage.data_ptr() + self.offset

    @property
    def ndims(self) -> int:
        return len(self.size)

    @property
    def nelem(self) -> int:
        n = 1
        for s in self.size:
            n *= s
        return n

    @property
    def elemsize(self) -> int:
        return dt.SIZE[self.dtype]

    @property
    def device_index(self) -> int:
        return self.storage.device.index or 0

    def is_contiguous(self) -> bool:
        step = self.elemsize
        for s, st in zip(self.size, self.strides):
            if s != 1 and st != step:
                return False
            step *= s
        return True

    # -- views (no data movement) ---------------------------------------------------
    def transpose(self, a: int = 0, b: int = 1) -> "Tensor":
        size, strides = list(self.size), list(self.strides)
        size[a], size[b] = size[b], size[a]
        strides[a], strides[b] = strides[b], strides[a]
        return Tensor(self.storage, self.dtype, size, strides, self.offset, self.byteswapped)

    @property
    def T(self) -> "Tensor":
        return Tensor(self.storage, self.dtype, self.size[::-1], self.strides[::-1], self.offset, self.byteswapped)

    def broadcast_to(self, size) -> "Tensor":
        size = list(size)
        strides = []
        own = [1] * (len(size) - self.ndims) + self.size
        ost = [0] * (len(size) - self.ndims) + self.strides
        for s, o, st in zip(size, own, ost):
            if o == s:
                strides.append(st)
            elif o == 1:
                strides.append(0)
            else:
                raise ValueError("cannot broadcast %s to %s" % (self.size, size))
        return Tensor(self.storage, self.dtype, size, strides, self.offset, self.byteswapped)

    def as_strided(self, size, strides, offset=None) -> "Tensor":
        return Tensor(self.storage, self.dtype, size, strides, self.offset if offset is None else offset, self.byteswapped)

    def slice(self, dim: int, start: int, stop: int, step: int = 1) -> "Tensor":
        size, strides = list(self.size), list(self.strides)
        size[dim] = max(0, (stop - start + step - 1) // step) if step > 0 else max(0, (start - stop - step - 1) // -step)
        off = self.offset + start * strides[dim]
        strides[dim] *= step
        return Tensor(self.storage, self.dtype, size, strides, off, self.byteswapped)

    # -- download -----------------------------------------------------------------------
    def numpy(self) -> np.ndarray:
        """Elements as a numpy array of the carrier type, shape `size` (Fortran order)."""
        from . import ops
        dense = ops.clone(self) if (not self.is_contiguous() or self.byteswapped) else self
        torch = _torch()
        torch.cuda.synchronize(dense.storage.device)
        raw = dense.storage[dense.offset: dense.offset + dense.nelem * dense.elemsize].cpu().numpy()
        arr = raw.view(dt.NUMPY[self.dtype])
        return arr.reshape(self.size, order="F") if self.size else arr.reshape(())

    def __repr__(self):
        return "Tensor(%s, size=%s, strides=%s%s)" % (self.dtype, self.size, self.strides,
                                                     ", byteswapped" if self.byteswapped else "")
