"""Device tensors without a tensor library: a pointer-stable buffer plus shape/dtype.

The reference hands torch.Tensor objects to its binding; callers of this backend may do the same
(anything with data_ptr()/shape/stride()/dtype works), or use this class, which needs only NumPy.
bf16 has no NumPy dtype: host arrays carry it as uint16 bit patterns.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from ._lib import check, lib

DTYPE_CODES = {"f32": 1, "f16": 2, "bf16": 3, "i32": 4}
DTYPE_SIZES = {"f32": 4, "f16": 2, "bf16": 2, "i32": 4}
_NP_OF = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16, "i32": np.int32}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned as uint16 bit patterns (NaN stays NaN)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    return np.where(nan, (u >> np.uint32(16)) | np.uint32(0x40), rounded).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


class Tensor:
    """Contiguous device buffer. Owns its memory unless built with `ptr=`."""

    def __init__(self, shape: Sequence[int], dtype: str, ptr: int | None = None):
        if dtype not in DTYPE_CODES:
            raise ValueError(f"unsupported dtype {dtype!r}")
        self.shape = tuple(int(s) for s in shape)
        if len(self.shape) > 4:
            raise ValueError("rank must be <= 4")
        self.dtype = dtype
        self.numel = int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1
        self.nbytes = self.numel * DTYPE_SIZES[dtype]
        self._owned = ptr is None
        if ptr is None:
            p = C.c_void_p()
            check(lib.aicf_b200_malloc(C.byref(p), max(self.nbytes, 1)), "malloc")
            ptr = p.value
        self.ptr = int(ptr)

    # --- duck-typing surface shared with torch.Tensor -------------------------------------------
    def data_ptr(self) -> int:
        return self.ptr

    def stride(self) -> tuple[int, ...]:
        st, acc = [], 1
        for s in reversed(self.shape):
            st.append(acc)
            acc *= s
        return tuple(reversed(st))

    def is_contiguous(self) -> bool:
        return True

    def dim(self) -> int:
        return len(self.shape)

    # --- construction / transfer -----------------------------------------------------------------
    @classmethod
    def empty(cls, shape, dtype="f32") -> "Tensor":
        return cls(shape, dtype)

    @classmethod
    def zeros(cls, shape, dtype="f32") -> "Tensor":
        t = cls(shape, dtype)
        t.zero_()
        return t

    @classmethod
    def from_numpy(cls, arr: np.ndarray, dtype: str | None = None) -> "Tensor":
        """dtype=None infers f32/f16/i32 from the array; dtype='bf16' accepts float32 (rounded to
        nearest even) or uint16 bit patterns."""
        arr = np.asarray(arr)
        if dtype is None:
            dtype = {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16", np.dtype(np.int32): "i32"}.get(arr.dtype)
            if dtype is None:
                raise ValueError(f"cannot infer device dtype from {arr.dtype}")
        if dtype == "bf16":
            host = arr.astype(np.uint16) if arr.dtype == np.uint16 else f32_to_bf16_bits(arr.astype(np.float32))
        else:
            host = arr.astype(_NP_OF[dtype])
        host = np.ascontiguousarray(host)
        t = cls(arr.shape, dtype)
        t.copy_from_host(host)
        return t

    def copy_from_host(self, host: np.ndarray, stream: int = 0) -> None:
        host = np.ascontiguousarray(host)
        if host.nbytes != self.nbytes:
            raise ValueError(f"size mismatch: host {host.nbytes} B vs device {self.nbytes} B")
        check(lib.aicf_b200_memcpy_h2d(self.ptr, host.ctypes.data, self.nbytes, stream), "memcpy_h2d")
        check(lib.aicf_b200_stream_sync(stream), "stream_sync")

    def numpy(self, stream: int = 0) -> np.ndarray:
        """Device -> host copy. bf16 comes back as uint16 bit patterns (see bf16_bits_to_f32)."""
        out = np.empty(self.shape, dtype=_NP_OF[self.dtype])
        if self.nbytes:
            check(lib.aicf_b200_memcpy_d2h(out.ctypes.data, self.ptr, self.nbytes, stream), "memcpy_d2h")
            check(lib.aicf_b200_stream_sync(stream), "stream_sync")
        return out

    def float_numpy(self) -> np.ndarray:
        """Host copy widened to float32 (int32 tensors are returned unchanged)."""
        a = self.numpy()
        if self.dtype == "bf16":
            return bf16_bits_to_f32(a).reshape(self.shape)
        return a.astype(np.float32) if self.dtype == "f16" else a

    def zero_(self) -> "Tensor":
        check(lib.aicf_b200_memset(self.ptr, 0, self.nbytes, 0), "memset")
        check(lib.aicf_b200_stream_sync(0), "stream_sync")
        return self

    def view(self, shape) -> "Tensor":
        v = Tensor(shape, self.dtype, ptr=self.ptr)
        if v.nbytes != self.nbytes:
            raise ValueError("view changes the number of bytes")
        v._base = self  # keep the owner alive
        return v

    def __del__(self):
        if getattr(self, "_owned", False) and getattr(self, "ptr", 0):
            try:
                lib.aicf_b200_free(self.ptr)
            except Exception:
                pass
            self.ptr = 0

    def __repr__(self) -> str:
        return f"aicf_cuda.Tensor(shape={self.shape}, dtype={self.dtype}, ptr=0x{self.ptr:x})"
