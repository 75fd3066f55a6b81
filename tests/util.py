"""Helpers shared by the GPU parity tests: call ops through the binding on aicf_cuda.Tensor buffers."""
from __future__ import annotations

import contextlib
import ctypes as C
import os
import struct

import numpy as np

import aicf_cuda
from aicf_cuda import _C, Tensor
from aicf_cuda._C import OpKind
from aicf_cuda._C_ctypes import _blob, _build_descs


def dev(arr, dtype=None) -> Tensor:
    return Tensor.from_numpy(np.asarray(arr), dtype)


def host(t: Tensor) -> np.ndarray:
    return t.float_numpy()


def by_id(kid: str, kind, ins, outs, schema=0, payload=b"") -> None:
    _C.launch_by_id(kid, OpKind(int(kind)), ins, outs, schema, payload)
    _C.device_sync()


def op_call(kind, ins, outs, schema=0, payload=b"") -> None:
    _C.op_call(OpKind(int(kind)), ins, outs, schema, payload)
    _C.device_sync()


def ref_by_id(ref_lib, kid: str, kind, ins, outs, schema=0, payload=b"") -> int:
    """Runs the REFERENCE's kernel `kid` on the same device buffers; returns its status code."""
    di, ni = _build_descs(ins, "inputs")
    do, no = _build_descs(outs, "outputs")
    blob, _keep = _blob(schema, payload)
    st = ref_lib.ref_launch_by_id(kid.encode(), int(kind), C.cast(di, C.c_void_p), ni, C.cast(do, C.c_void_p), no,
                                  C.cast(blob, C.c_void_p) if blob is not None else None, 0)
    ref_lib.ref_device_sync()
    return int(st)


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """Normwise relative error max|got-want| / max|want| (the GEMM tolerance is stated in this norm)."""
    want = np.asarray(want, np.float64)
    denom = max(float(np.max(np.abs(want))), 1e-30)
    return float(np.max(np.abs(np.asarray(got, np.float64) - want))) / denom


def assert_close_f32(got, want, rtol=1e-5, atol=1e-7, what=""):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    bad = np.abs(got - want) > (atol + rtol * np.abs(want))
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} elements off; max abs err {np.max(np.abs(got - want)):.3e}"


GEMM = struct.Struct("<ii")
GEPL = struct.Struct("<iii")


@contextlib.contextmanager
def gemm_tuning(**settings):
    """Runs the body with AICF_GEMM_<NAME>=value overrides in force (None removes a variable). The GEMM launcher reads
    its environment once per process, so every change is followed by a reload, and so is the restore."""
    names = {f"AICF_GEMM_{k.upper()}": v for k, v in settings.items()}
    saved = {n: os.environ.get(n) for n in names}

    def apply(values):
        for n, v in values.items():
            if v is None:
                os.environ.pop(n, None)
            else:
                os.environ[n] = str(v)
        aicf_cuda._lib.check(aicf_cuda.lib.aicf_b200_gemm_reload_tuning(), "gemm_reload_tuning")

    apply(names)
    try:
        yield
    finally:
        apply(saved)
