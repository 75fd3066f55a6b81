"""Loads libaicf_b200.so and declares the C ABI (include/aicf_b200.h) for ctypes.

There is no fallback: if the library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG_ROOT = Path(__file__).resolve().parents[2]  # .../ai-compiler-framework_b200
LIB_PATH = Path(os.environ.get("AICF_B200_LIB", _PKG_ROOT / "lib" / "libaicf_b200.so"))


class TensorDesc(C.Structure):
    """aicf_tensor_desc (96 bytes)."""
    _fields_ = [
        ("data", C.c_void_p),
        ("dtype", C.c_uint8),
        ("rank", C.c_int32),
        ("shape", C.c_int64 * 4),
        ("stride", C.c_int64 * 4),
        ("contiguous", C.c_uint8),
        ("alignment", C.c_int32),
        ("device", C.c_int32),
    ]


class AttrBlob(C.Structure):
    """aicf_attr_blob (16 bytes)."""
    _fields_ = [("schema_id", C.c_uint32), ("bytes", C.c_uint32), ("data", C.c_void_p)]


assert C.sizeof(TensorDesc) == 96 and C.sizeof(AttrBlob) == 16


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python {_PKG_ROOT / 'build.py'}` "
            "(there is no CPU or library fallback for the CUDA backend)")
    return C.CDLL(str(LIB_PATH))


lib = _load()

_P = C.POINTER
_desc_p, _blob_p = _P(TensorDesc), _P(AttrBlob)
_u64, _i, _sz, _vp, _cp = C.c_uint64, C.c_int, C.c_size_t, C.c_void_p, C.c_char_p

# name -> (restype, argtypes); mirrors include/aicf_b200.h one to one
PROTOTYPES = {
    "aicf_b200_abi_version": (_i, []),
    "aicf_b200_status_string": (_cp, [_i]),
    "aicf_b200_last_error": (_cp, []),
    "aicf_b200_op_name": (_cp, [_i]),
    "aicf_b200_op_call": (_i, [_i, _desc_p, _i, _desc_p, _i, _blob_p, _u64]),
    "aicf_b200_launch_by_id": (_i, [_cp, _i, _desc_p, _i, _desc_p, _i, _blob_p, _u64]),
    "aicf_b200_supported": (_i, [_cp, _i, _desc_p, _i, _desc_p, _i, _blob_p]),
    "aicf_b200_query_workspace": (_sz, [_cp, _i, _desc_p, _i, _blob_p]),
    "aicf_b200_launch_ws": (_i, [_cp, _i, _desc_p, _i, _desc_p, _i, _blob_p, _vp, _sz, _u64]),
    "aicf_b200_set_workspace": (_i, [_vp, _sz]),
    "aicf_b200_kernel_count": (_i, [_i]),
    "aicf_b200_kernel_id": (_cp, [_i, _i]),
    "aicf_b200_num_op_kinds": (_i, []),
    "aicf_b200_gemm_status": (_i, [_i]),
    "aicf_b200_gemm_reload_tuning": (_i, []),
    "aicf_b200_wait_status": (_i, [_i]),
    "aicf_b200_gemm_timeline": (_i, [_i, _P(C.c_uint64)]),
    "aicf_b200_colsum_f32_noalloc": (_i, [_vp, _vp, C.c_int64, C.c_int64, _u64]),
    "aicf_b200_trace_enable": (None, [_i]),
    "aicf_b200_trace_reset": (None, []),
    "aicf_b200_trace_count": (_i, []),
    "aicf_b200_trace_get": (_cp, [_i]),
    "aicf_b200_op_call_traced": (_i, [_i, _desc_p, _i, _desc_p, _i, _blob_p, _u64]),
    "aicf_b200_launch_by_id_traced": (_i, [_cp, _i, _desc_p, _i, _desc_p, _i, _blob_p, _u64]),
    "aicf_b200_graph_begin": (_i, [_P(_u64)]),
    "aicf_b200_graph_end": (_i, []),
    "aicf_b200_graph_launch": (_i, []),
    "aicf_b200_graph_reset": (_i, []),
    "aicf_b200_graph_stream": (_u64, []),
    "aicf_b200_device_count": (_i, []),
    "aicf_b200_set_device": (_i, [_i]),
    "aicf_b200_device_pci_bus_id": (_i, [_i, C.c_char_p, _i]),
    "aicf_b200_device_info": (_i, [_i, _P(C.c_int64), _P(C.c_int), _P(C.c_int64)]),
    "aicf_b200_stream_probe": (_i, [_i, _i, _P(_vp), _P(_vp), _sz, _i, _i, _u64]),
    "aicf_b200_malloc": (_i, [_P(_vp), _sz]),
    "aicf_b200_free": (_i, [_vp]),
    "aicf_b200_host_alloc_pinned": (_i, [_P(_vp), _sz]),
    "aicf_b200_host_alloc_staging": (_i, [_P(_vp), _sz]),
    "aicf_b200_host_free_pinned": (_i, [_vp]),
    "aicf_b200_memcpy_h2d": (_i, [_vp, _vp, _sz, _u64]),
    "aicf_b200_memcpy_d2h": (_i, [_vp, _vp, _sz, _u64]),
    "aicf_b200_memcpy_d2d": (_i, [_vp, _vp, _sz, _u64]),
    "aicf_b200_memset": (_i, [_vp, _i, _sz, _u64]),
    "aicf_b200_stream_create": (_i, [_P(_u64)]),
    "aicf_b200_stream_destroy": (_i, [_u64]),
    "aicf_b200_stream_sync": (_i, [_u64]),
    "aicf_b200_device_sync": (_i, []),
    "aicf_b200_event_create": (_i, [_P(_u64)]),
    "aicf_b200_event_destroy": (_i, [_u64]),
    "aicf_b200_event_record": (_i, [_u64, _u64]),
    "aicf_b200_event_sync": (_i, [_u64]),
    "aicf_b200_event_elapsed_ms": (_i, [_u64, _u64, _P(C.c_float)]),
    "aicf_b200_stream_wait_event": (_i, [_u64, _u64]),
    "aicf_b200_plan_create": (_vp, [_cp]),
    "aicf_b200_plan_destroy": (None, [_vp]),
    "aicf_b200_plan_add_value": (_i, [_vp, _i, _cp, _i, _i, _P(C.c_int64), _i, _i, _i]),
    "aicf_b200_plan_add_op": (_i, [_vp, _cp, _cp, _P(_i), _i, _P(_i), _i, C.c_uint32, _vp, C.c_uint32]),
    "aicf_b200_plan_alias": (_i, [_vp, _i, _i]),
    "aicf_b200_plan_bind": (_i, [_vp, _i, _vp]),
    "aicf_b200_plan_set_peer_visible": (_i, [_vp, _i]),
    "aicf_b200_plan_peer_handle": (_i, [_vp, _vp, _P(_sz)]),
    "aicf_b200_plan_open_peers": (_i, [_vp, _i, _i, _vp]),
    "aicf_b200_plan_open_peers_raw": (_i, [_vp, _i, _i, _P(_vp)]),
    "aicf_b200_plan_peer_pool_bytes": (_sz, [_vp]),
    "aicf_b200_plan_peer_pool_base": (_vp, [_vp, _i]),
    "aicf_b200_plan_finalize": (_i, [_vp]),
    "aicf_b200_plan_value_ptr": (_vp, [_vp, _i]),
    "aicf_b200_plan_value_bytes": (_sz, [_vp, _i]),
    "aicf_b200_plan_value_arena_offset": (C.c_int64, [_vp, _i]),
    "aicf_b200_plan_arena_bytes": (_sz, [_vp]),
    "aicf_b200_plan_arena_bytes_no_reuse": (_sz, [_vp]),
    "aicf_b200_plan_num_ops": (_i, [_vp]),
    "aicf_b200_plan_op_kernel_id": (_cp, [_vp, _i]),
    "aicf_b200_plan_run": (_i, [_vp, _u64]),
    "aicf_b200_plan_capture": (_i, [_vp]),
    "aicf_b200_plan_replay": (_i, [_vp, _i]),
    "aicf_b200_plan_replay_on": (_i, [_vp, _i, _u64]),
    "aicf_b200_plan_reset_graph": (_i, [_vp]),
    "aicf_b200_plan_stream": (_u64, [_vp]),
    "aicf_b200_plan_sync": (_i, [_vp]),
    "aicf_b200_plan_graph_nodes": (_i, [_vp]),
    "aicf_b200_plan_graph_kernel_nodes": (_i, [_vp]),
    "aicf_b200_plan_profile": (_i, [_vp, _P(C.c_float), _i]),
    "aicf_b200_dp_unique_id": (_i, [_vp]),
    "aicf_b200_dp_init": (_i, [_i, _i, _vp]),
    "aicf_b200_dp_finalize": (_i, []),
    "aicf_b200_dp_world_size": (_i, []),
    "aicf_b200_dp_rank": (_i, []),
}

for _name, (_res, _args) in PROTOTYPES.items():
    _fn = getattr(lib, _name)  # AttributeError here means header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.aicf_b200_last_error().decode()


def check(rc: int, what: str = "") -> None:
    """Raises RuntimeError carrying the library's message when a call did not return Ok."""
    if rc != 0:
        msg = last_error() or f"{what} failed with status {rc}"
        raise RuntimeError(msg)
