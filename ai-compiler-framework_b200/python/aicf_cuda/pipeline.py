"""Host-side input pipeline for the captured train step: double-buffered plans so that the host-to-device
copy of the next batch overlaps the replay of the current one.

A captured graph reads its input batch until its last backward GEMM, so the next batch cannot land in
the same buffer while a step runs. Two plans are built from the same lowered list; the second one binds
every parameter, optimizer-state and working-copy value to the first one's buffers, so both graphs
update the same model and only the inputs and activations exist twice. Replays of both plans go into
one stream (they are ordered); copies go through a second stream and are tied to the replays by events.

The reference feeds its executor with tensors that already live on the device
(python/aicf_fw/core_v2/exec.py:337-390) and has no input pipeline; this is an addition.
"""
from __future__ import annotations

import ctypes as C
from typing import Any, Callable, Dict, List, Sequence

import numpy as np

from ._lib import check, lib
from .plan import Plan, ValueSpec


def _shared(name: str) -> bool:
    """Values that are model state (shared by both plans) rather than per-batch data."""
    head = name.split(".")[0]
    return name.startswith("opt.") or head.isdigit()


def _event() -> int:
    e = C.c_uint64()
    check(lib.aicf_b200_event_create(C.byref(e)), "event_create")
    return int(e.value)


class DoubleBufferedStep:
    def __init__(self, name: str, values: Sequence[ValueSpec], lowered: Sequence[Dict[str, Any]],
                 input_names: Sequence[str] = ("x", "labels"), result_name: str = "loss"):
        self.a = Plan(name + ".a", values, lowered)
        bind = {v.vid: self.a.tensor(v.vid) for v in values if v.alias_of is None and _shared(v.name)}
        self.b = Plan(name + ".b", values, lowered, bind=bind)
        self.plans = [self.a, self.b]
        self.inputs = [[p.tensor(n) for n in input_names] for p in self.plans]
        self.results = [p.tensor(result_name) for p in self.plans]
        self.main = self.a.stream
        s = C.c_uint64()
        check(lib.aicf_b200_stream_create(C.byref(s)), "stream_create")
        self.copy_stream = int(s.value)
        self.ev_copied = [_event(), _event()]
        self.ev_done = [_event(), _event()]
        self.ev_result = [_event(), _event()]
        self.used = [False, False]
        self.t = 0
        # pinned landing zone for the per-step result (one slot per plan)
        p = C.c_void_p()
        check(lib.aicf_b200_host_alloc_pinned(C.byref(p), 2 * self.results[0].nbytes), "host_alloc_pinned")
        self._result_ptr = p.value
        nb = self.results[0].nbytes
        buf = (C.c_uint8 * (2 * nb)).from_address(p.value)
        self._result_host = np.frombuffer(buf, dtype=np.float32).reshape(2, -1)

    def connect(self, rank: int, world: int, allgather) -> None:
        """Data-parallel runs with dp_adam_step ops: maps the peers' pools for both plans (see dp.connect_plans)."""
        from .dp import connect_plans
        connect_plans(self.plans, rank, world, allgather)

    def capture(self) -> None:
        for p in self.plans:
            p.capture()

    def submit(self, host_arrays: Sequence[np.ndarray]) -> int:
        """Enqueues: copy of this step's (pinned) host inputs, one replay, copy-out of the result.
        Returns the slot to pass to result(). Does not block."""
        i = self.t & 1
        if self.used[i]:  # the slot's previous replay must have consumed its inputs
            check(lib.aicf_b200_stream_wait_event(self.copy_stream, self.ev_done[i]), "stream_wait_event")
        for dst, src in zip(self.inputs[i], host_arrays):
            check(lib.aicf_b200_memcpy_h2d(dst.ptr, src.ctypes.data, dst.nbytes, self.copy_stream), "memcpy_h2d")
        check(lib.aicf_b200_event_record(self.ev_copied[i], self.copy_stream), "event_record")
        check(lib.aicf_b200_stream_wait_event(self.main, self.ev_copied[i]), "stream_wait_event")
        self.plans[i].replay(1, stream=self.main)
        check(lib.aicf_b200_event_record(self.ev_done[i], self.main), "event_record")
        nb = self.results[i].nbytes
        check(lib.aicf_b200_memcpy_d2h(self._result_ptr + i * nb, self.results[i].ptr, nb, self.main), "memcpy_d2h")
        check(lib.aicf_b200_event_record(self.ev_result[i], self.main), "event_record")
        self.used[i] = True
        self.t += 1
        return i

    def result(self, slot: int) -> np.ndarray:
        """Blocks until the step submitted into `slot` has delivered its result to the host."""
        check(lib.aicf_b200_event_sync(self.ev_result[slot]), "event_sync")
        return self._result_host[slot].copy()

    def sync(self) -> None:
        check(lib.aicf_b200_stream_sync(self.copy_stream), "stream_sync")
        for p in self.plans:
            p.sync()

    def close(self) -> None:
        self.sync()
        self.b.close()
        self.a.close()
