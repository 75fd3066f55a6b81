"""Python face of the C++ captured plan (include/aicf_b200.h, "captured execution plan").

Mirrors the reference's executor surface - PlannedExecutor.run / capture / replay / reset_graph
(python/aicf_fw/core_v2/exec.py:455-497) and build_binding_plan's role rules
(python/aicf_fw/core_v2/plan.py:65-74,101-112,160-171) - but the per-op loop, the buffers and the
CUDA graph live in C++: Python only describes the lowered-op list once.
"""
from __future__ import annotations

import ctypes as C
import struct
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

from ._lib import check, lib
from .spec import ROLE_INPUT, ROLE_PARAM, ROLE_STATIC, ValueSpec, classify_role, needs_zero_init  # noqa: F401  (re-exported)
from .tensor import DTYPE_CODES, Tensor


# Attr schema tags: the contract is the numeric value (the reference spells some big-endian).
SCHEMA_GEMM = 0x47454D4D
SCHEMA_GEMM_EPILOGUE = 0x4750454C
SCHEMA_REDUCE_SUM = 0x5253554D
SCHEMA_ADAM = 0x4D414441
SCHEMA_BIAS_CORR = 0x524F4342
SCHEMA_SGD = 0x53444753
SCHEMA_BIAS_ADD = 0x44444142
SCHEMA_MSE_GRAD = 0x4745534D
SCHEMA_SOFTMAX_CE = 0x45434D53
SCHEMA_LAYERNORM = 0x50454E4C  # 'LNEP'

SCHEMA_ALL_REDUCE = 0x44455241
SCHEMA_DP_ADAM = 0x44415044
# What the reference's Python executor sends for gemm_epilogue (exec.py:215-217); the reference's C++
# does not know this tag and silently applies its defaults.
SCHEMA_GEPI_AS_SENT_BY_REFERENCE_EXECUTOR = int.from_bytes(b"GEPI", "little")


def _relu_flag(attrs: Dict[str, Any]) -> int:
    if "relu" in attrs:
        return 1 if attrs["relu"] else 0
    if "epilogue" in attrs:
        return 0 if str(attrs["epilogue"]).strip().lower() in ("bias", "bias_only", "biasonly") else 1
    if "epilogue_act" in attrs:
        return 1 if str(attrs["epilogue_act"]).strip().lower() == "relu" else 0
    return 1


def pack_attrs(op: str, attrs: Optional[Dict[str, Any]]) -> Tuple[int, bytes]:
    """(schema_id, payload) for every op that has a schema. Unlike the reference's _pack_attrs
    (exec.py:263-277), which only packs gemm / gemm_epilogue / adam_step, nothing is dropped."""
    op = str(op).strip().lower()
    a = dict(attrs or {})
    ta, tb = int(bool(a.get("transA", False))), int(bool(a.get("transB", False)))
    if op in ("gemm", "gemm_relu_bwd"):
        return SCHEMA_GEMM, struct.pack("<ii", ta, tb)
    if op == "gemm_epilogue":
        return SCHEMA_GEMM_EPILOGUE, struct.pack("<iii", ta, tb, _relu_flag(a))
    if op == "reduce_sum":
        return SCHEMA_REDUCE_SUM, struct.pack("<q", int(a.get("axis", 0)))
    if op == "adam_step":
        payload = struct.pack("<ffff", float(a.get("lr", 1e-3)), float(a.get("beta1", 0.9)),
                              float(a.get("beta2", 0.999)), float(a.get("eps", 1e-8)))
        if "weight_decay" in a or "decoupled" in a or "count" in a:
            payload += struct.pack("<fI", float(a.get("weight_decay", 0.0)), 1 if a.get("decoupled", False) else 0)
        if "count" in a:  # multi-tensor form (adam_step_f32_multi_v1): tensor count and which tensors have a 16-bit copy
            payload += struct.pack("<II", int(a["count"]), int(a.get("lp_mask", 0)))
        return SCHEMA_ADAM, payload
    if op == "dp_adam_step":
        payload = struct.pack("<fffffIi", float(a.get("lr", 1e-3)), float(a.get("beta1", 0.9)),
                              float(a.get("beta2", 0.999)), float(a.get("eps", 1e-8)),
                              float(a.get("weight_decay", 0.0)), 1 if a.get("decoupled", False) else 0, int(a["slot"]))
        if a.get("defer_done") or a.get("fence_slots") or a.get("solo"):
            # defer_done: this op does not wait for the peers' "done" words; fence_slots = n: this op (the last
            # exchange of the step) waits for the done words of slots [0, n) before it finishes; solo: nothing runs
            # beside this op, so it may fill the SMs instead of leaving room for GEMM CTAs
            payload += struct.pack("<ii", (1 if a.get("defer_done") else 0) | (2 if a.get("solo") else 0), int(a.get("fence_slots", 0)))
        return SCHEMA_DP_ADAM, payload
    if op == "bias_corr":
        return SCHEMA_BIAS_CORR, struct.pack("<ff", float(a.get("beta1", 0.9)), float(a.get("beta2", 0.999)))
    if op == "sgd_step" and "lr" in a:
        return SCHEMA_SGD, struct.pack("<f", float(a["lr"]))
    if op == "mse_grad" and "scale" in a:
        return SCHEMA_MSE_GRAD, struct.pack("<f", float(a["scale"]))
    if op == "bias_add" and "axis" in a:
        return SCHEMA_BIAS_ADD, struct.pack("<q", int(a["axis"]))
    if op == "softmax_ce" and "scale" in a:
        return SCHEMA_SOFTMAX_CE, struct.pack("<f", float(a["scale"]))
    if op == "layernorm_fwd" and "eps" in a:
        return SCHEMA_LAYERNORM, struct.pack("<f", float(a["eps"]))
    if op == "all_reduce":
        return SCHEMA_ALL_REDUCE, struct.pack("<i", int(a.get("bucket", 0)))
    return 0, b""


def pack_attrs_like_reference_executor(op: str, attrs: Optional[Dict[str, Any]]) -> Tuple[int, bytes]:
    """Bit-for-bit what the reference's exec.py:_pack_attrs emits (for strict-parity comparisons):
    gemm -> schema 0 <ii>; gemm_epilogue -> 'GEPI' <iii>(ta,tb,kind); adam_step -> 'ADAM' <ffff>;
    every other op -> no attrs."""
    op = str(op).strip().lower()
    a = dict(attrs or {})
    ta, tb = int(bool(a.get("transA", False))), int(bool(a.get("transB", False)))
    if op == "gemm":
        return 0, struct.pack("<ii", ta, tb)
    if op == "gemm_epilogue":
        epi = str(a.get("epilogue", "bias_relu")).strip().lower()
        kind = 1 if epi in ("bias", "bias_only", "biasonly") else 2 if epi in ("relu", "relu_only", "reluonly") else 0
        return SCHEMA_GEPI_AS_SENT_BY_REFERENCE_EXECUTOR, struct.pack("<iii", ta, tb, kind)
    if op == "adam_step":
        return SCHEMA_ADAM, struct.pack("<ffff", float(a.get("lr", 1e-3)), float(a.get("beta1", 0.9)),
                                        float(a.get("beta2", 0.999)), float(a.get("eps", 1e-8)))
    return 0, b""


def plan_to_json(name: str, values: Iterable[ValueSpec], lowered: Sequence[Dict[str, Any]]) -> str:
    """On-disk form of a compiled plan: the lowered-op list plus the value table, as JSON.

    The lowered part is the reference's own contract ({"op","inputs","outputs","attrs","kernel_id"},
    python/aicf_fw/core_v2/lower.py:9-21); the value table carries what its text dump prints per value
    (core_v2/printer.py:115-147: id, name, role, shape, dtype) plus this backend's placement flags."""
    import json
    vals = [{"vid": v.vid, "name": v.name, "shape": list(v.shape), "dtype": v.dtype,
             "role": classify_role(v.name) if v.role is None else v.role, "persistent": bool(v.persistent),
             "zero_init": needs_zero_init(v.name) if v.zero_init is None else bool(v.zero_init),
             "alias_of": v.alias_of, "peer_visible": bool(v.peer_visible)} for v in values]
    ops = [{"op": it["op"], "inputs": list(it.get("inputs", [])), "outputs": list(it.get("outputs", [])),
            "attrs": dict(it.get("attrs") or {}), **({"kernel_id": it["kernel_id"]} if it.get("kernel_id") else {})}
           for it in lowered]
    return json.dumps({"format": "aicf_b200.plan/1", "name": name, "values": vals, "lowered": ops}, indent=1)


def plan_from_json(text: str) -> Tuple[str, List[ValueSpec], List[Dict[str, Any]]]:
    import json
    d = json.loads(text)
    if d.get("format") != "aicf_b200.plan/1":
        raise ValueError(f"not a plan file: format={d.get('format')!r}")
    vals = [ValueSpec(v["vid"], v["name"], tuple(v["shape"]), v["dtype"], v["role"], v["persistent"], v["zero_init"],
                      v.get("alias_of"), v.get("peer_visible", False)) for v in d["values"]]
    return d["name"], vals, d["lowered"]


class Plan:
    """A finalized execution plan. Buffers are pointer-stable for the plan's lifetime."""

    def __init__(self, name: str, values: Iterable[ValueSpec], lowered: Sequence[Dict[str, Any]],
                 bind: Optional[Dict[int, Any]] = None, attr_packer=pack_attrs):
        self._h = lib.aicf_b200_plan_create(name.encode())
        if not self._h:
            raise RuntimeError("plan_create failed")
        self.name = name
        self.values: Dict[int, ValueSpec] = {}
        self.by_name: Dict[str, int] = {}
        self.lowered = [dict(it) for it in lowered]
        self._has_exchange = any(str(it.get("op")) == "dp_adam_step" for it in self.lowered)
        self._keep: List[Any] = []
        for v in values:
            role = classify_role(v.name) if v.role is None else v.role
            zero = needs_zero_init(v.name) if v.zero_init is None else v.zero_init
            shape = (C.c_int64 * max(len(v.shape), 1))(*v.shape)
            check(lib.aicf_b200_plan_add_value(self._h, v.vid, v.name.encode(), DTYPE_CODES[v.dtype], len(v.shape),
                                               shape, role, int(v.persistent), int(zero)), "plan_add_value")
            self.values[v.vid] = v
            self.by_name[v.name] = v.vid
        for v in self.values.values():
            if v.alias_of is not None:
                check(lib.aicf_b200_plan_alias(self._h, v.vid, v.alias_of), "plan_alias")
            if v.peer_visible:
                check(lib.aicf_b200_plan_set_peer_visible(self._h, v.vid), "plan_set_peer_visible")
        for vid, t in (bind or {}).items():
            check(lib.aicf_b200_plan_bind(self._h, int(vid), int(t.data_ptr())), "plan_bind")
            self._keep.append(t)
        for it in self.lowered:
            op = str(it["op"])
            ins = [int(x) for x in it.get("inputs", [])]
            outs = [int(x) for x in it.get("outputs", [])]
            schema, payload = attr_packer(op, it.get("attrs"))
            kid = it.get("kernel_id")
            check(lib.aicf_b200_plan_add_op(
                self._h, op.encode(), kid.encode() if kid else None,
                (C.c_int * max(len(ins), 1))(*ins), len(ins), (C.c_int * max(len(outs), 1))(*outs), len(outs),
                schema, payload if payload else None, len(payload)), "plan_add_op")
        check(lib.aicf_b200_plan_finalize(self._h), "plan_finalize")
        self._captured = False

    # ---- buffers -------------------------------------------------------------------------------
    def vid(self, key) -> int:
        return self.by_name[key] if isinstance(key, str) else int(key)

    def tensor(self, key) -> Tensor:
        """Non-owning view of a value's device buffer (valid while the plan lives)."""
        vid = self.vid(key)
        spec = self.values[vid]
        ptr = lib.aicf_b200_plan_value_ptr(self._h, vid)
        if not ptr:
            raise KeyError(f"value {key!r} has no buffer")
        t = Tensor(spec.shape, spec.dtype, ptr=ptr)
        t._base = self
        return t

    def state_names(self) -> List[str]:
        """Values that carry training state across steps: parameters, optimizer state, working copies."""
        out = []
        for v in self.values.values():
            role = classify_role(v.name) if v.role is None else v.role
            if v.alias_of is None and (role == ROLE_PARAM or v.name.startswith("opt.") or v.name.endswith(".lp")):
                out.append(v.name)
        return out

    def state_dict(self) -> Dict[str, Any]:
        """Host copies of the training state (numpy arrays; bf16 as uint16 bit patterns), e.g. for np.savez."""
        return {n: self.tensor(n).numpy() for n in self.state_names()}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        for n in self.state_names():
            if n not in state:
                raise KeyError(f"state is missing {n!r}")
            self.tensor(n).copy_from_host(state[n])

    def memory_map(self) -> List[Dict[str, Any]]:
        """Where every value lives: bytes, and either its offset in the shared arena or None for a buffer of its own.
        This is the arena layout of the compiled plan: values with disjoint live ranges share offsets. (`arena_bytes`
        is the whole static footprint, the shared arena plus the statics that own their buffers.)"""
        out = []
        for vid, v in sorted(self.values.items()):
            off = int(lib.aicf_b200_plan_value_arena_offset(self._h, vid))
            out.append({"vid": vid, "name": v.name, "bytes": int(lib.aicf_b200_plan_value_bytes(self._h, vid)),
                        "arena_offset": off if off >= 0 else None})
        return out

    def to_json(self) -> str:
        """plan_to_json of this plan plus its memory layout (`arena_bytes`, `arena_bytes_no_reuse`, `memory_map`)."""
        import json
        d = json.loads(plan_to_json(self.name, self.values.values(), self.lowered))
        d["arena_bytes"] = self.arena_bytes
        d["arena_bytes_no_reuse"] = self.arena_bytes_no_reuse
        d["memory_map"] = self.memory_map()
        return json.dumps(d, indent=1)

    @property
    def arena_bytes(self) -> int:
        return int(lib.aicf_b200_plan_arena_bytes(self._h))

    @property
    def arena_bytes_no_reuse(self) -> int:
        return int(lib.aicf_b200_plan_arena_bytes_no_reuse(self._h))

    @property
    def stream(self) -> int:
        return int(lib.aicf_b200_plan_stream(self._h))

    def kernel_ids(self) -> List[str]:
        return [lib.aicf_b200_plan_op_kernel_id(self._h, i).decode() for i in range(lib.aicf_b200_plan_num_ops(self._h))]

    # ---- data-parallel peer memory ---------------------------------------------------------------------
    def peer_handle(self) -> bytes:
        """64-byte IPC handle of this plan's peer-visible pool (all zero when there is none)."""
        buf = (C.c_uint8 * 64)()
        n = C.c_size_t(0)
        check(lib.aicf_b200_plan_peer_handle(self._h, buf, C.byref(n)), "plan_peer_handle")
        return bytes(buf)

    def open_peers(self, rank: int, world: int, handles: Sequence[bytes]) -> None:
        """Maps the other ranks' pools; `handles[k]` is rank k's peer_handle()."""
        blob = b"".join(bytes(h) for h in handles)
        if len(blob) != 64 * world:
            raise ValueError("need one 64-byte handle per rank")
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        check(lib.aicf_b200_plan_open_peers(self._h, int(rank), int(world), buf), "plan_open_peers")

    @property
    def peer_pool_bytes(self) -> int:
        return int(lib.aicf_b200_plan_peer_pool_bytes(self._h))

    def peer_pool_base(self, rank: int) -> int:
        """Device address of rank `rank`'s pool as mapped into this process (0 if not mapped)."""
        return int(lib.aicf_b200_plan_peer_pool_base(self._h, int(rank)) or 0)

    def open_peers_raw(self, rank: int, world: int, bases: Sequence[int]) -> None:
        """Like open_peers, from device addresses of the other ranks' pools (bases[rank] is ignored)."""
        arr = (C.c_void_p * world)(*[C.c_void_p(int(b)) for b in bases])
        check(lib.aicf_b200_plan_open_peers_raw(self._h, int(rank), int(world), arr), "plan_open_peers_raw")

    # ---- execution (names follow PlannedExecutor) --------------------------------------------------
    def run(self, stream: int = 0) -> None:
        """Eager step: one launch per lowered op on the plan's stream (or `stream`)."""
        check(lib.aicf_b200_plan_run(self._h, int(stream)), "plan_run")

    def capture(self) -> None:
        check(lib.aicf_b200_plan_capture(self._h), "plan_capture")
        self._captured = True

    def replay(self, n: int = 1, stream: int = 0) -> None:
        """n launches of the captured graph into the plan's stream (or `stream`), without synchronising."""
        if n <= 0:
            return
        if not self._captured:
            raise RuntimeError("[exec] replay called before capture()")
        check(lib.aicf_b200_plan_replay_on(self._h, int(n), int(stream)), "plan_replay")

    def reset_graph(self) -> None:
        check(lib.aicf_b200_plan_reset_graph(self._h), "plan_reset_graph")
        self._captured = False

    def sync(self) -> None:
        """Waits for everything the plan has enqueued. For a plan with dp_adam_step ops it then reads the wait-status
        word and raises if a cross-GPU wait of the exchange expired: some rank skipped an update, the replicas can
        no longer be assumed equal, and the model and optimizer state must be restored from a checkpoint. The word
        is left set (clear it with `_C.wait_status(clear=True)`)."""
        check(lib.aicf_b200_plan_sync(self._h), "plan_sync")
        if self._has_exchange:
            st = int(lib.aicf_b200_wait_status(0))
            if st > 0 and (st >> 17) & 3:
                raise RuntimeError(f"[plan {self.name}] a bounded wait of the data-parallel exchange expired "
                                   f"(phase {(st >> 17) & 3}: 1 = waiting for gradients, 2 = waiting for completion); "
                                   "replicas may have diverged: restore parameters and optimizer state from a checkpoint")

    @property
    def graph_nodes(self) -> int:
        return int(lib.aicf_b200_plan_graph_nodes(self._h))

    @property
    def graph_kernel_nodes(self) -> int:
        return int(lib.aicf_b200_plan_graph_kernel_nodes(self._h))

    def profile(self) -> List[float]:
        """One eager step with an event pair around every op; returns milliseconds per lowered op."""
        n = len(self.lowered)
        buf = (C.c_float * max(n, 1))()
        check(lib.aicf_b200_plan_profile(self._h, buf, n), "plan_profile")
        return [float(buf[i]) for i in range(n)]

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.aicf_b200_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
