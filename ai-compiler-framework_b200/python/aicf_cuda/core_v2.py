"""Tracing front end, lowering stages and executor with the reference's `core_v2` names, without torch.

What each part stands in for (reference paths are relative to its python/aicf_fw/core_v2 directory):

  IRValue / IRNode / IRGraph          ir.py (value table keyed by id, node list in emission order)
  tracing / is_tracing / get_ir       trace.py:16-85 (one active graph, values created on first use)
  SymTensor / sym_tensor / the ops    ops.py (meta-only tensors; every op only emits a node)
  trace_ir                            compile.py:9-13
  lower_to_backend_ops   (stage A)    lower.py:24-147
  apply_kernel_selection              kernel_select.py:25-142 (dtype-based kernel ids)
  apply_kernel_decisions_stageB       plan.py:371-441 (shape-based vec2 / half2 upgrades)
  stageC_fuse_gemm_epilogue           rewrites/stageC_fuse_epilogue.py:6-76
  apply_opt_rules                     opt_rules.py:34-118
  build_binding_plan / BindingPlan    plan.py:20-140
  dump_ir / dump_lowered / dump_plan  printer.py
  PlannedExecutor / ExecOptions       exec.py:37-497

Differences: dtypes may be given as 'f16' / 'f32' / 'bf16' strings, NumPy dtypes or torch dtypes; IR values
store them the way the reference's dumps print them ('torch.float16'), so text produced by either
implementation compares equal. The executor's capture()/replay() go through the C++ plan (one CUDA graph
owned by the executor) instead of the process-global graph, and run() launches on the legacy default stream
exactly as the reference does. Operators beyond the reference's set (softmax cross-entropy, bf16) are
accepted by the same stages.
"""
from __future__ import annotations

import re
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple

# ---------------------------------------------------------------------------------------------------
# dtypes
# ---------------------------------------------------------------------------------------------------
_LONG_OF = {"f16": "torch.float16", "f32": "torch.float32", "bf16": "torch.bfloat16", "i32": "torch.int32",
            "f64": "torch.float64", "i64": "torch.int64"}
_SHORT_OF_SUBSTR = (("bfloat16", "bf16"), ("float16", "f16"), ("half", "f16"), ("float32", "f32"), ("float64", "f64"),
                    ("int32", "i32"), ("int64", "i64"))


def short_dtype(dtype: Any) -> str:
    """'f16' / 'bf16' / 'f32' / 'i32' ... from a short name, a 'torch.float16'-style string, a NumPy or a torch dtype."""
    if isinstance(dtype, str) and dtype in _LONG_OF:
        return dtype
    low = str(dtype).lower()
    for sub, short in _SHORT_OF_SUBSTR:
        if sub in low:
            return short
    if low == "float":
        return "f32"
    raise ValueError(f"unsupported dtype {dtype!r}")


def long_dtype(dtype: Any) -> str:
    return _LONG_OF[short_dtype(dtype)]


# ---------------------------------------------------------------------------------------------------
# IR
# ---------------------------------------------------------------------------------------------------
@dataclass
class IRValue:
    id: int
    name: str
    shape: Tuple[int, ...]
    dtype: str
    device: str


@dataclass
class IRNode:
    op: str
    inputs: List[int]
    outputs: List[int]
    attrs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class IRGraph:
    name: str = "graph"
    values: Dict[int, IRValue] = field(default_factory=dict)
    nodes: List[IRNode] = field(default_factory=list)
    _next: int = 0

    def new_value(self, *, name: str, shape: Sequence[int], dtype: Any, device: Any = "cuda:0") -> IRValue:
        v = IRValue(self._next, str(name), tuple(int(d) for d in shape), long_dtype(dtype), str(device))
        self.values[v.id] = v
        self._next += 1
        return v

    def emit(self, *, op: str, inputs: Iterable[Any], outputs: Iterable[Any], attrs: Optional[Dict[str, Any]] = None) -> IRNode:
        as_id = lambda x: int(x.id) if isinstance(x, IRValue) else int(x)
        n = IRNode(str(op), [as_id(x) for x in inputs], [as_id(x) for x in outputs], dict(attrs or {}))
        self.nodes.append(n)
        return n

    def to_dict(self) -> Dict[str, Any]:
        return {"name": self.name,
                "values": [{"id": v.id, "name": v.name, "shape": list(v.shape), "dtype": v.dtype, "device": v.device}
                           for _, v in sorted(self.values.items())],
                "nodes": [{"op": n.op, "inputs": list(n.inputs), "outputs": list(n.outputs), "attrs": dict(n.attrs)}
                          for n in self.nodes]}


# ---------------------------------------------------------------------------------------------------
# tracing state
# ---------------------------------------------------------------------------------------------------
class _TraceState:
    def __init__(self, ir: IRGraph):
        self.ir = ir
        # id(obj) -> (obj, value). The object is held so that its id cannot be reused by a later temporary
        # while the trace is open.
        self.by_obj: Dict[int, Tuple[Any, IRValue]] = {}


_STATE: Optional[_TraceState] = None


def is_tracing() -> bool:
    return _STATE is not None


def get_ir() -> IRGraph:
    if _STATE is None:
        raise RuntimeError("core_v2.trace.get_ir(): not tracing")
    return _STATE.ir


def as_ir_value_obj(obj: Any, *, name: str, shape, dtype, device) -> IRValue:
    if _STATE is None:
        raise RuntimeError("as_ir_value_obj() called outside tracing")
    hit = _STATE.by_obj.get(id(obj))
    if hit is not None:
        return hit[1]
    v = _STATE.ir.new_value(name=name, shape=shape, dtype=dtype, device=device)
    _STATE.by_obj[id(obj)] = (obj, v)
    return v


@contextmanager
def tracing(ir: IRGraph):
    global _STATE
    prev, _STATE = _STATE, _TraceState(ir)
    try:
        yield ir
    finally:
        _STATE = prev


def trace_ir(step_fn: Callable[[], None], *, name: str = "train_step") -> IRGraph:
    ir = IRGraph(name=name)
    with tracing(ir):
        step_fn()
    return ir


# ---------------------------------------------------------------------------------------------------
# symbolic tensors and ops (each op only records a node; nothing is computed while tracing)
# ---------------------------------------------------------------------------------------------------
@dataclass(eq=False)
class SymTensor:
    name: str
    shape: Tuple[int, ...]
    dtype: Any
    device: Any = "cuda:0"


def sym_tensor(*, name: str, shape: Sequence[int], dtype: Any, device: Any = "cuda:0") -> SymTensor:
    return SymTensor(str(name), tuple(int(d) for d in shape), dtype, device)


def _val(t: SymTensor, fallback: str) -> IRValue:
    return as_ir_value_obj(t, name=t.name or fallback, shape=t.shape, dtype=t.dtype, device=t.device)


def _need_trace(fn: str) -> IRGraph:
    if not is_tracing():
        raise RuntimeError(f"core_v2.ops.{fn}(): tracing-only")
    return get_ir()


def _like(t: SymTensor, name: str, shape: Optional[Sequence[int]] = None) -> SymTensor:
    return sym_tensor(name=name, shape=t.shape if shape is None else shape, dtype=t.dtype, device=t.device)


_LINEAR_LAYOUT = "y = x @ W^T + b"


def linear(x: SymTensor, W: SymTensor, b: Optional[SymTensor] = None, *, name: str = "linear_out") -> SymTensor:
    """y[B, OUT] = x[B, IN] @ W[OUT, IN]^T (+ b[OUT])."""
    ir = _need_trace("linear")
    if len(x.shape) != 2 or len(W.shape) != 2:
        raise RuntimeError(f"linear expects 2D x/W. got x={x.shape} W={W.shape}")
    if x.shape[1] != W.shape[1]:
        raise RuntimeError(f"linear shape mismatch: x={x.shape} W={W.shape} (W must be (OUT, IN))")
    ins = [_val(x, "x"), _val(W, "W")]
    if b is not None:
        ins.append(_val(b, "b"))
    y = _like(x, name, (x.shape[0], W.shape[0]))
    ir.emit(op="Linear", inputs=ins, outputs=[_val(y, name)], attrs={"bias": b is not None, "layout": _LINEAR_LAYOUT})
    return y


def relu(x: SymTensor, *, name: str = "relu_out") -> SymTensor:
    ir = _need_trace("relu")
    xv = _val(x, "x")
    y = _like(x, name)
    ir.emit(op="ReLU", inputs=[xv], outputs=[_val(y, name)], attrs={})
    return y


def save(x: SymTensor, *, name: str = "saved") -> SymTensor:
    """Copy of an activation kept for the backward pass."""
    ir = _need_trace("save")
    xv = _val(x, "x")
    y = _like(x, name)
    ir.emit(op="Save", inputs=[xv], outputs=[_val(y, name)], attrs={})
    return y


def mse_grad(pred: SymTensor, target: SymTensor, *, scale: Optional[float] = None, name: str = "mse_grad_out") -> SymTensor:
    ir = _need_trace("mse_grad")
    if tuple(pred.shape) != tuple(target.shape):
        raise RuntimeError(f"mse_grad shape mismatch: pred={pred.shape} target={target.shape}")
    ins = [_val(pred, "pred"), _val(target, "target")]
    out = _like(pred, name)
    ir.emit(op="MseGrad", inputs=ins, outputs=[_val(out, name)], attrs={} if scale is None else {"scale": float(scale)})
    return out


def linear_bwd(x: SymTensor, W: SymTensor, dY: SymTensor, *, bias: bool = True, dx_name: str = "d_x",
               dW_name: str = "d_W", db_name: str = "d_b") -> Tuple[SymTensor, SymTensor, Optional[SymTensor]]:
    """(dx[B, IN], dW[OUT, IN], db[OUT] or None) of y = x @ W^T + b given dY[B, OUT]."""
    ir = _need_trace("linear_bwd")
    if len(x.shape) != 2 or len(W.shape) != 2 or len(dY.shape) != 2:
        raise RuntimeError(f"linear_bwd expects 2D x/W/dY. got x={x.shape} W={W.shape} dY={dY.shape}")
    (B, IN), (OUT, IN2) = x.shape, W.shape
    if IN != IN2 or tuple(dY.shape) != (B, OUT):
        raise RuntimeError(f"linear_bwd shape mismatch: x={x.shape} W={W.shape} dY={dY.shape}")
    ins = [_val(x, "x"), _val(W, "W"), _val(dY, "dY")]
    dx = _like(x, dx_name, (B, IN))
    dW = _like(W, dW_name, (OUT, IN))
    outs = [_val(dx, dx_name), _val(dW, dW_name)]
    db = None
    if bias:
        db = _like(W, db_name, (OUT,))
        outs.append(_val(db, db_name))
    ir.emit(op="LinearBwd", inputs=ins, outputs=outs, attrs={"bias": bool(bias), "layout": _LINEAR_LAYOUT})
    return dx, dW, db


def relu_bwd(dY: SymTensor, saved: SymTensor, *, name: str = "d_relu_in") -> SymTensor:
    ir = _need_trace("relu_bwd")
    if tuple(dY.shape) != tuple(saved.shape):
        raise RuntimeError(f"relu_bwd shape mismatch: dY={dY.shape} saved={saved.shape}")
    ins = [_val(dY, "dY"), _val(saved, "saved")]
    out = _like(dY, name)
    ir.emit(op="ReluBwd", inputs=ins, outputs=[_val(out, name)], attrs={})
    return out


def step_inc(step_i32: SymTensor, *, name: str = "opt.step") -> SymTensor:
    ir = _need_trace("step_inc")
    if short_dtype(step_i32.dtype) not in ("i32", "i64"):
        raise RuntimeError(f"step_inc expects int32/int64 tensor, got {step_i32.dtype}")
    si = _val(step_i32, "step")
    out = _like(step_i32, name)
    ir.emit(op="StepInc", inputs=[si], outputs=[_val(out, name)], attrs={})
    return out


def bias_corr(step_i32: SymTensor, bc1_inv: SymTensor, bc2_inv: SymTensor, *, beta1: float, beta2: float,
              out1_name: str = "opt.bc1_inv_out", out2_name: str = "opt.bc2_inv_out") -> Tuple[SymTensor, SymTensor]:
    """(1 / (1 - beta1^t), 1 / (1 - beta2^t)) from the step counter; the two inputs only give shape and dtype."""
    ir = _need_trace("bias_corr")
    sv = _val(step_i32, "step")
    o1, o2 = _like(bc1_inv, out1_name), _like(bc2_inv, out2_name)
    ir.emit(op="BiasCorr", inputs=[sv], outputs=[_val(o1, out1_name), _val(o2, out2_name)],
            attrs={"beta1": float(beta1), "beta2": float(beta2)})
    return o1, o2


def adam_step(p: SymTensor, g: SymTensor, m: SymTensor, v: SymTensor, bc1_inv: SymTensor, bc2_inv: SymTensor, *,
              lr: float, beta1: float, beta2: float, eps: float) -> Tuple[SymTensor, SymTensor, SymTensor]:
    """In place on (p, m, v): the node's outputs are the same value ids as its first, third and fourth inputs."""
    ir = _need_trace("adam_step")
    pv, gv, mv, vv = _val(p, "p"), _val(g, "g"), _val(m, "m"), _val(v, "v")
    b1, b2 = _val(bc1_inv, "bc1_inv"), _val(bc2_inv, "bc2_inv")
    ir.emit(op="AdamStep", inputs=[pv, gv, mv, vv, b1, b2], outputs=[pv, mv, vv],
            attrs={"lr": float(lr), "beta1": float(beta1), "beta2": float(beta2), "eps": float(eps)})
    return p, m, v


def sgd_step(p: SymTensor, g: SymTensor, *, lr: float) -> SymTensor:
    """In place: p -= lr * g."""
    ir = _need_trace("sgd_step")
    pv, gv = _val(p, "p"), _val(g, "g")
    ir.emit(op="SgdStep", inputs=[pv, gv], outputs=[pv], attrs={"lr": float(lr)})
    return p


def softmax_ce_grad(logits: SymTensor, labels: SymTensor, *, scale: Optional[float] = None, loss_name: str = "loss",
                    name: str = "dY") -> Tuple[SymTensor, SymTensor]:
    """(per-row loss[B] f32, dlogits[B, C]) of softmax cross-entropy with int32 labels[B]. Not in the reference's
    op set; lowers to this backend's fused softmax_ce kernel."""
    ir = _need_trace("softmax_ce_grad")
    if len(logits.shape) != 2 or tuple(labels.shape) != (logits.shape[0],):
        raise RuntimeError(f"softmax_ce_grad shape mismatch: logits={logits.shape} labels={labels.shape}")
    ins = [_val(logits, "logits"), _val(labels, "labels")]
    loss = sym_tensor(name=loss_name, shape=(logits.shape[0],), dtype="f32", device=logits.device)
    d = _like(logits, name)
    ir.emit(op="SoftmaxCE", inputs=ins, outputs=[_val(loss, loss_name), _val(d, name)],
            attrs={} if scale is None else {"scale": float(scale)})
    return loss, d


# ---------------------------------------------------------------------------------------------------
# stage A: IR -> primitive backend ops (semantics only; no kernel ids)
# ---------------------------------------------------------------------------------------------------
LoweredOp = Dict[str, Any]

# IR op names are matched case-insensitively; CamelCase names without a separator map to these primitives.
_IR_ALIASES = {"adamstep": "adam_step", "stepinc": "step_inc", "biascorr": "bias_corr", "msegrad": "mse_grad",
               "relubwd": "relu_bwd", "linearbwd": "linear_bwd", "sgdstep": "sgd_step", "softmaxce": "softmax_ce"}
_PASS_THROUGH = frozenset((
    "gemm", "bias_add", "add", "relu", "reduce_sum", "mse_grad", "relu_bwd", "copy", "copy_saved", "copy_aux", "grad_zero",
    "adam_step", "step_inc", "bias_corr", "layernorm_fwd", "layernorm_bwd", "batchnorm_fwd", "batchnorm_bwd", "sgd_step",
    # this backend's additions
    "gemm_epilogue", "gemm_relu_bwd", "softmax", "softmax_ce", "reduce_max", "reduce_mean", "cast", "all_reduce", "dp_adam_step"))


def _item(op: str, inputs: Sequence[int], outputs: Sequence[int], attrs: Optional[Dict[str, Any]] = None) -> LoweredOp:
    return {"op": op, "inputs": [int(v) for v in inputs], "outputs": [int(v) for v in outputs], "attrs": dict(attrs or {})}


def _lower_linear(ins, outs, attrs) -> List[LoweredOp]:
    # y = x @ W^T is gemm{transB}; the bias is added in place on y.
    y = outs[0]
    ops = [_item("gemm", ins[:2], [y], {"transB": True})]
    if attrs.get("bias", False) and len(ins) >= 3:
        ops.append(_item("bias_add", [y, ins[2]], [y]))
    return ops


def _lower_linear_bwd(ins, outs, attrs) -> List[LoweredOp]:
    x, w, dy = ins[:3]
    ops = [_item("gemm", [dy, w], [outs[0]], {"transA": False, "transB": False}),       # dx = dY @ W
           _item("gemm", [dy, x], [outs[1]], {"transA": True, "transB": False})]        # dW = dY^T @ x
    if attrs.get("bias", False) and len(outs) >= 3:
        ops.append(_item("reduce_sum", [dy], [outs[2]], {"axis": 0, "keepdim": False}))  # db = column sums of dY
    return ops


_EXPANDERS: Dict[str, Callable[[List[int], List[int], Dict[str, Any]], List[LoweredOp]]] = {
    "linear": _lower_linear,
    "linear_bwd": _lower_linear_bwd,
    "save": lambda ins, outs, attrs: [_item("copy_saved", ins[:1], outs[:1])],
    "relu": lambda ins, outs, attrs: [_item("relu", ins[:1], outs[:1])],
    "relu_bwd": lambda ins, outs, attrs: [_item("relu_bwd", ins[:2], outs[:1])],
    "mse_grad": lambda ins, outs, attrs: [_item("mse_grad", ins[:2], outs[:1], attrs)],
    "sgd_step": lambda ins, outs, attrs: [_item("sgd_step", ins[:2], outs[:1], attrs)],
}


def lower_to_backend_ops(ir: IRGraph) -> List[LoweredOp]:
    """Stage A. One IR node becomes one or more primitive ops over the same value ids."""
    lowered: List[LoweredOp] = []
    for n in ir.nodes:
        ir_op = str(getattr(n, "op", getattr(n, "kind", ""))).strip()
        op = _IR_ALIASES.get(ir_op.lower(), ir_op.lower())
        ins, outs, attrs = [int(v) for v in n.inputs], [int(v) for v in n.outputs], dict(n.attrs or {})
        expand = _EXPANDERS.get(op)
        if expand is not None:
            lowered.extend(expand(ins, outs, attrs))
        elif op in _PASS_THROUGH:
            lowered.append(_item(op, ins, outs, attrs))
        else:
            raise RuntimeError(f"[lower] unsupported IR op '{ir_op}' (normalized='{op}')")
    return lowered


# ---------------------------------------------------------------------------------------------------
# kernel ids: dtype-based selection, then shape-based upgrades (stage B)
# ---------------------------------------------------------------------------------------------------
def _vdtype(ir: IRGraph, vid: int) -> str:
    return short_dtype(ir.values[int(vid)].dtype)


def _numel(ir: IRGraph, vid: int) -> int:
    n = 1
    for d in ir.values[int(vid)].shape:
        n *= int(d)
    return n


def _last_dim(ir: IRGraph, vid: int) -> int:
    shape = ir.values[int(vid)].shape
    return int(shape[-1]) if shape else 1


# op -> (id when the first input or output is f16, id otherwise); the reference's naming.
_BY_DTYPE = {
    "gemm": ("gemm_f16_tc_wmma_out_f16_v0", "gemm_f32_naive_v0"),
    "gemm_epilogue": ("gemm_bias_relu_f16_tc_wmma_out_f16_v0", "gemm_bias_relu_f32_naive_v0"),
    "bias_add": ("bias_add_f16_v0", "bias_add_f32_v0"),
    "add": ("add_f16_v0", "add_f32_v0"),
    "relu": ("relu_f16_v0", "relu_f32_v0"),
    "mse_grad": ("mse_grad_f16_v0", "mse_grad_f32_v0"),
    "relu_bwd": ("relu_bwd_f16_v0", "relu_bwd_f32_v0"),
    "sgd_step": ("sgd_step_f16_v0", "sgd_step_f32_v0"),
    "copy": ("copy_f16_v0", "copy_f32_v0"),
    "copy_saved": ("copy_f16_v0", "copy_f32_v0"),
    "copy_aux": ("copy_f16_v0", "copy_f32_v0"),
    "layernorm_fwd": ("layernorm_fwd_f16_v0", "layernorm_fwd_f32_v0"),
    "layernorm_bwd": ("layernorm_bwd_f16_v0", "layernorm_bwd_f32_v0"),
    "batchnorm_fwd": ("batchnorm_fwd_f16_v0", "batchnorm_fwd_f16_v0"),
    "batchnorm_bwd": ("batchnorm_bwd_f16_v0", "batchnorm_bwd_f16_v0"),
    "grad_zero": ("grad_zero_v0", "grad_zero_v0"),
    "adam_step": ("adam_step_f32_v0", "adam_step_f32_v0"),
    "step_inc": ("step_inc_v0", "step_inc_v0"),
    "bias_corr": ("bias_corr_v0", "bias_corr_v0"),
}


def pick_kernel_id(op: str, in_dtypes: Sequence[str], out_dtypes: Sequence[str], attrs: Dict[str, Any]) -> Optional[str]:
    """Kernel id for a primitive from the dtypes of its first input and first output, or None when the
    choice is left to priority dispatch (bf16 and this backend's added ops have no pinned id)."""
    op = str(op).strip().lower()
    in0 = short_dtype(in_dtypes[0]) if in_dtypes else ""
    out0 = short_dtype(out_dtypes[0]) if out_dtypes else ""
    if "bf16" in (in0, out0):
        return None
    f16 = "f16" in (in0, out0)
    if op == "gemm_epilogue":
        if "epilogue" in attrs and str(attrs["epilogue"]).strip().lower() not in ("bias_relu", "bias+relu", "biasrelu"):
            return None
    if op == "reduce_sum":
        if out0 == "f16":
            return "reduce_sum_keep_lastdim_f16_v0"
        return "reduce_sum_keep_lastdim_f16_to_f32_v0" if in0 == "f16" else "reduce_sum_keep_lastdim_f32_v0"
    pair = _BY_DTYPE.get(op)
    return None if pair is None else pair[0 if f16 else 1]


def apply_kernel_selection(ir: IRGraph, lowered: Sequence[LoweredOp], *, overwrite: bool = True) -> List[LoweredOp]:
    """Attach a dtype-based kernel id to every op that has one. overwrite=False keeps ids already present."""
    out: List[LoweredOp] = []
    for it in lowered:
        new = dict(it)
        if overwrite or new.get("kernel_id") is None:
            kid = pick_kernel_id(str(it.get("op", "")), [ir.values[int(v)].dtype for v in it.get("inputs", [])],
                                 [ir.values[int(v)].dtype for v in it.get("outputs", [])], dict(it.get("attrs") or {}))
            if kid is not None:
                new["kernel_id"] = kid
        out.append(new)
    return out


_VEC2_BY_LASTDIM = {"add": "add_f16_vec2_v0", "bias_add": "bias_add_f16_vec2_v0", "relu": "relu_f16_vec2_v0",
                    "relu_bwd": "relu_bwd_f16_vec2_v0"}


def apply_kernel_decisions_stageB(ir: IRGraph, lowered: Sequence[LoweredOp]) -> List[LoweredOp]:
    """Stage B: shape-based decisions for f16 ops. Element-wise ops take the two-wide kernel when the last
    dimension of their output is even; sgd_step takes it when the parameter's element count is even. Other
    ops keep whatever id they carry (possibly none)."""
    out: List[LoweredOp] = []
    for it in lowered:
        new = dict(it)
        op = str(it.get("op", "")).strip().lower()
        ins, outs = list(it.get("inputs", [])), list(it.get("outputs", []))
        f16 = bool(ins and _vdtype(ir, ins[0]) == "f16") or bool(outs and _vdtype(ir, outs[0]) == "f16")
        ref = outs[0] if outs else (ins[0] if ins else None)
        if f16 and ref is not None:
            if op in _VEC2_BY_LASTDIM and _last_dim(ir, ref) % 2 == 0:
                new["kernel_id"] = _VEC2_BY_LASTDIM[op]
            elif op == "sgd_step" and outs and _numel(ir, outs[0]) % 2 == 0:
                new["kernel_id"] = "sgd_step_f16_half2_v0"
        out.append(new)
    return out


# ---------------------------------------------------------------------------------------------------
# stage C: gemm (+ in-place bias_add) + relu -> gemm_epilogue
# ---------------------------------------------------------------------------------------------------
def _opname(it: LoweredOp) -> str:
    return str(it.get("op", it.get("kind", ""))).strip().lower()


def _match_epilogue_chain(lowered: Sequence[LoweredOp], i: int, *, bias_required: bool):
    """If lowered[i] is a gemm whose single output y feeds an adjacent in-place bias_add(y, b) -> y (optional
    unless bias_required) and then relu(y) -> z, returns (ops consumed, bias vid or None, z); else None."""
    g = lowered[i]
    if _opname(g) != "gemm" or len(g.get("outputs", [])) != 1:
        return None
    y = int(g["outputs"][0])
    j, bias = i + 1, None
    if j < len(lowered) and _opname(lowered[j]) == "bias_add":
        b_in, b_out = lowered[j].get("inputs", []), lowered[j].get("outputs", [])
        if len(b_in) == 2 and len(b_out) == 1 and int(b_in[0]) == y and int(b_out[0]) == y:
            bias, j = int(b_in[1]), j + 1
    if bias is None and bias_required:
        return None
    if j >= len(lowered) or _opname(lowered[j]) != "relu":
        return None
    r_in, r_out = lowered[j].get("inputs", []), lowered[j].get("outputs", [])
    if len(r_in) != 1 or len(r_out) != 1 or int(r_in[0]) != y:
        return None
    return j + 1 - i, bias, int(r_out[0])


def stageC_fuse_gemm_epilogue(ir: Optional[IRGraph], lowered: Sequence[LoweredOp]) -> List[LoweredOp]:
    """Adjacent gemm -> [bias_add in place] -> relu becomes one gemm_epilogue(x, W[, b]) -> relu's output, carrying the
    gemm's attrs plus epilogue_act='relu' and epilogue_bias. The fused op has no kernel id (a later selection fills it)."""
    out: List[LoweredOp] = []
    i = 0
    while i < len(lowered):
        m = _match_epilogue_chain(lowered, i, bias_required=False)
        if m is None:
            out.append(lowered[i])
            i += 1
            continue
        consumed, bias, z = m
        g = lowered[i]
        attrs = dict(g.get("attrs") or {})
        attrs["epilogue_act"] = "relu"
        attrs["epilogue_bias"] = bias is not None
        out.append({"op": "gemm_epilogue", "inputs": [int(v) for v in g["inputs"]] + ([bias] if bias is not None else []),
                    "outputs": [z], "attrs": attrs})
        i += consumed
    return out


def apply_opt_rules(ir: Optional[IRGraph], lowered: Sequence[LoweredOp]) -> List[LoweredOp]:
    """The older spelling of the same fusion: the bias is mandatory, the gemm must have exactly two inputs, and the fused
    op is tagged epilogue='bias_relu'. Every item is normalised (lower-case op, int ids, attrs dict, extra keys kept)."""
    norm = [{**{k: v for k, v in it.items() if k not in ("op", "inputs", "outputs", "attrs")}, "op": _opname(it),
             "inputs": [int(v) for v in it.get("inputs", [])], "outputs": [int(v) for v in it.get("outputs", [])],
             "attrs": dict(it.get("attrs") or {})} for it in lowered]
    out: List[LoweredOp] = []
    i = 0
    while i < len(norm):
        m = _match_epilogue_chain(norm, i, bias_required=True) if len(norm[i]["inputs"]) == 2 else None
        if m is None:
            out.append(norm[i])
            i += 1
            continue
        consumed, bias, z = m
        out.append({"op": "gemm_epilogue", "inputs": norm[i]["inputs"] + [bias], "outputs": [z],
                    "attrs": {**norm[i]["attrs"], "epilogue": "bias_relu"}})
        i += consumed
    return out


def elide_saved_copies(ir: Optional[IRGraph], lowered: Sequence[LoweredOp]) -> List[LoweredOp]:
    """Drops every `copy_saved (src) -> (saved)` whose source is not written again before the last read of `saved`,
    and lets those reads use `src` directly. In the reference's lowering the activation saved for relu_bwd is a
    second full-size copy of a value that stays alive and unchanged until the backward pass
    (README_stage6.md:340-359 lists this as pending work); the copy is one read and one write of the activation per
    hidden layer. Not part of compile_lowered(): the reference's lowered list keeps the copies."""
    out: List[LoweredOp] = [dict(it) for it in lowered]
    remap: Dict[int, int] = {}
    keep = [True] * len(out)
    for i, it in enumerate(out):
        if _opname(it) != "copy_saved" or len(it.get("inputs", [])) != 1 or len(it.get("outputs", [])) != 1:
            continue
        src, saved = int(it["inputs"][0]), int(it["outputs"][0])
        if src == saved:
            continue
        readers = [j for j in range(i + 1, len(out)) if saved in [int(v) for v in out[j].get("inputs", [])]]
        last_read = max(readers) if readers else i
        rewritten = any(src in [int(v) for v in out[j].get("outputs", [])] or saved in [int(v) for v in out[j].get("outputs", [])]
                        for j in range(i + 1, last_read + 1))
        if rewritten:
            continue
        keep[i] = False
        remap[saved] = src
    result: List[LoweredOp] = []
    for flag, it in zip(keep, out):
        if not flag:
            continue
        it["inputs"] = [remap.get(int(v), int(v)) for v in it.get("inputs", [])]
        result.append(it)
    return result


def compile_lowered(ir: IRGraph, *, fuse: bool = True, pin_kernel_ids: bool = True) -> List[LoweredOp]:
    """The stages in the order the reference's end-to-end test runs them: A, B, C, then dtype-based ids for
    every op that is still without one."""
    lowered = lower_to_backend_ops(ir)
    if pin_kernel_ids:
        lowered = apply_kernel_decisions_stageB(ir, lowered)
    if fuse:
        lowered = stageC_fuse_gemm_epilogue(ir, lowered)
    if pin_kernel_ids:
        lowered = apply_kernel_selection(ir, lowered, overwrite=False)
    return lowered


# ---------------------------------------------------------------------------------------------------
# binding plan: which values the caller provides and which the runtime owns
# ---------------------------------------------------------------------------------------------------
ROLE_INPUT = "input"
ROLE_PARAM = "param"
ROLE_STATIC = "static"


@dataclass
class BindSpec:
    vid: int
    role: str
    name: str
    shape: Tuple[int, ...]
    dtype: str
    device: str


@dataclass
class BindingPlan:
    name: str
    specs: Dict[int, BindSpec] = field(default_factory=dict)
    inputs: List[int] = field(default_factory=list)
    params: List[int] = field(default_factory=list)
    statics: List[int] = field(default_factory=list)

    def role_of(self, vid: int) -> str:
        s = self.specs.get(int(vid))
        return s.role if s is not None else "unknown"


@dataclass
class PlanOptions:
    input_names: Set[str] = field(default_factory=lambda: {"x", "t"})
    param_regex: str = r"^\d+\.(W|b)$"                               # model parameters only: '0.W', '2.b', ...
    static_prefixes: Tuple[str, ...] = ("d_", "grad", "dY", "opt.")  # gradients and optimizer state are runtime-owned


def build_binding_plan(ir: IRGraph, *, opts: Optional[PlanOptions] = None) -> BindingPlan:
    """Role of every IR value from its name: the input names first, then the forced-static prefixes, then the parameter
    pattern; everything else is static. The three id lists are in ascending id order."""
    opts = opts or PlanOptions()
    param_re = re.compile(opts.param_regex)
    plan = BindingPlan(name=f"{ir.name}:binding_plan")
    for vid in sorted(ir.values):
        v = ir.values[vid]
        nm = str(v.name)
        if nm in opts.input_names:
            role = ROLE_INPUT
        elif any(nm.startswith(p) for p in opts.static_prefixes):
            role = ROLE_STATIC
        elif param_re.match(nm):
            role = ROLE_PARAM
        else:
            role = ROLE_STATIC
        plan.specs[int(vid)] = BindSpec(int(vid), role, nm, tuple(v.shape), str(v.dtype), str(v.device))
        {ROLE_INPUT: plan.inputs, ROLE_PARAM: plan.params, ROLE_STATIC: plan.statics}[role].append(int(vid))
    return plan


# ---------------------------------------------------------------------------------------------------
# text dumps (line formats equal to the reference's printer, so dumps can be diffed across implementations)
# ---------------------------------------------------------------------------------------------------
def _shape_s(shape: Sequence[int]) -> str:
    return str(tuple(int(d) for d in shape))


def dump_ir(ir: IRGraph) -> str:
    def attrs_s(attrs: Dict[str, Any]) -> str:
        if not attrs:
            return ""
        return "  {" + ", ".join(f"{k}={v:.6g}" if isinstance(v, float) else f"{k}={v}" for k, v in attrs.items()) + "}"

    ids = lambda vs: ", ".join(f"v{int(v):03d}" for v in vs)
    lines = [f"=== IRGraph: {ir.name} ===", f"values: {len(ir.values)}, nodes: {len(ir.nodes)}", "", "[values]"]
    for vid in sorted(ir.values):
        v = ir.values[vid]
        lines.append(f"  v{int(v.id):03d}  {str(v.name):12s} shape={_shape_s(v.shape)} dtype={v.dtype} device={v.device}")
    lines += ["", "[nodes]"]
    for i, n in enumerate(ir.nodes):
        lines.append(f"  #{i:03d} {str(n.op):10s} ({ids(n.inputs)}) -> ({ids(n.outputs)}){attrs_s(n.attrs or {})}")
    return "\n".join(lines)


def dump_lowered(lowered: Sequence[LoweredOp], name: str = "lowered") -> str:
    lines = [f"=== LoweredOps({name}) ===", f"ops: {len(lowered)}\n"]
    for i, it in enumerate(lowered):
        kind = it.get("kind") or it.get("op") or it.get("op_kind") or "unknown"
        ins = ", ".join(str(v) for v in it.get("inputs") or [])
        outs = ", ".join(str(v) for v in it.get("outputs") or [])
        attrs = it.get("attrs") or {}
        line = f"  #{i:03d} {kind:<10} ({ins}) -> ({outs})"
        if attrs:
            line += "  {" + ", ".join(f"{k}={attrs[k]}" for k in sorted(attrs)) + "}"
        if it.get("kernel_id") is not None:
            line += f"  kid={it['kernel_id']}"
        lines.append(line)
    return "\n".join(lines)


def dump_plan(plan: BindingPlan, *, title: str = "BindingPlan", name: Optional[str] = None) -> str:
    lines = [f"=== {title}({name}) ===" if name else f"=== {title} ===", f"name: {plan.name}",
             f"inputs: {len(plan.inputs)}, params: {len(plan.params)}, statics: {len(plan.statics)}", ""]
    for header, vids in (("inputs", plan.inputs), ("params", plan.params), ("statics", plan.statics)):
        lines.append(f"[{header}]")
        for vid in vids:
            s = plan.specs[int(vid)]
            lines.append(f"  v{s.vid:03d}  {s.name:12s} role={s.role:6s} shape={_shape_s(s.shape)} dtype={s.dtype} device={s.device}")
        lines.append("")
    return "\n".join(lines)


# ---------------------------------------------------------------------------------------------------
# executor
# ---------------------------------------------------------------------------------------------------
@dataclass
class ExecOptions:
    debug: bool = False
    debug_limit: int = 50
    check_shapes: bool = True
    check_device: bool = True   # accepted for compatibility; device placement is the caller's contract here
    check_dtype: bool = True
    require_kernel_id: bool = False  # True: an op without kernel_id is an error (no priority dispatch at run time)


_OP_KIND_NAMES = {
    "add": "EltwiseAdd", "relu": "EltwiseRelu", "gemm": "Gemm", "bias_add": "BiasAdd", "reduce_sum": "ReduceSum",
    "mse_grad": "MseGrad", "relu_bwd": "ReluBwd", "sgd_step": "SgdStep", "copy": "Copy", "copy_saved": "Copy",
    "copy_aux": "Copy", "grad_zero": "GradZero", "adam_step": "AdamStep", "step_inc": "StepInc", "bias_corr": "BiasCorr",
    "layernorm_fwd": "LayerNormFwd", "layernorm_bwd": "LayerNormBwd", "batchnorm_fwd": "BatchNormFwd",
    "batchnorm_bwd": "BatchNormBwd", "gemm_epilogue": "GemmEpilogue",
    "softmax": "Softmax", "softmax_ce": "SoftmaxCE", "reduce_max": "ReduceMax", "reduce_mean": "ReduceMean",
    "all_reduce": "AllReduce", "cast": "Cast", "gemm_relu_bwd": "GemmReluBwd", "dp_adam_step": "DpAdamStep",
}


def opkind_from_name(op: str) -> int:
    from . import _C
    k = str(op).strip().lower()
    if k not in _OP_KIND_NAMES:
        raise RuntimeError(f"[exec] unsupported lowered op '{op}' (no OpKind mapping)")
    return int(getattr(_C.OpKind, _OP_KIND_NAMES[k]))


def _canon_name(s: str) -> str:
    return re.sub(r"[^0-9a-z]+", "_", str(s).strip().lower()).strip("_")


class PlannedExecutor:
    """Runs a lowered-op list over a binding plan.

    run() launches the ops one by one on the legacy default stream through `_C.launch_by_id` (or `_C.op_call` for
    ops without a kernel id), so the op trace records them as the reference's executor does. capture() builds one
    CUDA graph of the whole list in the C++ plan and replay(n) launches it n times with no per-op host work.
    Inputs and parameters are used in place (their device pointers are bound into the plan); statics live in the
    plan's arena, zero-filled for 'opt.step*', 'opt.m.*' and 'opt.v.*', and are returned as `aicf_cuda.Tensor` views.
    Calling run()/capture() again with tensors at other addresses rebuilds the plan (statics start afresh) and
    drops a captured graph.

    AICF_WARMUP=1 in the environment (read at every run()/capture(), like the reference's executor,
    python/aicf_fw/core_v2/exec.py:396,422-431) makes a step that leaves the model where it is, so that gradients
    of a first step can be inspected before any weight moves: `step_inc` becomes a copy of its input to its output
    (the counter does not advance) and every `adam_step` runs with lr = 0 (moments are still updated, as there).
    """

    def __init__(self, *, ir: IRGraph, lowered: Sequence[LoweredOp], plan: BindingPlan, device: Any = None,
                 opts: Optional[ExecOptions] = None):
        self.ir = ir
        self.lowered = [dict(it) for it in lowered]
        self.plan = plan
        self.device = device
        self.opts = opts or ExecOptions()
        self.env: Dict[int, Any] = {}
        self._captured = False
        self._cplan = None
        self._bound_ptrs: Dict[int, int] = {}
        self._plan_is_warmup = False
        if self.opts.require_kernel_id:
            for i, it in enumerate(self.lowered):
                if it.get("kernel_id") is None:
                    raise RuntimeError(f"[exec] require_kernel_id=True but lowered op #{i} '{it.get('op')}' has no kernel_id. "
                                       "This means decisions are still happening at runtime (op_call/dispatch).")

    # ---- trace ---------------------------------------------------------------------------------
    def trace_enable(self, flag: bool = True) -> None:
        from . import _C
        _C.trace_enable(bool(flag))

    def trace_reset(self) -> None:
        from . import _C
        _C.trace_reset()

    def trace_get(self) -> List[str]:
        from . import _C
        return list(_C.trace_get())

    # ---- binding -------------------------------------------------------------------------------
    def _resolve(self, key: str, kind: str) -> int:
        exact = [s.vid for s in self.plan.specs.values() if s.name == key]
        cands = exact or [s.vid for s in self.plan.specs.values() if _canon_name(s.name) == _canon_name(key)]
        same_role = [v for v in cands if self.plan.specs[v].role == kind]
        pick = same_role or cands
        if len(pick) != 1:
            known = [s.name for s in self.plan.specs.values()]
            more = "" if len(known) <= 24 else f" ...(+{len(known) - 24})"
            raise KeyError(f"[plan] unknown or ambiguous {kind} name='{key}'. candidates={cands}. known={known[:24]}{more}")
        return pick[0]

    def _check(self, spec: BindSpec, t: Any) -> None:
        if self.opts.check_shapes and tuple(int(d) for d in t.shape) != tuple(spec.shape):
            raise RuntimeError(f"[plan] shape mismatch for '{spec.name}': expected {tuple(spec.shape)}, got {tuple(t.shape)}")
        if self.opts.check_dtype and short_dtype(t.dtype) != short_dtype(spec.dtype):
            raise RuntimeError(f"[plan] dtype mismatch for '{spec.name}': expected {spec.dtype}, got {t.dtype}")
        contiguous = getattr(t, "is_contiguous", None)
        if callable(contiguous) and not contiguous():
            raise RuntimeError(f"[plan] '{spec.name}' must be contiguous")

    @staticmethod
    def _warmup_requested() -> bool:
        import os
        return os.getenv("AICF_WARMUP", "0") == "1"

    def _effective_lowered(self, warmup: bool) -> List[Dict[str, Any]]:
        """The lowered list as it is launched: unchanged, or the warm-up form (see the class docstring)."""
        if not warmup:
            return self.lowered
        out = []
        for it in self.lowered:
            op = str(it["op"])
            if op == "step_inc":
                src, dst = list(it.get("inputs", [])), list(it.get("outputs", []))
                if src and dst and int(src[0]) != int(dst[0]):
                    out.append({"op": "copy", "inputs": src[:1], "outputs": dst[:1], "attrs": {}, "kernel_id": "copy_i32_v0"})
                continue  # in place: copying a counter onto itself is nothing
            if op == "adam_step":
                it = dict(it, attrs=dict(it.get("attrs") or {}, lr=0.0))
            out.append(it)
        return out

    def build_env(self, *, inputs: Dict[str, Any], params: Dict[str, Any], reuse_static: bool = False) -> Dict[int, Any]:
        from .plan import ROLE_INPUT as R_IN, ROLE_PARAM as R_PARAM, ROLE_STATIC as R_STATIC, Plan, ValueSpec
        bound: Dict[int, Any] = {}
        for src, kind in ((inputs, ROLE_INPUT), (params, ROLE_PARAM)):
            for name, obj in src.items():
                t = getattr(obj, "data", obj) if not hasattr(obj, "data_ptr") else obj
                if not hasattr(t, "data_ptr"):
                    raise TypeError(f"[plan] {kind} '{name}' must be a device tensor (data_ptr/shape/dtype), got {type(obj)}")
                vid = self._resolve(str(name), kind)
                self._check(self.plan.specs[vid], t)
                bound[vid] = t
        for vid in self.plan.inputs + self.plan.params:
            if vid not in bound:
                spec = self.plan.specs[vid]
                raise RuntimeError(f"[plan] env missing vid{vid} ({spec.name}) role={spec.role}")
        ptrs = {vid: int(t.data_ptr()) for vid, t in bound.items()}
        warmup = self._warmup_requested()
        if self._cplan is None or ptrs != self._bound_ptrs or not reuse_static or warmup != self._plan_is_warmup:
            if self._cplan is not None:
                self._cplan.close()
            role_code = {ROLE_INPUT: R_IN, ROLE_PARAM: R_PARAM, ROLE_STATIC: R_STATIC}
            # Every static is kept out of arena reuse: the caller may read any of them after the step.
            specs = [ValueSpec(s.vid, s.name, tuple(s.shape), short_dtype(s.dtype), role_code[s.role],
                               persistent=(s.role == ROLE_STATIC))
                     for _, s in sorted(self.plan.specs.items())]
            self._cplan = Plan(self.ir.name, specs, self._effective_lowered(warmup), bind=bound)
            self._plan_is_warmup = warmup
            self._bound_ptrs = ptrs
            self._captured = False
        self.env = {vid: bound[vid] if vid in bound else self._cplan.tensor(vid) for vid in sorted(self.plan.specs)}
        return self.env

    # ---- execution -----------------------------------------------------------------------------
    def _execute_lowered(self, *, stream: int) -> None:
        from . import _C
        from .plan import pack_attrs
        for i, it in enumerate(self._effective_lowered(self._warmup_requested())):
            op = str(it["op"])
            kind = opkind_from_name(op)
            ins = [self.env[int(v)] for v in it.get("inputs", [])]
            outs = [self.env[int(v)] for v in it.get("outputs", [])]
            schema_id, payload = pack_attrs(op, it.get("attrs"))
            kid = it.get("kernel_id")
            if self.opts.debug and i < int(self.opts.debug_limit):
                print(f"[exec][#{i:03d}] {op} kind={kind}{'' if not kid else f' kernel_id={kid}'} attrs={it.get('attrs') or {}}")
            if kid is not None:
                _C.launch_by_id(str(kid), _C.OpKind(kind), ins, outs, int(schema_id), payload, int(stream))
            else:
                _C.op_call(int(kind), ins, outs, int(schema_id), payload, int(stream))

    def run(self, *, inputs: Dict[str, Any], params: Dict[str, Any], reuse_static: bool = True) -> Dict[int, Any]:
        self.build_env(inputs=inputs, params=params, reuse_static=reuse_static)
        self._execute_lowered(stream=0)
        return self.env

    def capture(self, *, inputs: Dict[str, Any], params: Dict[str, Any], reuse_static: bool = True) -> Dict[int, Any]:
        """Records the step into a CUDA graph. As with any stream capture the step does not execute here."""
        self.build_env(inputs=inputs, params=params, reuse_static=reuse_static)
        self._cplan.capture()
        self._captured = True
        return self.env

    def replay(self, n: int = 1) -> None:
        if n <= 0:
            return
        if not self._captured:
            raise RuntimeError("[exec] replay called before capture()")
        self._cplan.replay(int(n))

    def reset_graph(self) -> None:
        if self._cplan is not None:
            self._cplan.reset_graph()
        self._captured = False

    def sync(self) -> None:
        if self._cplan is not None:
            self._cplan.sync()

    @property
    def compiled_plan(self):
        """The C++ plan behind this executor (None before the first run()/capture())."""
        return self._cplan


__all__ = [
    "IRValue", "IRNode", "IRGraph", "tracing", "is_tracing", "get_ir", "as_ir_value_obj", "trace_ir",
    "SymTensor", "sym_tensor", "linear", "relu", "save", "mse_grad", "linear_bwd", "relu_bwd", "step_inc", "bias_corr",
    "adam_step", "sgd_step", "softmax_ce_grad",
    "lower_to_backend_ops", "pick_kernel_id", "apply_kernel_selection", "apply_kernel_decisions_stageB",
    "stageC_fuse_gemm_epilogue", "apply_opt_rules", "compile_lowered", "elide_saved_copies",
    "BindSpec", "BindingPlan", "PlanOptions", "build_binding_plan", "ROLE_INPUT", "ROLE_PARAM", "ROLE_STATIC",
    "dump_ir", "dump_lowered", "dump_plan", "ExecOptions", "PlannedExecutor", "opkind_from_name", "short_dtype", "long_dtype",
]
