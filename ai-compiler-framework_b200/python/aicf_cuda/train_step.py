"""compile_train_step: from a layer list to a captured train step, through the tracing front end.

The reference's user API calls `aicf_fw.fw.compile.compile_train_step(model, optimizer, B=, D=, device=, dtype=,
name=, warmup_runs=, ...)` (fw/module.py:64-97) and expects back an object with train_step / capture / replay /
reset (fw/train_step.py:15-101); the module that defines it is absent from the reference's tree. This is that entry
point for the MLP family the hot path covers, without torch: the model is given as its layer widths, the step is
traced with `core_v2` ops (Linear, ReLU, Save, MseGrad, LinearBwd, ReluBwd, then SgdStep or StepInc + BiasCorr +
AdamStep), lowered with stages A/B/C, and run by `PlannedExecutor` over the C++ plan.

One deliberate difference: the reference's Adam keeps the step count and the two bias-correction scalars on the host
and refreshes them before every eager step (optim/adam.py:40-45), which a graph replay cannot do. Here the counter
and the scalars are device values updated by step_inc and bias_corr inside the step, so replay(n) advances them.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from . import core_v2 as cv
from .tensor import _NP_OF, Tensor, f32_to_bf16_bits


def same_name_is_same_storage(ir: cv.IRGraph, lowered: Sequence[Dict[str, Any]], prefix: str = "opt.") -> List[Dict[str, Any]]:
    """Rewrites value ids so that every value whose name starts with `prefix` and equals an earlier value's name uses
    that earlier value: optimizer state named twice in a trace (the step counter before and after step_inc) is one
    buffer. The reference gets the same effect when both handles are one torch tensor (trace.py:59-74)."""
    first: Dict[str, int] = {}
    remap: Dict[int, int] = {}
    for vid in sorted(ir.values):
        nm = ir.values[vid].name
        if nm.startswith(prefix):
            remap[vid] = first.setdefault(nm, vid)
    fix = lambda vs: [remap.get(int(v), int(v)) for v in vs]
    return [dict(it, inputs=fix(it.get("inputs", [])), outputs=fix(it.get("outputs", []))) for it in lowered]


class CompiledTrainStep:
    """Handle returned by compile_train_step. `params` and `inputs` are device tensors owned by this object; batches
    given as host arrays are copied into `inputs`, so their addresses never change under a captured graph."""

    def __init__(self, *, ir, lowered, plan, ex: cv.PlannedExecutor, params: Dict[str, Tensor], inputs: Dict[str, Tensor],
                 warmup_runs: int = 0):
        self.ir, self.lowered, self.plan, self.ex = ir, lowered, plan, ex
        self.params, self.inputs = params, inputs
        self.warmup_runs = int(warmup_runs)
        self._names = {v.name: vid for vid, v in sorted(ir.values.items(), reverse=True)}

    def _stage(self, batch: Optional[Dict[str, Any]]) -> None:
        for k, v in (batch or {}).items():
            if k not in self.inputs:
                raise KeyError(f"unknown input '{k}' (inputs: {sorted(self.inputs)})")
            if isinstance(v, np.ndarray):
                dt = self.inputs[k].dtype
                self.inputs[k].copy_from_host(f32_to_bf16_bits(v.astype(np.float32)) if dt == "bf16" else v.astype(_NP_OF[dt]))
            elif int(v.data_ptr()) != int(self.inputs[k].data_ptr()):
                raise ValueError(f"input '{k}' must be a host array or this step's own input tensor")

    def train_step(self, batch: Optional[Dict[str, Any]] = None, reuse_static: bool = True):
        self._stage(batch)
        return self.ex.run(inputs=self.inputs, params=self.params, reuse_static=reuse_static)

    run = train_step

    def capture(self, batch: Optional[Dict[str, Any]] = None, reuse_static: bool = True) -> None:
        self._stage(batch)
        self.ex.reset_graph()
        self.ex.capture(inputs=self.inputs, params=self.params, reuse_static=reuse_static)

    def replay(self, n: int = 1, sync: bool = False) -> None:
        self.ex.replay(n=int(n))
        if sync:
            self.ex.sync()

    def reset(self) -> None:
        self.ex.reset_graph()

    def sync(self) -> None:
        from . import _C
        self.ex.sync()
        _C.device_sync()

    def value(self, name: str) -> Tensor:
        """Device tensor of any value of the step by name (gradients 'd_0.W', optimizer state 'opt.m.0.W', ...)."""
        if not self.ex.env:
            self.ex.build_env(inputs=self.inputs, params=self.params, reuse_static=True)
        return self.ex.env[self._names[name]]


def compile_train_step(dims: Sequence[int], *, B: int, dtype: str = "f32", bias: bool = True, optimizer: str = "sgd",
                       lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                       loss_scale: Optional[float] = None, name: str = "train_step", seed: int = 0,
                       init_scale: float = 0.02, params: Optional[Dict[str, np.ndarray]] = None,
                       require_kernel_id: bool = True) -> CompiledTrainStep:
    """MLP dims[0] -> ... -> dims[-1] with ReLU between layers, MSE loss gradient, SGD or Adam. Layers are named
    0, 2, 4, ... (a Sequential with activations in between). Parameters start as N(0, init_scale^2) weights and zero
    biases, or from `params` (host arrays by name). Parameters, activations and gradients are all `dtype`."""
    dims = [int(d) for d in dims]
    L = len(dims) - 1
    if L < 1:
        raise ValueError("dims needs at least an input and an output width")
    if optimizer not in ("sgd", "adam"):
        raise ValueError(f"unknown optimizer {optimizer!r}")
    pnames = [(f"{2 * i}.W", (dims[i + 1], dims[i])) for i in range(L)]
    if bias:
        pnames = [p for i in range(L) for p in (pnames[i], (f"{2 * i}.b", (dims[i + 1],)))]

    def step():
        sym = lambda nm, shape, dt=dtype: cv.sym_tensor(name=nm, shape=shape, dtype=dt)
        x, t = sym("x", (B, dims[0])), sym("t", (B, dims[-1]))
        P = {nm: sym(nm, shape) for nm, shape in pnames}
        acts, saved, h = [x], [], x
        for i in range(L):
            h = cv.linear(h, P[f"{2 * i}.W"], P.get(f"{2 * i}.b"), name=f"lin{i}_out")
            if i < L - 1:
                h = cv.relu(h, name=f"relu{i}_out")
                saved.append(cv.save(h, name=f"relu{i}_saved"))
            acts.append(h)
        d = cv.mse_grad(h, t, scale=loss_scale, name="dY")
        G: Dict[str, cv.SymTensor] = {}
        for i in reversed(range(L)):
            dx, dW, db = cv.linear_bwd(acts[i], P[f"{2 * i}.W"], d, bias=bias, dx_name=f"d_in{i}", dW_name=f"d_{2 * i}.W",
                                       db_name=f"d_{2 * i}.b")
            G[f"{2 * i}.W"] = dW
            if bias:
                G[f"{2 * i}.b"] = db
            if i > 0:
                d = cv.relu_bwd(dx, saved[i - 1], name=f"d_lin{i - 1}_out")
        if optimizer == "sgd":
            for nm, _ in pnames:
                cv.sgd_step(P[nm], G[nm], lr=lr)
            return
        st = cv.step_inc(sym("opt.step", (), "i32"), name="opt.step")
        bc1, bc2 = cv.bias_corr(st, sym("opt.bc1_inv", (), "f32"), sym("opt.bc2_inv", (), "f32"), beta1=beta1, beta2=beta2,
                                out1_name="opt.bc1_inv", out2_name="opt.bc2_inv")
        for nm, shape in pnames:
            cv.adam_step(P[nm], G[nm], sym(f"opt.m.{nm}", shape, "f32"), sym(f"opt.v.{nm}", shape, "f32"), bc1, bc2,
                         lr=lr, beta1=beta1, beta2=beta2, eps=eps)

    ir = cv.trace_ir(step, name=name)
    lowered = same_name_is_same_storage(ir, cv.compile_lowered(ir))
    plan = cv.build_binding_plan(ir)
    ex = cv.PlannedExecutor(ir=ir, lowered=lowered, plan=plan, opts=cv.ExecOptions(require_kernel_id=require_kernel_id))
    rng = np.random.default_rng(seed)
    host: Dict[str, np.ndarray] = {}
    for nm, shape in pnames:
        if params is not None:
            host[nm] = np.asarray(params[nm], dtype=np.float32).reshape(shape)
        else:
            host[nm] = (rng.standard_normal(shape) * init_scale).astype(np.float32) if nm.endswith(".W") else np.zeros(shape, np.float32)
    dev_params = {nm: Tensor.from_numpy(a, dtype) for nm, a in host.items()}
    dev_inputs = {"x": Tensor.zeros((B, dims[0]), dtype), "t": Tensor.zeros((B, dims[-1]), dtype)}
    return CompiledTrainStep(ir=ir, lowered=lowered, plan=plan, ex=ex, params=dev_params, inputs=dev_inputs)
