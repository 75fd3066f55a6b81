"""Interpreter for a lowered-op list over NumPy arrays (the CPU execution of the same op graph).
TEST INFRASTRUCTURE - see oracle/__init__.py.

Storage rounding follows the device: a value whose declared dtype is bf16 / f16 is rounded to that
type whenever an op writes it, while arithmetic runs in `dt` (fp64 = truth, fp32 = timed baseline).
The op names and attr keys are those of the reference's lowering
(python/aicf_fw/core_v2/lower.py:9-21, exec.py:178-201) plus this backend's additions."""
from __future__ import annotations

from typing import Any, Dict, Sequence

import numpy as np

from . import ops as O

_ROUND = {"f32": lambda a: np.asarray(a, np.float32), "bf16": O.bf16_round, "f16": O.f16_round,
          "i32": lambda a: np.asarray(a, np.int32)}


def _relu_flag(attrs: Dict[str, Any]) -> bool:
    if "relu" in attrs:
        return bool(attrs["relu"])
    if "epilogue" in attrs:
        return str(attrs["epilogue"]).lower() not in ("bias", "bias_only", "biasonly")
    if "epilogue_act" in attrs:
        return str(attrs["epilogue_act"]).lower() == "relu"
    return True


def run_lowered(lowered: Sequence[Dict[str, Any]], env: Dict[int, np.ndarray], dtypes: Dict[int, str], dt=np.float64,
                world_grads=None) -> Dict[int, np.ndarray]:
    """Executes `lowered` in place on `env` (vid -> array holding the value as float32/int32 after
    storage rounding). `world_grads`, if given, is called as world_grads(vid, local_array) for every
    all_reduce and must return the sum over ranks (the data-parallel oracle sums shards in rank order)."""

    def store(vid, arr):
        env[vid] = _ROUND[dtypes[vid]](np.asarray(arr))

    for it in lowered:
        op = it["op"]
        a = dict(it.get("attrs") or {})
        i = [env[v] for v in it["inputs"]]
        o = it["outputs"]
        if op == "gemm":
            store(o[0], O.gemm(i[0], i[1], a.get("transA", False), a.get("transB", False), dt))
        elif op == "gemm_epilogue":
            store(o[0], O.gemm_epilogue(i[0], i[1], i[2], a.get("transA", False), a.get("transB", False), _relu_flag(a), dt))
        elif op == "gemm_relu_bwd":
            store(o[0], O.gemm_relu_bwd(i[0], i[1], i[2], a.get("transA", False), a.get("transB", False), dt))
        elif op == "bias_add":
            store(o[0], O.bias_add(i[0], i[1], dt))
        elif op == "relu":
            store(o[0], O.relu(i[0], dt))
        elif op == "relu_bwd":
            store(o[0], O.relu_bwd(i[0], i[1], dt))
        elif op in ("copy", "copy_saved", "copy_aux", "cast"):
            store(o[0], i[0])
        elif op == "grad_zero":
            store(o[0], O.grad_zero(i[0], dt))
        elif op == "mse_grad":
            store(o[0], O.mse_grad(i[0], i[1], a.get("scale"), dt))
        elif op == "reduce_sum":
            if int(a.get("axis", 0)) == 0 and np.ndim(i[0]) >= 2:
                store(o[0], O.reduce_sum_columns(i[0], dt))
            else:
                store(o[0], np.reshape(O.reduce_lastaxis(i[0], "sum", dt), env[o[0]].shape if o[0] in env else -1))
        elif op in ("reduce_max", "reduce_mean"):
            r = O.reduce_lastaxis(i[0], op.split("_")[1], dt)
            store(o[0], np.reshape(r, (-1,)) if np.ndim(r) == 0 else r)
        elif op == "softmax":
            store(o[0], O.softmax(i[0], dt))
        elif op == "softmax_ce":
            d, loss, am = O.softmax_ce(i[0], i[1], a.get("scale"), dt)
            store(o[0], d)
            store(o[1], loss)
            if len(o) > 2:
                store(o[2], am)
        elif op == "layernorm_fwd":
            y, mu, rs = O.layernorm_fwd(i[0], i[1] if len(i) == 3 else None, i[2] if len(i) == 3 else None, a.get("eps", 1e-5), dt)
            store(o[0], y), store(o[1], mu), store(o[2], rs)
        elif op == "layernorm_bwd":
            aff = len(i) == 5
            dx, dg, db = O.layernorm_bwd(i[0], i[1], i[2] if aff else None, i[3 if aff else 2], i[4 if aff else 3], dt)
            store(o[0], dx)
            if aff:
                store(o[1], dg), store(o[2], db)
        elif op == "step_inc":
            store(o[0], O.step_inc(env[o[0]]))
        elif op == "bias_corr":
            b1, b2 = O.bias_corr(int(np.ravel(i[0])[0]), a.get("beta1", 0.9), a.get("beta2", 0.999), dt)
            store(o[0], np.reshape(b1, env[o[0]].shape))
            store(o[1], np.reshape(b2, env[o[1]].shape))
        elif op == "sgd_step":
            store(o[0], O.sgd_step(i[0], i[1], a.get("lr", 1e-3), dt))
        elif op == "add":
            store(o[0], O.add(i[0], i[1], dt))
        elif op == "adam_step":
            kw = dict(lr=a.get("lr", 1e-3), beta1=a.get("beta1", 0.9), beta2=a.get("beta2", 0.999), eps=a.get("eps", 1e-8))
            if len(i) > 6:   # multi-tensor form: [P,G,M,V] per tensor, then the step counter; in place
                T, step_now, k = (len(i) - 1) // 4, int(np.ravel(i[-1])[0]), 0
                for q in range(T):
                    p, m, v = O.adam_step_fused(i[4 * q], i[4 * q + 1], i[4 * q + 2], i[4 * q + 3], step_now,
                                                weight_decay=a.get("weight_decay", 0.0), decoupled=a.get("decoupled", False), dt=dt, **kw)
                    store(o[k], p), store(o[k + 1], m), store(o[k + 2], v)
                    k += 3
                    if (int(a.get("lp_mask", 0)) >> q) & 1:
                        store(o[k], p)  # low-precision working copy of the new parameter
                        k += 1
                continue
            if len(i) == 6:  # reference contract: divisor scalars
                p, m, v = O.adam_step_v0(i[0], i[1], i[2], i[3], float(np.ravel(i[4])[0]), float(np.ravel(i[5])[0]), dt=dt, **kw)
            else:            # fused contract: device step counter
                p, m, v = O.adam_step_fused(i[0], i[1], i[2], i[3], int(np.ravel(i[4])[0]), weight_decay=a.get("weight_decay", 0.0),
                                            decoupled=a.get("decoupled", False), dt=dt, **kw)
            store(o[0], p)
            store(o[1], m)
            store(o[2], v)
            if len(o) > 3:
                store(o[3], p)  # low-precision working copy of the new parameter
        elif op == "dp_adam_step":  # gradient summed over the ranks, then Adam; every rank ends with the same result
            g = world_grads(it["inputs"][1], i[1]) if world_grads else i[1]
            p, m, v = O.adam_step_fused(i[0], g, i[2], i[3], int(np.ravel(i[4])[0]), lr=a.get("lr", 1e-3),
                                        beta1=a.get("beta1", 0.9), beta2=a.get("beta2", 0.999), eps=a.get("eps", 1e-8),
                                        weight_decay=a.get("weight_decay", 0.0), decoupled=a.get("decoupled", False), dt=dt)
            store(o[0], p)
            store(o[1], m)
            store(o[2], v)
            if len(o) > 3:
                store(o[3], p)
        elif op == "all_reduce":
            store(o[0], world_grads(it["inputs"][0], i[0]) if world_grads else i[0])
        else:
            raise RuntimeError(f"[oracle] unsupported lowered op '{op}'")
    return env
