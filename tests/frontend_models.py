"""Model descriptions shared by tests/golden/make_frontend_golden.py (which traces them through the reference's
core_v2 front end) and tests/test_core_v2_frontend.py (which traces them through this repository's)."""
from __future__ import annotations

from typing import Any, Dict, List

MODELS: List[Dict[str, Any]] = [
    {"name": "mlp2_f16_sgd", "dtype": "f16", "batch": 64, "dims": [8, 8, 8], "bias": True, "opt": "sgd", "lr": 0.01},
    {"name": "mlp3_f16_sgd_odd", "dtype": "f16", "batch": 5, "dims": [7, 9, 3, 5], "bias": True, "opt": "sgd", "lr": 0.5},
    {"name": "mlp3_f32_sgd", "dtype": "f32", "batch": 16, "dims": [12, 6, 6, 4], "bias": True, "opt": "sgd", "lr": 0.125},
    {"name": "mlp2_f16_nobias", "dtype": "f16", "batch": 8, "dims": [4, 6, 2], "bias": False, "opt": "sgd", "lr": 0.01},
    {"name": "mlp1_f32_nobias", "dtype": "f32", "batch": 3, "dims": [5, 1], "bias": False, "opt": "sgd", "lr": 1.0},
    {"name": "mlp2_f32_adam", "dtype": "f32", "batch": 32, "dims": [16, 32, 10], "bias": True, "opt": "adam", "lr": 0.001,
     "beta1": 0.9, "beta2": 0.999, "eps": 1e-8, "scale": 0.03125},
    {"name": "mlp4_f16_sgd_scaled", "dtype": "f16", "batch": 128, "dims": [32, 64, 64, 64, 16], "bias": True, "opt": "sgd",
     "lr": 0.001, "scale": 0.0078125},
]


def build_model(api, spec: Dict[str, Any], dtype: Any, f32: Any, i32: Any, keep_alive: bool = True, **tensor_kw) -> None:
    """Emits one train step of `spec` through `api` (a module with sym_tensor, linear, relu, save, mse_grad, linear_bwd,
    relu_bwd, sgd_step, step_inc, bias_corr, adam_step). Layers are named 0, 2, 4, ... like torch.nn.Sequential
    with activations in between.

    With keep_alive every symbolic tensor stays referenced until the step is fully emitted. The reference maps a
    tensor to its IR value by id(object) without holding the object, so a temporary that is freed mid-trace can
    hand its id, and with it its IR value, to a later tensor; its own tests keep everything in locals."""
    keep: List[Any] = []

    class _Keep:
        def __getattr__(self, fn):
            def call(*a, **k):
                r = getattr(api_raw, fn)(*a, **k)
                if keep_alive:
                    keep.append(r)
                return r
            return call
    api_raw, api = api, _Keep()
    sym = lambda name, shape, dt=dtype: api.sym_tensor(name=name, shape=tuple(shape), dtype=dt, **tensor_kw)
    dims, Bn, bias = spec["dims"], spec["batch"], spec["bias"]
    L = len(dims) - 1
    x = sym("x", (Bn, dims[0]))
    t = sym("t", (Bn, dims[-1]))
    Ws = [sym(f"{2 * i}.W", (dims[i + 1], dims[i])) for i in range(L)]
    bs = [sym(f"{2 * i}.b", (dims[i + 1],)) if bias else None for i in range(L)]
    acts, saved, h = [x], [], x
    for i in range(L):
        h = api.linear(h, Ws[i], bs[i], name=f"lin{i}_out")
        if i < L - 1:
            h = api.relu(h, name=f"relu{i}_out")
            saved.append(api.save(h, name=f"relu{i}_saved"))
        acts.append(h)
    d = api.mse_grad(h, t, name="dY") if "scale" not in spec else api.mse_grad(h, t, scale=spec["scale"], name="dY")
    grads = [None] * L
    for i in reversed(range(L)):
        dx, dW, db = api.linear_bwd(acts[i], Ws[i], d, bias=bias, dx_name=f"d_in{i}", dW_name=f"d_{2 * i}.W",
                                    db_name=f"d_{2 * i}.b")
        grads[i] = (dW, db)
        if i > 0:
            d = api.relu_bwd(dx, saved[i - 1], name=f"d_lin{i - 1}_out")
    if spec["opt"] == "sgd":
        for i in range(L):
            api.sgd_step(Ws[i], grads[i][0], lr=spec["lr"])
            if bias:
                api.sgd_step(bs[i], grads[i][1], lr=spec["lr"])
        return
    step = api.step_inc(sym("opt.step", (), i32), name="opt.step")
    bc1, bc2 = api.bias_corr(step, sym("opt.bc1_inv", (), f32), sym("opt.bc2_inv", (), f32), beta1=spec["beta1"],
                             beta2=spec["beta2"])
    hyper = {k: spec[k] for k in ("lr", "beta1", "beta2", "eps")}
    for i in range(L):
        for p, g in ((Ws[i], grads[i][0]),) + (((bs[i], grads[i][1]),) if bias else ()):
            m, v = sym(f"opt.m.{p.name}", p.shape, f32), sym(f"opt.v.{p.name}", p.shape, f32)
            api.adam_step(p, g, m, v, bc1, bc2, **hyper)
