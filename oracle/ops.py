"""One function per lowered op. `dt` selects the arithmetic type: np.float64 = truth, np.float32 = the
timed CPU baseline. File:line citations are relative to the reference's ai-compiler-framework/ tree.
TEST INFRASTRUCTURE - see oracle/__init__.py."""
from __future__ import annotations

import numpy as np

__all__ = ["bf16_round", "f16_round", "gemm", "gemm_epilogue", "gemm_relu_bwd", "bias_add", "relu", "relu_bwd", "copy", "grad_zero",
           "mse_grad", "reduce_sum_columns", "reduce_lastaxis", "adam_step_v0", "adam_step_fused", "step_inc",
           "bias_corr", "sgd_step", "add", "softmax", "softmax_ce", "cast", "layernorm_fwd", "layernorm_bwd"]


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 -> fp32 with round-to-nearest-even (what the device stores in a bf16 tensor)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)) << np.uint32(16)
    return r.view(np.float32).reshape(np.shape(x))


def f16_round(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def _op(a: np.ndarray, trans: bool) -> np.ndarray:
    return a.T if trans else a


def gemm(A, B, transA=False, transB=False, dt=np.float64):
    """C = op(A) @ op(B)  (ops/gemm/launcher.cu:155-172; transposes are stride swaps, :98-114)."""
    return _op(np.asarray(A, dt), transA) @ _op(np.asarray(B, dt), transB)


def gemm_epilogue(A, B, bias, transA=False, transB=False, relu=True, dt=np.float64):
    """C = [relu](op(A) @ op(B) + bias[col])  (ops/gemm_epilogue/launcher.cu:202-225; relu defaults
    to on when no attrs are given, :57-60)."""
    c = gemm(A, B, transA, transB, dt) + np.asarray(bias, dt)[None, :]
    return np.maximum(c, 0) if relu else c


def gemm_relu_bwd(dY, W, Y, transA=False, transB=False, dt=np.float64):
    """dX = (Y > 0) ? op(dY) @ op(W) : 0 - the reference's gemm followed by its relu_bwd
    (python/aicf_fw/core_v2/lower.py:88-111 emits them as two ops; ops/relu_bwd/launcher.cu:37-44)."""
    return relu_bwd(gemm(dY, W, transA, transB, dt), Y, dt)


def bias_add(Y, bias, dt=np.float64):
    """Out = Y + bias over the last axis (ops/bias_add/launcher.cu:36-47)."""
    return np.asarray(Y, dt) + np.asarray(bias, dt)


def relu(X, dt=np.float64):
    """max(x, 0)  (ops/relu/launcher.cu:44-51)."""
    return np.maximum(np.asarray(X, dt), 0)


def relu_bwd(dOut, Y, dt=np.float64):
    """dY = Y > 0 ? dOut : 0; operand order (dOut, Y)  (ops/relu_bwd/launcher.cu:37-44)."""
    return np.where(np.asarray(Y, dt) > 0, np.asarray(dOut, dt), 0).astype(dt)


def copy(X, dt=np.float64):
    """y = x  (ops/copy/kernels.cuh:8-18)."""
    return np.array(X, dtype=dt, copy=True)


def grad_zero(X, dt=np.float64):
    """zero fill (ops/grad_zero/launcher.cu:93-119)."""
    return np.zeros_like(np.asarray(X, dt))


def mse_grad(pred, target, scale=None, dt=np.float64):
    """(pred - target) * scale, scale defaults to 2/numel  (ops/mse_grad/launcher.cu:61-70,213-215)."""
    p = np.asarray(pred, dt)
    s = dt(2.0) / dt(p.size) if scale is None else dt(scale)
    return (p - np.asarray(target, dt)) * s


def reduce_sum_columns(dY, dt=np.float64):
    """[..., N] -> [N]: sum over every leading axis (the bias gradient)
    (ops/reduce_sum/launcher.cu:38-57,140-154)."""
    a = np.asarray(dY, dt)
    return a.reshape(-1, a.shape[-1]).sum(axis=0)


def reduce_lastaxis(X, kind="sum", dt=np.float64):
    """[..., N] -> [...]: sum / max / mean over the last axis (not in the reference)."""
    a = np.asarray(X, dt)
    return {"sum": a.sum, "max": a.max, "mean": a.mean}[kind](axis=-1)


def adam_step_v0(P, G, M, V, bc1, bc2, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, dt=np.float64):
    """The reference kernel verbatim in NumPy: bc1/bc2 are DIVISORS
    (ops/adam_step/launcher.cu:269-291):
        m' = b1 m + (1-b1) g;  v' = b2 v + (1-b2) g^2;  p' = p - lr * (m'/bc1) / (sqrt(v'/bc2) + eps)."""
    p, g, m, v = (np.asarray(t, dt) for t in (P, G, M, V))
    m2 = dt(beta1) * m + (dt(1) - dt(beta1)) * g
    v2 = dt(beta2) * v + (dt(1) - dt(beta2)) * (g * g)
    p2 = p - dt(lr) * ((m2 / dt(bc1)) / (np.sqrt(v2 / dt(bc2)) + dt(eps)))
    return p2, m2, v2


def adam_step_fused(P, G, M, V, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0,
                    decoupled=False, dt=np.float64):
    """Textbook Adam (Kingma & Ba 2015, algorithm 1) with bias correction 1-beta^t, t = max(step, 1).
    weight_decay: coupled adds wd*p to the gradient (L2); decoupled shrinks p by lr*wd*p (AdamW).
    Not in the reference, whose chained step_inc -> bias_corr -> adam_step path multiplies by the
    inverse corrections instead of dividing (see the Adam note in the oracle tests)."""
    p, g, m, v = (np.asarray(t, dt) for t in (P, G, M, V))
    t = max(int(step), 1)
    if weight_decay and not decoupled:
        g = g + dt(weight_decay) * p
    m2 = dt(beta1) * m + (dt(1) - dt(beta1)) * g
    v2 = dt(beta2) * v + (dt(1) - dt(beta2)) * (g * g)
    d1 = dt(1) - dt(beta1) ** t
    d2 = dt(1) - dt(beta2) ** t
    base = p - dt(lr) * dt(weight_decay) * p if (weight_decay and decoupled) else p
    p2 = base - dt(lr) * ((m2 / d1) / (np.sqrt(v2 / d2) + dt(eps)))
    return p2, m2, v2


def step_inc(S_out):
    """step += 1 on the OUTPUT buffer; the input is never read (ops/step_inc/launcher.cu:34-38,140-141)."""
    return np.asarray(S_out, np.int32) + np.int32(1)


def bias_corr(step, beta1=0.9, beta2=0.999, dt=np.float64):
    """(1/(1-b1^t), 1/(1-b2^t)), t = max(step,1), denominators clamped at 1e-20
    (ops/biascorr/launcher.cu:82-101)."""
    t = max(int(step), 1)
    d1 = dt(1) - dt(beta1) ** dt(t)
    d2 = dt(1) - dt(beta2) ** dt(t)
    d1 = dt(1e-20) if abs(d1) < 1e-20 else d1
    d2 = dt(1e-20) if abs(d2) < 1e-20 else d2
    return dt(1) / d1, dt(1) / d2


def sgd_step(P, G, lr=1e-3, dt=np.float64):
    """P - lr*G, lr defaults to 1e-3  (ops/sgd_step/launcher.cu:111-119,210)."""
    return np.asarray(P, dt) - dt(lr) * np.asarray(G, dt)


def add(A, B, dt=np.float64):
    """a + b  (ops/add/launcher.cu:44-50)."""
    return np.asarray(A, dt) + np.asarray(B, dt)


def cast(X, to: str):
    x = np.asarray(X, np.float32)
    return {"f32": lambda a: a, "bf16": bf16_round, "f16": f16_round}[to](x)


def softmax(X, dt=np.float64):
    """Row softmax over the last axis, max-subtracted (not in the reference)."""
    a = np.asarray(X, dt)
    e = np.exp(a - a.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def softmax_ce(logits, labels, scale=None, dt=np.float64):
    """Fused softmax cross-entropy (not in the reference):
        loss_row = logsumexp(z) - z[label];  dlogits = (softmax(z) - onehot(label)) * scale;
        argmax = first index of the row maximum.  scale defaults to 1/B.
    Labels outside [0, C) give zero loss and no one-hot term."""
    z = np.asarray(logits, dt)
    lab = np.asarray(labels, np.int64)
    B, Cn = z.shape
    s = dt(1.0 / B) if scale is None else dt(scale)
    mx = z.max(axis=1, keepdims=True)
    e = np.exp(z - mx)
    se = e.sum(axis=1, keepdims=True)
    ok = (lab >= 0) & (lab < Cn)
    safe = np.where(ok, lab, 0)
    loss = np.where(ok, (np.log(se) + mx)[:, 0] - z[np.arange(B), safe], 0).astype(dt)
    d = (e / se) * s
    rows = np.nonzero(ok)[0]
    d[rows, lab[rows]] -= s
    return d, loss, z.argmax(axis=1).astype(np.int32)


def layernorm_fwd(X, gamma=None, beta=None, eps=1e-5, dt=np.float64):
    """(y, mean, rstd) over the last axis of X[M, N]: mean = sum(x)/N, var = max(sum(x^2)/N - mean^2, 0),
    rstd = 1/sqrt(var + eps), y = (x - mean) * rstd [* gamma + beta]; eps defaults to 1e-5
    (ops/layernorm/launcher.cu:128-170 forward kernel, :49-56 and :456 eps)."""
    x = np.asarray(X, dt)
    n = x.shape[-1]
    mu = x.sum(axis=-1) / dt(n)
    var = np.maximum((x * x).sum(axis=-1) / dt(n) - mu * mu, dt(0))
    rs = dt(1) / np.sqrt(var + dt(eps))
    y = (x - mu[..., None]) * rs[..., None]
    if gamma is not None:
        y = y * np.asarray(gamma, dt) + np.asarray(beta, dt)
    return y, mu, rs


def layernorm_bwd(X, dY, gamma, mean, rstd, dt=np.float64):
    """(dx, dgamma, dbeta); gamma=None is the non-affine form and returns (dx, None, None).
    xhat = (x - mean) * rstd, g = dy [* gamma], dx = (N*g - sum(g) - xhat * sum(g * xhat)) * rstd / N
    (ops/layernorm/launcher.cu:221-262); dgamma = sum over rows of dy * xhat, dbeta = sum over rows of dy
    (:309-340)."""
    x, dy = np.asarray(X, dt), np.asarray(dY, dt)
    n = x.shape[-1]
    mu, rs = np.asarray(mean, dt)[..., None], np.asarray(rstd, dt)[..., None]
    xhat = (x - mu) * rs
    g = dy if gamma is None else dy * np.asarray(gamma, dt)
    s1 = g.sum(axis=-1, keepdims=True)
    s2 = (g * xhat).sum(axis=-1, keepdims=True)
    dx = (dt(n) * g - s1 - xhat * s2) * (rs / dt(n))
    if gamma is None:
        return dx, None, None
    lead = tuple(range(x.ndim - 1))
    return dx, (dy * xhat).sum(axis=lead), dy.sum(axis=lead)
