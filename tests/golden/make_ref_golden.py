"""Generates tests/golden/ref_cuda_golden.npz: outputs of the REFERENCE's own CUDA kernels.

Needs a GPU and oracle/_ref/libaicf_ref.so (oracle/ref_build.py). Run from the repository root:

    python tests/golden/make_ref_golden.py [out.npz]

Inputs are small seeded arrays (kept in the file next to the outputs), so the CPU test
tests/test_oracle_cpu.py::test_oracle_against_reference_cuda_golden_vectors can check the NumPy oracle
against what the reference really computes without a GPU.
"""
from __future__ import annotations

import ctypes as C
import struct
import sys
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parents[2]
sys.path[:0] = [str(REPO), str(REPO / "ai-compiler-framework_b200" / "python"), str(REPO / "tests")]

from aicf_cuda import Tensor  # noqa: E402  (device buffers only; every kernel run here is the reference's)
from aicf_cuda._C import OpKind  # noqa: E402
from util import ref_by_id  # noqa: E402


def main(out_path: Path) -> None:
    ref = C.CDLL(str(REPO / "oracle" / "_ref" / "libaicf_ref.so"))
    ref.ref_launch_by_id.restype = C.c_int
    ref.ref_launch_by_id.argtypes = [C.c_char_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_uint64]
    rng = np.random.default_rng(2026)
    g: dict[str, np.ndarray] = {}

    def run(kid, kind, ins, out_shape, schema=0, payload=b"", out_dtype="f32", n_out=1):
        outs = [Tensor.zeros(out_shape, out_dtype) for _ in range(n_out)]
        st = ref_by_id(ref, kid, kind, ins, outs, schema, payload)
        assert st == 0, (kid, st)
        return [o.numpy() for o in outs]

    M, K, N = 48, 40, 56
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    g.update(gemm_A=A, gemm_B=B, gemm_bias=bias)
    for ta in (0, 1):
        for tb in (0, 1):
            a = Tensor.from_numpy(np.ascontiguousarray(A.T) if ta else A)
            b = Tensor.from_numpy(np.ascontiguousarray(B.T) if tb else B)
            g[f"gemm_f32_{ta}{tb}"] = run("gemm_f32_naive_v0", OpKind.Gemm, [a, b], (M, N), 0x47454D4D, struct.pack("<ii", ta, tb))[0]
            for relu in (0, 1):
                g[f"gemm_epi_f32_{ta}{tb}{relu}"] = run("gemm_bias_relu_f32_naive_v0", OpKind.GemmEpilogue,
                                                        [a, b, Tensor.from_numpy(bias)], (M, N), 0x4750454C,
                                                        struct.pack("<iii", ta, tb, relu))[0]
    shape = (8, 32, 128)
    x = rng.standard_normal(shape).astype(np.float32)
    y = rng.standard_normal(shape).astype(np.float32)
    eb = rng.standard_normal(shape[-1]).astype(np.float32)
    X, Y = Tensor.from_numpy(x), Tensor.from_numpy(y)
    g.update(elt_x=x, elt_y=y, elt_bias=eb)
    g["relu_f32"] = run("relu_f32_v0", OpKind.EltwiseRelu, [X], shape)[0]
    g["relu_bwd_f32"] = run("relu_bwd_f32_v0", OpKind.ReluBwd, [X, Y], shape)[0]
    g["mse_grad_f32"] = run("mse_grad_f32_v0", OpKind.MseGrad, [X, Y], shape)[0]
    g["add_f32"] = run("add_f32_v0", OpKind.EltwiseAdd, [X, Y], shape)[0]
    g["sgd_f32"] = run("sgd_step_f32_v0", OpKind.SgdStep, [X, Y], shape)[0]
    g["bias_add_f32"] = run("bias_add_f32_v0", OpKind.BiasAdd, [X, Tensor.from_numpy(eb)], shape)[0]
    rx = rng.standard_normal((257, 64)).astype(np.float32)
    g["red_x"] = rx
    g["colsum_f32"] = run("reduce_sum_keep_lastdim_f32_v0", OpKind.ReduceSum, [Tensor.from_numpy(rx)], (64,))[0]
    p = rng.standard_normal((64, 256)).astype(np.float32)
    gr = (rng.standard_normal((64, 256)) * 1e-2).astype(np.float32)
    m = (rng.standard_normal((64, 256)) * 1e-2).astype(np.float32)
    v = np.abs(rng.standard_normal((64, 256)) * 1e-3).astype(np.float32)
    bc = np.array([1 - 0.9 ** 3, 1 - 0.999 ** 3], np.float32)
    g.update(adam_p=p, adam_g=gr, adam_m=m, adam_v=v, adam_bc=bc)
    outs = run("adam_step_f32_v0", OpKind.AdamStep,
               [Tensor.from_numpy(p), Tensor.from_numpy(gr), Tensor.from_numpy(m), Tensor.from_numpy(v),
                Tensor.from_numpy(np.array(bc[0], np.float32)), Tensor.from_numpy(np.array(bc[1], np.float32))],
               (64, 256), 0x4D414441, struct.pack("<ffff", 1e-3, 0.9, 0.999, 1e-8), n_out=3)
    g["adam_p_out"], g["adam_m_out"], g["adam_v_out"] = outs
    for t in (1, 10):
        o = run("bias_corr_v0", OpKind.BiasCorr, [Tensor.from_numpy(np.array(t, np.int32))], (), 0x524F4342,
                struct.pack("<ff", 0.9, 0.999), n_out=2)
        g[f"bias_corr_{t}"] = np.array([o[0].ravel()[0], o[1].ravel()[0]], np.float32)
    # layer norm (drawn after everything above so that the earlier inputs keep their values)
    def run_multi(kid, kind, ins, out_specs, schema=0, payload=b""):
        outs = [Tensor.zeros(s, d) for s, d in out_specs]
        st = ref_by_id(ref, kid, kind, ins, outs, schema, payload)
        assert st == 0, (kid, st)
        return [o.numpy() for o in outs]

    LM, LN = 37, 96
    lx = (rng.standard_normal((LM, LN)) * 2.0 + 0.5).astype(np.float32)
    ldy = rng.standard_normal((LM, LN)).astype(np.float32)
    lg = (1.0 + 0.1 * rng.standard_normal(LN)).astype(np.float32)
    lb = (0.1 * rng.standard_normal(LN)).astype(np.float32)
    g.update(ln_x=lx, ln_dy=ldy, ln_gamma=lg, ln_beta=lb)
    LX, LDY, LG, LB = (Tensor.from_numpy(a) for a in (lx, ldy, lg, lb))
    fwd_specs = [((LM, LN), "f32"), ((LM,), "f32"), ((LM,), "f32")]
    lnep = struct.pack("<f", 1e-5)
    y, mu, rs = run_multi("layernorm_fwd_f32_v0", OpKind.LayerNormFwd, [LX, LG, LB], fwd_specs, 0x50454E4C, lnep)
    g.update(ln_y_affine=y, ln_mean=mu, ln_rstd=rs)
    g["ln_y_plain"] = run_multi("layernorm_fwd_f32_v0", OpKind.LayerNormFwd, [LX], fwd_specs, 0x50454E4C, lnep)[0]
    MU, RS = Tensor.from_numpy(mu), Tensor.from_numpy(rs)
    dx, dg, db = run_multi("layernorm_bwd_f32_v0", OpKind.LayerNormBwd, [LX, LDY, LG, MU, RS],
                           [((LM, LN), "f32"), ((LN,), "f32"), ((LN,), "f32")])
    g.update(ln_dx_affine=dx, ln_dgamma=dg, ln_dbeta=db)
    g["ln_dx_plain"] = run_multi("layernorm_bwd_f32_v0", OpKind.LayerNormBwd, [LX, LDY, MU, RS], [((LM, LN), "f32")])[0]
    out_path.parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(out_path, **g)
    print(f"wrote {out_path} ({out_path.stat().st_size >> 10} KiB, {len(g)} arrays)")


if __name__ == "__main__":
    main(Path(sys.argv[1]) if len(sys.argv) > 1 else REPO / "tests" / "golden" / "ref_cuda_golden.npz")
