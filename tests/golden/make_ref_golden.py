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
    # f16 variants of the same ops (drawn last; values are stored as float32 holding exact f16 numbers)
    h16 = lambda a: np.asarray(a, np.float32).astype(np.float16)
    hshape = (6, 40, 64)
    hx, hy = h16(rng.standard_normal(hshape)), h16(rng.standard_normal(hshape))
    hb = h16(rng.standard_normal(hshape[-1]))
    g.update(h_x=hx.astype(np.float32), h_y=hy.astype(np.float32), h_bias=hb.astype(np.float32))
    HX, HY, HB = Tensor.from_numpy(hx), Tensor.from_numpy(hy), Tensor.from_numpy(hb)
    f16out = lambda kid, kind, ins, shape, **kw: run(kid, kind, ins, shape, out_dtype="f16", **kw)[0].astype(np.float32)
    g["h_relu"] = f16out("relu_f16_v0", OpKind.EltwiseRelu, [HX], hshape)
    g["h_relu_bwd"] = f16out("relu_bwd_f16_v0", OpKind.ReluBwd, [HX, HY], hshape)
    g["h_add"] = f16out("add_f16_v0", OpKind.EltwiseAdd, [HX, HY], hshape)
    g["h_mse_grad"] = f16out("mse_grad_f16_v0", OpKind.MseGrad, [HX, HY], hshape)
    g["h_sgd"] = f16out("sgd_step_f16_v0", OpKind.SgdStep, [HX, HY], hshape)
    g["h_bias_add"] = f16out("bias_add_f16_v0", OpKind.BiasAdd, [HX, HB], hshape)
    hr = h16(rng.standard_normal((129, 48)))
    g["h_red_x"] = hr.astype(np.float32)
    HR = Tensor.from_numpy(hr)
    g["h_colsum_f16"] = f16out("reduce_sum_keep_lastdim_f16_v0", OpKind.ReduceSum, [HR], (48,))
    g["h_colsum_f32"] = run("reduce_sum_keep_lastdim_f16_to_f32_v0", OpKind.ReduceSum, [HR], (48,))[0]
    HMm, HKk, HNn = 64, 48, 80
    hA, hB = h16(rng.uniform(-1, 1, (HMm, HKk))), h16(rng.uniform(-1, 1, (HKk, HNn)))
    hbias = h16(rng.standard_normal(HNn))
    g.update(h_gemm_A=hA.astype(np.float32), h_gemm_B=hB.astype(np.float32), h_gemm_bias=hbias.astype(np.float32))
    for ta in (0, 1):
        for tb in (0, 1):
            a = Tensor.from_numpy(np.ascontiguousarray(hA.T) if ta else hA)
            b = Tensor.from_numpy(np.ascontiguousarray(hB.T) if tb else hB)
            g[f"h_gemm_{ta}{tb}"] = f16out("gemm_f16_tc_wmma_out_f16_v0", OpKind.Gemm, [a, b], (HMm, HNn), schema=0x47454D4D,
                                           payload=struct.pack("<ii", ta, tb))
            g[f"h_gemm_epi_{ta}{tb}"] = f16out("gemm_bias_relu_f16_tc_wmma_out_f16_v0", OpKind.GemmEpilogue,
                                               [a, b, Tensor.from_numpy(hbias)], (HMm, HNn), schema=0x4750454C,
                                               payload=struct.pack("<iii", ta, tb, 1))
    hlx, hldy = h16(rng.standard_normal((LM, LN)) * 2.0 + 0.5), h16(rng.standard_normal((LM, LN)))
    hlg, hlb = h16(1.0 + 0.1 * rng.standard_normal(LN)), h16(0.1 * rng.standard_normal(LN))
    g.update(h_ln_x=hlx.astype(np.float32), h_ln_dy=hldy.astype(np.float32), h_ln_gamma=hlg.astype(np.float32),
             h_ln_beta=hlb.astype(np.float32))
    HLX, HLDY, HLG, HLB = (Tensor.from_numpy(a) for a in (hlx, hldy, hlg, hlb))
    y, mu, rs = run_multi("layernorm_fwd_f16_v0", OpKind.LayerNormFwd, [HLX, HLG, HLB],
                          [((LM, LN), "f16"), ((LM,), "f32"), ((LM,), "f32")], 0x50454E4C, lnep)
    g.update(h_ln_y=y.astype(np.float32), h_ln_mean=mu, h_ln_rstd=rs)
    dx, dg, db = run_multi("layernorm_bwd_f16_v0", OpKind.LayerNormBwd,
                           [HLX, HLDY, HLG, Tensor.from_numpy(mu), Tensor.from_numpy(rs)],
                           [((LM, LN), "f16"), ((LN,), "f32"), ((LN,), "f32")])
    g.update(h_ln_dx=dx.astype(np.float32), h_ln_dgamma=dg, h_ln_dbeta=db)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(out_path, **g)
    print(f"wrote {out_path} ({out_path.stat().st_size >> 10} KiB, {len(g)} arrays)")


if __name__ == "__main__":
    main(Path(sys.argv[1]) if len(sys.argv) > 1 else REPO / "tests" / "golden" / "ref_cuda_golden.npz")
