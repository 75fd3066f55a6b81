"""Builds the lowered-op list of an MLP train step (the contract the plan consumes).

The op/attr vocabulary is the reference's (python/aicf_fw/core_v2/lower.py:24-147: Linear ->
gemm{transB} + bias, LinearBwd -> gemm(dY,W), gemm(dY^T,X), reduce_sum(dY){axis 0}; Stage C fuses
gemm + bias_add + relu into gemm_epilogue, rewrites/stageC_fuse_epilogue.py:22-74), extended with the
ops this backend adds: softmax_ce as the loss, the fused Adam that reads the device step counter, bf16
working copies of fp32 master weights, and all_reduce for data parallelism.

Differences from what the reference's lowering would emit, all of them removing work:
  * the activation saved for relu_bwd is the gemm_epilogue output itself (no copy_saved op),
  * no dX for the first layer,
  * the last Linear is a gemm_epilogue with relu off instead of gemm + bias_add,
  * gemm(dY, W) followed by relu_bwd is one gemm_relu_bwd op: the mask is applied in the GEMM epilogue, which
    saves one read and one write of the activation gradient per hidden layer.
"""
from __future__ import annotations

from typing import Any, Dict, List, Sequence, Tuple

from .spec import ROLE_INPUT, ROLE_PARAM, ROLE_STATIC, ValueSpec


def build_mlp_train_step(batch: int, dims: Sequence[int], *, compute_dtype: str = "bf16", global_batch: int | None = None,
                         lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                         weight_decay: float = 0.0, data_parallel=False, with_argmax: bool = False,
                         input_f32: bool = True, fuse_relu_bwd: bool = True,
                         fp32_gemm: str = "exact", fuse_adam: bool = True) -> Tuple[List[ValueSpec], List[Dict[str, Any]]]:
    """dims = [in, hidden..., out]. Every Linear but the last is followed by ReLU.

    compute_dtype 'f32': GEMMs run on fp32 parameters directly.
    compute_dtype 'bf16' / 'f16': parameters, gradients and Adam state stay fp32; GEMMs read 16-bit
    working copies ('<i>.W.lp') which the fused Adam rewrites every step; activations are 16-bit.
    The loss gradient is scaled by 1/global_batch so that summed shard gradients equal the
    single-device gradient.

    fp32_gemm (compute_dtype 'f32' only): 'exact' pins the fp32 FMA kernels (bit-identical to the reference's);
    '3xtf32' pins the tensor-core ids that form every product from three TF32 products (~6x faster on large layers,
    normwise error ~2e-6 instead of ~4e-7).

    fuse_adam: the whole optimizer step is one `adam_step` op over all parameter tensors (kernel
    adam_step_f32_multi_v1) instead of one op per tensor; the arithmetic per element is the same.

    data_parallel: False - single device; True / "nccl" - an all_reduce op per gradient tensor, then the
    ordinary fused Adam; "fused" - one dp_adam_step op per parameter that exchanges the gradient over peer
    memory, updates the owning rank's shard and broadcasts the new weights (master weights and moments of
    matrices are then sharded over the ranks).
    """
    L = len(dims) - 1
    assert L >= 1
    dp_mode = {False: None, None: None, True: "nccl", "nccl": "nccl", "fused": "fused"}[data_parallel]
    fused_dp = dp_mode == "fused"
    cd = compute_dtype
    mixed = cd != "f32"
    gb = int(global_batch or batch)
    vals: List[ValueSpec] = []
    ops: List[Dict[str, Any]] = []
    ids: Dict[str, int] = {}

    def val(name, shape, dtype, role=None, persistent=False, zero=None, peer=False) -> int:
        vid = len(vals)
        vals.append(ValueSpec(vid, name, tuple(shape), dtype, role, persistent, zero, None, peer))
        ids[name] = vid
        return vid

    def op(name, inputs, outputs, attrs=None, kid=None):
        d: Dict[str, Any] = {"op": name, "inputs": list(inputs), "outputs": list(outputs), "attrs": dict(attrs or {})}
        if kid:
            d["kernel_id"] = kid
        ops.append(d)

    gemm_kid = {"f32": "gemm_f32_naive_v0", "bf16": "gemm_bf16_tcgen05_out_bf16_v0", "f16": "gemm_f16_tcgen05_out_f16_v0"}[cd]
    gemm_f32out_kid = {"f32": "gemm_f32_naive_v0", "bf16": "gemm_bf16_tcgen05_out_f32_v0", "f16": "gemm_f16_tcgen05_out_f32_v0"}[cd]
    epi_kid = {"f32": "gemm_bias_relu_f32_naive_v0", "bf16": "gemm_bias_relu_bf16_tcgen05_out_bf16_v0",
               "f16": "gemm_bias_relu_f16_tcgen05_out_f16_v0"}[cd]
    colsum_kid = {"f32": "reduce_sum_keep_lastdim_f32_v0", "bf16": "reduce_sum_keep_lastdim_bf16_to_f32_v0",
                  "f16": "reduce_sum_keep_lastdim_f16_to_f32_v0"}[cd]
    relu_bwd_kid = {"f32": "relu_bwd_f32_v0", "bf16": "relu_bwd_bf16_v0", "f16": "relu_bwd_f16_v0"}[cd]
    fused_kid = {"f32": "gemm_relu_bwd_f32_v0", "bf16": "gemm_relu_bwd_bf16_tcgen05_out_bf16_v0",
                 "f16": "gemm_relu_bwd_f16_tcgen05_out_f16_v0"}[cd]
    if fp32_gemm not in ("exact", "3xtf32"):
        raise ValueError(f"fp32_gemm must be 'exact' or '3xtf32', got {fp32_gemm!r}")
    if cd == "f32" and fp32_gemm == "3xtf32":
        gemm_kid = gemm_f32out_kid = "gemm_f32_3xtf32_v0"
        epi_kid = "gemm_bias_relu_f32_3xtf32_v0"
        fused_kid = "gemm_relu_bwd_f32_3xtf32_v0"
    ce_kid = {"f32": "softmax_ce_f32_i32_v0", "bf16": "softmax_ce_bf16_i32_v0", "f16": "softmax_ce_f16_i32_v0"}[cd]

    # ---- inputs -------------------------------------------------------------------------------
    if mixed and input_f32:
        x_in = val("x", (batch, dims[0]), "f32", ROLE_INPUT)
        x = val("x.lp", (batch, dims[0]), cd)
        op("cast", [x_in], [x], kid="cast_v0")
    else:
        x = val("x", (batch, dims[0]), cd, ROLE_INPUT)
    labels = val("labels", (batch,), "i32", ROLE_INPUT)

    # ---- parameters and optimizer state ---------------------------------------------------------
    W, b, Wlp, mW, vW, mb, vb = [], [], [], [], [], [], []
    for i in range(L):
        li = 2 * i  # reference naming: Sequential index of the Linear ("0.W", "2.W", ...)
        # with the fused exchange, whatever the owning rank broadcasts must be mapped by the peers: the working
        # copy of a matrix (or the matrix itself in fp32 mode) and the bias
        W.append(val(f"{li}.W", (dims[i + 1], dims[i]), "f32", ROLE_PARAM, peer=fused_dp and not mixed))
        b.append(val(f"{li}.b", (dims[i + 1],), "f32", ROLE_PARAM, peer=fused_dp))
        Wlp.append(val(f"{li}.W.lp", (dims[i + 1], dims[i]), cd, ROLE_STATIC, persistent=True, peer=fused_dp) if mixed else W[-1])
        mW.append(val(f"opt.m.{li}.W", (dims[i + 1], dims[i]), "f32", persistent=True))
        vW.append(val(f"opt.v.{li}.W", (dims[i + 1], dims[i]), "f32", persistent=True))
        mb.append(val(f"opt.m.{li}.b", (dims[i + 1],), "f32", persistent=True))
        vb.append(val(f"opt.v.{li}.b", (dims[i + 1],), "f32", persistent=True))
    step = val("opt.step", (1,), "i32", persistent=True)

    hyper = {"lr": lr, "beta1": beta1, "beta2": beta2, "eps": eps}
    if weight_decay:
        hyper["weight_decay"] = weight_decay
    if fused_dp:  # the optimizer ops are interleaved with the backward pass, so the counter moves first
        op("step_inc", [step], [step], None, "step_inc_v0")

    # ---- forward ---------------------------------------------------------------------------------
    acts = [x]
    for i in range(L):
        last = i == L - 1
        name = "logits" if last else f"relu{i}_out"
        h = val(name, (batch, dims[i + 1]), cd, persistent=last)
        op("gemm_epilogue", [acts[-1], Wlp[i], b[i]], [h],
           {"transB": True, "epilogue": "bias" if last else "bias_relu"}, epi_kid)
        acts.append(h)
    logits = acts[-1]

    # ---- loss ------------------------------------------------------------------------------------
    dlogits = val("d_logits", (batch, dims[-1]), cd)
    loss_row = val("loss_row", (batch,), "f32")
    loss = val("loss", (1,), "f32", persistent=True)
    ce_out = [dlogits, loss_row]
    if with_argmax:
        ce_out.append(val("argmax", (batch,), "i32", persistent=True))
    op("softmax_ce", [logits, labels], ce_out, {"scale": 1.0 / gb}, ce_kid)
    op("reduce_mean", [loss_row], [loss], None, "reduce_mean_lastaxis_f32_v0")

    # ---- backward ----------------------------------------------------------------------------------
    dW, db = [None] * L, [None] * L
    dY = dlogits
    for i in reversed(range(L)):
        li = 2 * i
        dW[i] = val(f"d_{li}.W", (dims[i + 1], dims[i]), "f32", peer=fused_dp)
        db[i] = val(f"d_{li}.b", (dims[i + 1],), "f32", peer=fused_dp)
        op("gemm", [dY, acts[i]], [dW[i]], {"transA": True, "transB": False}, gemm_f32out_kid)
        op("reduce_sum", [dY], [db[i]], {"axis": 0, "keepdim": False}, colsum_kid)
        if dp_mode == "nccl":
            op("all_reduce", [dW[i]], [dW[i]], {"bucket": 2 * i}, "all_reduce_nccl_f32_v0")
            op("all_reduce", [db[i]], [db[i]], {"bucket": 2 * i + 1}, "all_reduce_nccl_f32_v0")
        if i > 0:
            dX = val(f"d_relu{i - 1}_out", (batch, dims[i]), cd)
            if fuse_relu_bwd:
                op("gemm_relu_bwd", [dY, Wlp[i], acts[i]], [dX], {"transA": False, "transB": False}, fused_kid)
            else:
                op("gemm", [dY, Wlp[i]], [dX], {"transA": False, "transB": False}, gemm_kid)
                op("relu_bwd", [dX, acts[i]], [dX], None, relu_bwd_kid)  # in place: dX becomes d(pre-activation)
            dY = dX
        if fused_dp:
            # after dX: from here on this rank no longer reads layer i's weights, so peers may overwrite them.
            # No exchange waits for its peers' "done" words by itself: nothing later in the step reads a working
            # copy or rewrites a gradient, so the last exchange of the step (layer 0's bias) is the one fence for all.
            outs = [W[i], mW[i], vW[i]] + ([Wlp[i]] if mixed else [])
            # layer 0's exchange is the last work of the step: no GEMM is left to share the SMs with ("solo")
            op("dp_adam_step", [W[i], dW[i], mW[i], vW[i], step], outs, dict(hyper, slot=2 * i, defer_done=True, solo=(i == 0)),
               "dp_adam_step_f32_p2p_v0")
            fence = {"fence_slots": 2 * L, "solo": True} if i == 0 else {"defer_done": True}
            op("dp_adam_step", [b[i], db[i], mb[i], vb[i], step], [b[i], mb[i], vb[i]], dict(hyper, slot=2 * i + 1, **fence),
               "dp_adam_step_f32_p2p_v0")
    if fused_dp:
        return vals, ops

    # ---- optimizer ---------------------------------------------------------------------------------
    op("step_inc", [step], [step], None, "step_inc_v0")
    if fuse_adam and 2 * L <= 16:
        # one launch for all 2L parameter tensors: inputs [P,G,M,V] per tensor then the step counter; outputs
        # [P,M,V(,working copy)] per tensor
        ins, outs, mask = [], [], 0
        for t, (P, G, Mo, Vo, lp) in enumerate([(W[i], dW[i], mW[i], vW[i], Wlp[i] if mixed else None) for i in range(L)] +
                                               [(b[i], db[i], mb[i], vb[i], None) for i in range(L)]):
            ins += [P, G, Mo, Vo]
            outs += [P, Mo, Vo] + ([lp] if lp is not None else [])
            mask |= (1 << t) if lp is not None else 0
        op("adam_step", ins + [step], outs, dict(hyper, count=2 * L, lp_mask=mask), "adam_step_f32_multi_v1")
        return vals, ops
    for i in range(L):
        outs = [W[i], mW[i], vW[i]] + ([Wlp[i]] if mixed else [])
        op("adam_step", [W[i], dW[i], mW[i], vW[i], step], outs, hyper, "adam_step_f32_fused_v1")
        op("adam_step", [b[i], db[i], mb[i], vb[i], step], [b[i], mb[i], vb[i]], hyper, "adam_step_f32_fused_v1")
    return vals, ops
