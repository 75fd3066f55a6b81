"""Data-parallel captured MLP on 2 GPUs (skipped with fewer): replicas stay bit-identical, the all-reduced
gradient equals the single-device gradient of the whole batch, weights track the oracle."""
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import aicf_cuda
import oracle
from aicf_cuda import build_mlp_train_step

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def shard_bounds(n, rank, world):
    """Element range of a flat tensor owned by `rank` in the fused exchange (4-element packets, contiguous)."""
    packets = (n + 3) // 4
    return min(n, (packets * rank // world) * 4), min(n, (packets * (rank + 1) // world) * 4)


def assemble(parts):
    """Master tensor from the per-rank copies of the fused mode: every rank contributes its own shard."""
    out = np.empty_like(parts[0]).reshape(-1)
    for r, a in enumerate(parts):
        lo, hi = shard_bounds(out.size, r, len(parts))
        out[lo:hi] = a.reshape(-1)[lo:hi]
    return out.reshape(parts[0].shape)


@pytest.mark.parametrize("mode", ["nccl", "fused"])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_two_rank_captured_step(gpu, tmp_path, dtype, mode):
    if aicf_cuda.lib.aicf_b200_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = str(_free_port())
    procs = [subprocess.Popen([sys.executable, str(HERE / "dp_worker.py"), str(r), "2", port, str(tmp_path), dtype, mode])
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    r0, r1 = dict(np.load(tmp_path / "rank0.npz")), dict(np.load(tmp_path / "rank1.npz"))
    if mode == "fused":
        # biases are replicated; matrix masters are sharded (each rank is current inside its own shard); the
        # gradient buffers hold each rank's LOCAL gradient, the oracle's is their sum
        assert np.array_equal(r0["b4"], r1["b4"]), "b4: replicas diverged"
        for k in ("W0", "W4", "W0_step1"):
            r0[k] = r1[k] = assemble([r0[k], r1[k]])
        for k in ("dW0", "dW0_step1"):
            r0[k] = r1[k] = r0[k] + r1[k]
    for k in ("W0", "W4", "b4", "dW0"):
        assert np.array_equal(r0[k], r1[k]), f"{k}: replicas diverged"
    assert int(r0["step"][0]) == 3 and int(r0["status"][0]) == 0 and int(r1["status"][0]) == 0

    dims, gbatch = [256, 512, 384, 64], 1024
    vals, low = build_mlp_train_step(gbatch, dims, compute_dtype=dtype)
    params = oracle.mlp_params(dims, seed=4)
    x, y = oracle.mlp_batch(gbatch, dims[0], dims[-1], seed=4)
    env, dtypes = {}, {}
    for v in vals:
        dtypes[v.vid] = v.dtype
        arr = x if v.name == "x" else y if v.name == "labels" else params.get(v.name)
        if arr is None and v.name.endswith(".W.lp"):
            arr = oracle.cast(params[v.name[:-3]], v.dtype)
        env[v.vid] = np.array(arr, copy=True) if arr is not None else np.zeros(v.shape, np.int32 if v.dtype == "i32" else np.float32)
    by = {v.name: v.vid for v in vals}
    # step 1: the all-reduced gradient equals the whole-batch gradient; the weight update agrees except where a
    # gradient is so close to zero that its sign is rounding noise (Adam's first update is lr * sign(g))
    oracle.run_lowered(low, env, dtypes, np.float64)
    g_tol = 1e-5 if dtype == "f32" else 2e-2
    want = env[by["d_0.W"]]
    assert np.max(np.abs(r0["dW0_step1"] - want)) <= g_tol * np.max(np.abs(want))
    off = np.abs(r0["W0_step1"] - env[by["0.W"]]) > 1e-5 * np.abs(env[by["0.W"]]) + 2e-6
    assert off.mean() <= (1e-3 if dtype == "f32" else 5e-2), f"{off.mean():.2e} of the weights moved the other way"
    assert (r0["loss_step1"][0] + r1["loss_step1"][0]) / 2 == pytest.approx(float(env[by["loss"]][0]), rel=1e-5 if dtype == "f32" else 2e-3)
    # step 3 (two captured replays later): each rank reports the mean loss of its shard
    for _ in range(2):
        oracle.run_lowered(low, env, dtypes, np.float64)
    assert (r0["loss"][0] + r1["loss"][0]) / 2 == pytest.approx(float(env[by["loss"]][0]), rel=1e-3 if dtype == "f32" else 2e-2)


# ---- the exchange arithmetic for every world size, on ONE GPU ----------------------------------------------------------
def _exchange_plan(shape, world_bias_len):
    from aicf_cuda import Plan, ValueSpec
    from aicf_cuda.plan import ROLE_PARAM, ROLE_STATIC
    nb = world_bias_len
    vals = [ValueSpec(0, "0.W", shape, "f32", ROLE_PARAM),
            ValueSpec(1, "d_0.W", shape, "f32", ROLE_STATIC, persistent=True, peer_visible=True),
            ValueSpec(2, "opt.m.0.W", shape, "f32", persistent=True), ValueSpec(3, "opt.v.0.W", shape, "f32", persistent=True),
            ValueSpec(4, "opt.step", (1,), "i32", persistent=True),
            ValueSpec(5, "0.W.lp", shape, "bf16", ROLE_STATIC, persistent=True, peer_visible=True),
            ValueSpec(6, "0.b", (nb,), "f32", ROLE_PARAM, peer_visible=True),
            ValueSpec(7, "d_0.b", (nb,), "f32", ROLE_STATIC, persistent=True, peer_visible=True),
            ValueSpec(8, "opt.m.0.b", (nb,), "f32", persistent=True), ValueSpec(9, "opt.v.0.b", (nb,), "f32", persistent=True)]
    hyper = {"lr": 1e-2, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8, "weight_decay": 0.01}
    low = [{"op": "dp_adam_step", "inputs": [0, 1, 2, 3, 4], "outputs": [0, 2, 3, 5], "attrs": dict(hyper, slot=0, defer_done=True),
            "kernel_id": "dp_adam_step_f32_p2p_v0"},
           {"op": "dp_adam_step", "inputs": [6, 7, 8, 9, 4], "outputs": [6, 8, 9], "attrs": dict(hyper, slot=1, fence_slots=2),
            "kernel_id": "dp_adam_step_f32_p2p_v0"}]
    return Plan("exchange_math", vals, low), hyper


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (3, 1), (4, 0), (4, 3), (8, 0), (8, 5), (8, 7)])
def test_exchange_arithmetic_of_one_rank_among_n(gpu, world, rank):
    """One rank of an N-rank exchange run alone: the other ranks' pools are buffers on the same GPU that already
    hold their gradients and whose flags already say "ready" and "done", so the kernel never waits and its whole data
    path (sum of N gradient shards in rank order, Adam on the owned shard, broadcast into all N working copies, the
    unrolled, single-packet and ragged-tail loops of every world size) is checked against the oracle."""
    from aicf_cuda import Tensor, _C, bf16_bits_to_f32
    shape, nb = (3001, 2003), 4099  # element counts that are no multiple of 4 x ranks: shards end on odd packets
    n = shape[0] * shape[1]
    plan, hyper = _exchange_plan(shape, nb)
    pool_bytes = plan.peer_pool_bytes
    peer_vals = ["d_0.W", "0.W.lp", "0.b", "d_0.b"]
    base = min(plan.tensor(v).ptr for v in peer_vals) - 8192   # the pool starts with the 8 KiB control block
    off = {v: plan.tensor(v).ptr - base for v in peer_vals}
    pools = [None if k == rank else Tensor.zeros((pool_bytes // 4,), "f32") for k in range(world)]
    plan.open_peers_raw(rank, world, [0 if q is None else q.ptr for q in pools])
    at = lambda k, name, count, dt="f32": Tensor((count,), dt, ptr=(base if k == rank else pools[k].ptr) + off[name])

    rng = np.random.default_rng(100 * world + rank)
    p = (rng.standard_normal(n) * 0.02).astype(np.float32)
    pb = (rng.standard_normal(nb) * 0.02).astype(np.float32)
    gW = [(rng.standard_normal(n) * 1e-3).astype(np.float32) for _ in range(world)]
    gB = [(rng.standard_normal(nb) * 1e-3).astype(np.float32) for _ in range(world)]
    plan.tensor("0.W").copy_from_host(p.reshape(shape))
    plan.tensor("0.b").copy_from_host(pb)
    for k in range(world):
        at(k, "d_0.W", n).copy_from_host(gW[k])
        at(k, "d_0.b", nb).copy_from_host(gB[k])
    F = np.float32
    m = v = mb = vb = 0.0
    for step in (1, 2):
        plan.tensor("opt.step").copy_from_host(np.array([step], np.int32))
        # slots 0 and 1, phases ready and done, every rank: "arrived at epoch `step`"
        Tensor((32,), "i32", ptr=base).copy_from_host(np.full(32, step, np.int32))
        plan.run()
        plan.sync()
        assert _C.wait_status() == 0
        for name, cnt, par0, grads, mom in (("0.W", n, p, gW, (m, v)), ("0.b", nb, pb, gB, (mb, vb))):
            lo, hi = shard_bounds(cnt, rank, world)
            g = grads[0][lo:hi].copy()
            for k in range(1, world):
                g = g + grads[k][lo:hi]   # fp32, rank order, like the kernel
            m0 = mom[0][lo:hi] if isinstance(mom[0], np.ndarray) else 0.0
            v0 = mom[1][lo:hi] if isinstance(mom[1], np.ndarray) else 0.0
            wp, wm, wv = oracle.adam_step_fused(par0[lo:hi], g, m0, v0, step, F(hyper["lr"]), F(0.9), F(0.999), F(1e-8),
                                                weight_decay=F(hyper["weight_decay"]))
            got = plan.tensor(name).numpy().reshape(-1)
            assert np.allclose(got[lo:hi], wp, rtol=1e-5, atol=1e-7), f"{name}: owned shard, step {step}"
            assert np.array_equal(got[:lo], par0[:lo]) and np.array_equal(got[hi:], par0[hi:]), f"{name}: outside the shard"
            gm = plan.tensor("opt.m." + name).numpy().reshape(-1)
            assert np.allclose(gm[lo:hi], wm, rtol=1e-5, atol=1e-9) and not gm[:lo].any() and not gm[hi:].any()
            for k in range(world):   # the broadcast reached every rank's copy, and only inside the shard
                if name == "0.W":
                    lp = bf16_bits_to_f32(at(k, "0.W.lp", cnt, "bf16").numpy())
                    assert np.array_equal(lp[lo:hi], oracle.bf16_round(got[lo:hi])), f"working copy of rank {k}"
                    assert not lp[:lo].any() and not lp[hi:].any()
                elif k != rank:
                    cp = at(k, "0.b", cnt).numpy()
                    assert np.array_equal(cp[lo:hi], got[lo:hi]) and not cp[:lo].any() and not cp[hi:].any()
            # carry the state of the owned shard into the next step
            full_m, full_v = np.zeros(cnt, np.float32), np.zeros(cnt, np.float32)
            full_m[lo:hi], full_v[lo:hi] = gm[lo:hi], plan.tensor("opt.v." + name).numpy().reshape(-1)[lo:hi]
            new_p = par0.copy()
            new_p[lo:hi] = got[lo:hi]
            if name == "0.W":
                p, m, v = new_p, full_m, full_v
            else:
                pb, mb, vb = new_p, full_m, full_v
        for k in range(world):       # both phases of both slots were announced to every rank
            if k != rank:
                flags = Tensor((32,), "i32", ptr=pools[k].ptr).numpy().reshape(2, 2, 8)
                assert (flags[:, :, rank] == step).all(), f"flags in rank {k}'s pool after step {step}"
    plan.close()
