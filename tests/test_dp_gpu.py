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
