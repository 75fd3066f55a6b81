"""Data-parallel host logic on CPU: two gloo ranks execute the data-parallel lowered graph with the NumPy
interpreter on their shards (all_reduce = gloo sum) and must reproduce the single-process run on the whole
batch. Checks the sharding rule, the 1/global-batch loss scale and the placement of all_reduce ops."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _env_for(vals, params, x, y):
    import oracle
    env, dtypes = {}, {}
    for v in vals:
        dtypes[v.vid] = v.dtype
        if v.name == "x":
            env[v.vid] = x
        elif v.name == "labels":
            env[v.vid] = y
        elif v.name in params:
            env[v.vid] = params[v.name].copy()
        else:
            env[v.vid] = np.zeros(v.shape, np.int32 if v.dtype == "i32" else np.float32)
    return env, dtypes


DIMS, GLOBAL_BATCH, STEPS = [32, 48, 10], 64, 3


def _worker(rank: int, world: int, port: int, out_dir: str, mode):
    for p in (REPO, REPO / "ai-compiler-framework_b200" / "python"):
        sys.path.insert(0, str(p))
    import torch
    import torch.distributed as td
    import oracle
    from aicf_cuda import build_mlp_train_step
    from aicf_cuda.dp import shard_rows
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    td.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = shard_rows(GLOBAL_BATCH, rank, world)
    vals, low = build_mlp_train_step(hi - lo, DIMS, compute_dtype="f32", global_batch=GLOBAL_BATCH, data_parallel=mode)
    x, y = oracle.mlp_batch(GLOBAL_BATCH, DIMS[0], DIMS[-1], seed=4)
    env, dtypes = _env_for(vals, oracle.mlp_params(DIMS, seed=4), x[lo:hi], y[lo:hi])

    def world_sum(vid, local):  # gloo sums in rank order for two ranks
        t = torch.from_numpy(np.array(local, dtype=np.float64))
        td.all_reduce(t)
        return t.numpy()

    for _ in range(STEPS):
        oracle.run_lowered(low, env, dtypes, np.float64, world_grads=world_sum)
    by = {v.name: v.vid for v in vals}
    np.savez(Path(out_dir) / f"rank{rank}.npz", W0=env[by["0.W"]], W2=env[by["2.W"]], b2=env[by["2.b"]], loss=env[by["loss"]])
    td.destroy_process_group()


@pytest.mark.parametrize("mode", ["nccl", "fused"])
def test_two_gloo_ranks_reproduce_the_single_process_step(tmp_path, mode):
    import torch.multiprocessing as mp
    import oracle
    from aicf_cuda import build_mlp_train_step
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path), mode), nprocs=2, join=True)
    vals, low = build_mlp_train_step(GLOBAL_BATCH, DIMS, compute_dtype="f32")
    x, y = oracle.mlp_batch(GLOBAL_BATCH, DIMS[0], DIMS[-1], seed=4)
    env, dtypes = _env_for(vals, oracle.mlp_params(DIMS, seed=4), x, y)
    for _ in range(STEPS):
        oracle.run_lowered(low, env, dtypes, np.float64)
    by = {v.name: v.vid for v in vals}
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    for k, name in (("W0", "0.W"), ("W2", "2.W"), ("b2", "2.b")):
        assert np.array_equal(r0[k], r1[k]), "replicas must stay identical"
        assert np.allclose(r0[k], env[by[name]], rtol=1e-5, atol=1e-7), name
    # each rank reports the mean loss of its shard; their average is the global mean
    assert (r0["loss"][0] + r1["loss"][0]) / 2 == pytest.approx(float(env[by["loss"]][0]), rel=1e-5)


def test_sharding_rule_and_lowering_shape():
    from aicf_cuda import build_mlp_train_step
    from aicf_cuda.dp import loss_scale, shard_rows
    assert [shard_rows(65536, r, 8) for r in (0, 7)] == [(0, 8192), (57344, 65536)]
    with pytest.raises(ValueError):
        shard_rows(10, 0, 3)
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)
    assert loss_scale(65536) == 1.0 / 65536
    vals, low = build_mlp_train_step(8192, [8192] * 5 + [1000], compute_dtype="bf16", global_batch=65536, data_parallel=True)
    names = [it["op"] for it in low]
    assert names.count("all_reduce") == 10 and names.count("gemm") == 5 and names.count("gemm_relu_bwd") == 4
    assert names.count("gemm_epilogue") == 5 and "relu_bwd" not in names
    # every all_reduce sits after the op that produces its gradient and before the Adam that consumes it
    for i, it in enumerate(low):
        if it["op"] == "all_reduce":
            g = it["inputs"][0]
            producer = max(j for j, o in enumerate(low[:i]) if g in o["outputs"] and o["op"] != "all_reduce")
            consumer = min(j for j, o in enumerate(low) if o["op"] == "adam_step" and g in o["inputs"])
            assert producer < i < consumer
    fv, fl = build_mlp_train_step(8192, [8192] * 5 + [1000], compute_dtype="bf16", global_batch=65536, data_parallel="fused")
    fnames = [it["op"] for it in fl]
    assert fnames.count("dp_adam_step") == 10 and "all_reduce" not in fnames and "adam_step" not in fnames
    assert fnames.index("step_inc") < fnames.index("gemm_epilogue"), "the step counter moves before the interleaved updates"
    for i, it in enumerate(fl):  # a layer's exchange starts only after that layer's dX: peers may then overwrite its weights
        if it["op"] == "dp_adam_step" and len(it["outputs"]) == 4:
            lp = it["outputs"][3]
            readers = [j for j, o in enumerate(fl) if lp in o["inputs"] and o["op"] != "dp_adam_step"]
            assert max(readers) < i
    assert sorted(it["attrs"]["slot"] for it in fl if it["op"] == "dp_adam_step") == list(range(10))
    peer = {v.name for v in fv if v.peer_visible}
    assert {"0.W.lp", "0.b", "d_0.W", "d_0.b"} <= peer and "0.W" not in peer and "x" not in peer
    ce = next(it for it in low if it["op"] == "softmax_ce")
    assert ce["attrs"]["scale"] == 1.0 / 65536
    params = sum(int(np.prod(v.shape)) for v in vals if v.role == 1)
    assert params == 276_661_224


# ---- bench.py host logic: every N trains on the same global batch; the host arm is a fraction of one step ----------------
def test_bench_shards_are_slices_of_one_global_batch():
    import bench
    gb, d, classes = 64, 24, 10
    full_x, full_y = np.empty((gb, d), np.float32), np.empty(gb, np.int32)
    bench.fill_global_batch_rows(full_x, full_y, 0, gb, classes)
    assert full_y.min() >= 0 and full_y.max() < classes and abs(float(full_x.mean())) < 0.2
    for world in (2, 4, 8):
        b = gb // world
        for r in range(world):
            x, y = np.empty((b, d), np.float32), np.empty(b, np.int32)
            bench.fill_global_batch_rows(x, y, r * b, gb, classes)
            assert np.array_equal(x, full_x[r * b:(r + 1) * b]) and np.array_equal(y, full_y[r * b:(r + 1) * b]), (world, r)


def test_bench_host_arm_runs_a_fraction_of_a_step_without_the_cuda_library():
    import subprocess
    import sys
    code = (
        "import sys, json; sys.argv=['bench.py']; import bench\n"
        "bench.MLP_DIMS, bench.MLP_GLOBAL_BATCH = [32, 48, 16], 4096\n"
        "s = bench.CpuMlpSample(bench.MLP_DIMS, 512, bench.MLP_GLOBAL_BATCH)\n"
        "t = s.step(); assert t > 0\n"
        "want = sum(max(1, round(r * 512 / 4096)) * c for r, c in ((48, 32), (16, 48))) + sum(max(1, round(n * 512 / 4096)) for n in (48, 16))\n"
        "assert s.opt_elements == want, (s.opt_elements, want)\n"
        "assert not [l for l in open('/proc/self/maps') if 'libaicf_b200' in l], 'the host arm must not map the CUDA library'\n"
        "a, b = bench.mlp_config([8, 4], 64, 2, 'fused', False), bench.mlp_config([8, 4], 64, 2, 'fused', False)\n"
        "assert a == b and a['per_gpu_batch'] == 32\n"
        "print('HOST_ARM_OK')\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(REPO), timeout=300)
    assert r.returncode == 0 and "HOST_ARM_OK" in r.stdout, r.stdout + r.stderr


# ------------------------------------------------------------------ host placement (fake sysfs, no GPU)
def _fake_sysfs(tmp_path, bus_id="0000:1b:00.0", node="1", cpulists=("0-3", "4-7")):
    d = tmp_path / "bus" / "pci" / "devices" / bus_id
    d.mkdir(parents=True)
    (d / "numa_node").write_text(node + "\n")
    for i, cl in enumerate(cpulists):
        n = tmp_path / "devices" / "system" / "node" / f"node{i}"
        n.mkdir(parents=True)
        (n / "cpulist").write_text(cl + "\n")
    return tmp_path


def test_cpulist_parsing():
    from aicf_cuda import hostmem
    assert hostmem.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert hostmem.parse_cpulist("") == []
    assert hostmem.parse_cpulist("5") == [5]
    with pytest.raises(ValueError):
        hostmem.parse_cpulist("7-3")


def test_rank_is_bound_to_the_cpus_of_its_gpus_node(tmp_path, monkeypatch):
    from aicf_cuda import hostmem
    monkeypatch.delenv("AICF_HOST_AFFINITY", raising=False)
    sysfs = _fake_sysfs(tmp_path)
    calls = []
    info = hostmem.bind_to_device_node(3, bus_id="0000:1B:00.0", sysfs=sysfs, setaffinity=lambda pid, cpus: calls.append((pid, list(cpus))),
                                       allowed={0, 1, 4, 5, 6})
    assert info["bound"] and info["numa_node"] == 1 and info["cpus"] == 3
    assert calls == [(0, [4, 5, 6])]  # node 1's CPUs, minus the one the process may not use


def test_binding_declines_and_says_why(tmp_path, monkeypatch):
    from aicf_cuda import hostmem
    monkeypatch.delenv("AICF_HOST_AFFINITY", raising=False)
    never = lambda pid, cpus: pytest.fail("must not bind")
    # the host reports no node (-1)
    info = hostmem.bind_to_device_node(0, bus_id="0000:1b:00.0", sysfs=_fake_sysfs(tmp_path / "a", node="-1"), setaffinity=never,
                                       allowed={0, 1})
    assert not info["bound"] and "no NUMA node" in info["why_not"]
    # unknown device address
    info = hostmem.bind_to_device_node(0, bus_id="0000:ff:00.0", sysfs=_fake_sysfs(tmp_path / "b"), setaffinity=never, allowed={0})
    assert not info["bound"] and "no NUMA node" in info["why_not"]
    # none of the node's CPUs is allowed (a container's cpuset)
    info = hostmem.bind_to_device_node(0, bus_id="0000:1b:00.0", sysfs=_fake_sysfs(tmp_path / "c"), setaffinity=never, allowed={0, 1})
    assert not info["bound"] and "no CPU" in info["why_not"]
    # switched off
    monkeypatch.setenv("AICF_HOST_AFFINITY", "0")
    info = hostmem.bind_to_device_node(0, bus_id="0000:1b:00.0", sysfs=_fake_sysfs(tmp_path / "d"), setaffinity=never, allowed={4})
    assert not info["bound"] and info["why_not"] == "AICF_HOST_AFFINITY=0"
