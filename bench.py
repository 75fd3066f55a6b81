#!/usr/bin/env python
"""Benchmark of the op backend + captured-plan hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload mlp|mlp_c1|gemm|gemm_f32|gemm_tf32x3|softmax|ce|reduce|adam|ln_fwd|ln_bwd|stream_mix]
                    [--impl reference] [--small] [--no-check] [--no-kernels]

Default workload `mlp`: the data-parallel captured MLP train step (4x Linear(8192->8192)+ReLU ->
Linear(8192->1000), bf16 GEMMs over fp32 master weights, softmax cross-entropy, fused Adam, global batch
65536 split over the ranks, CUDA-graph replay). One "step" = one replay of the captured graph. Prints ONE
JSON line on rank 0. Under torchrun (N > 1) every rank drives one GPU and takes its contiguous block of rows of the
same 65536-row global batch; gradients are exchanged by the fused dp_adam_step kernel over NVLink peer memory
(`--dp-mode nccl`: NCCL all-reduce nodes inside the graph). At N = 1 the line also carries a `kernels` object: the
other two parts of the metric (GEMM TFLOP/s; softmax / cross-entropy / reduction / Adam HBM GB/s) on the benchmark
shapes, each timed like the single-kernel workloads and, unless `--no-check`, compared with the oracle on a sample
read back outside the timed region.

`--impl reference`: the reference project has no CPU implementation and none of the ops this workload
needs beyond its f16/f32 MLP ops, so the reference arm is the NumPy (fp32) execution of the same
lowered-op graph on the host cores. One timed step of that arm is the fraction b/65536 of a train step: b rows
through forward and backward and the optimizer on the same fraction of every parameter tensor, so that
samples/s = b / time estimates the full step without amortising a full-size optimizer pass over a few rows.

All inputs are seeded synthetic data of the configured shapes and distributions (no dataset).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import struct
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent
for _p in (REPO, REPO / "ai-compiler-framework_b200" / "python"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

MLP_DIMS = [8192, 8192, 8192, 8192, 8192, 1000]
MLP_GLOBAL_BATCH = 65536
SMALL_MLP_DIMS = [2048, 2048, 2048, 1000]
SMALL_MLP_BATCH = 8192
ADAM = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)


# ------------------------------------------------------------------------------------------ helpers
def device_info(lib, device=0):
    """L2 size, SM count and memory size of `device`, for the result line."""
    import ctypes as C
    l2, sms, mem = C.c_int64(0), C.c_int(0), C.c_int64(0)
    if lib.aicf_b200_device_info(int(device), C.byref(l2), C.byref(sms), C.byref(mem)) != 0:
        return {}
    return {"l2_bytes": l2.value, "sm_count": sms.value, "memory_bytes": mem.value}


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.rows: list[list[str]] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, cell in zip(names, r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


class Dist:
    """Control plane for N > 1: torch.distributed (gloo) for the id broadcast, barriers and the max over ranks;
    the data path is the library's own NCCL communicator."""

    def __init__(self, world):
        self.world = world
        self.rank = 0
        self.td = None
        if world > 1:
            import torch.distributed as td
            self.td = td
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            td.init_process_group("gloo")
            self.rank = td.get_rank()

    def barrier(self):
        if self.td:
            self.td.barrier()

    def bcast_bytes(self, b: bytes | None) -> bytes:
        if not self.td:
            return b
        box = [b]
        self.td.broadcast_object_list(box, src=0)
        return box[0]

    def allgather(self, obj):
        if not self.td:
            return [obj]
        out = [None] * self.world
        self.td.all_gather_object(out, obj)
        return out

    def max_float(self, v: float) -> float:
        if not self.td:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        self.td.all_reduce(t, op=self.td.ReduceOp.MAX)
        return float(t[0])

    def close(self):
        if self.td:
            self.td.destroy_process_group()


class Events:
    def __init__(self, lib):
        import ctypes as C
        self.lib, self.C = lib, C
        self.a, self.b = C.c_uint64(), C.c_uint64()
        lib.aicf_b200_event_create(C.byref(self.a))
        lib.aicf_b200_event_create(C.byref(self.b))

    def start(self, stream):
        self.lib.aicf_b200_event_record(self.a.value, stream)

    def stop_ms(self, stream) -> float:
        self.lib.aicf_b200_event_record(self.b.value, stream)
        self.lib.aicf_b200_event_sync(self.b.value)
        ms = self.C.c_float()
        self.lib.aicf_b200_event_elapsed_ms(self.a.value, self.b.value, self.C.byref(ms))
        return float(ms.value)


def pinned_array(lib, shape, dtype, staging=False):
    """A NumPy view of pinned host memory. staging=True: write-combined memory, for a buffer the host only fills and the
    device reads (AICF_BENCH_STAGING=0 keeps it cacheable, to compare)."""
    import ctypes as C
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    p = C.c_void_p()
    if staging and os.environ.get("AICF_BENCH_STAGING", "1") != "0":
        rc = lib.aicf_b200_host_alloc_staging(C.byref(p), n)
    else:
        rc = lib.aicf_b200_host_alloc_pinned(C.byref(p), n)
    if rc != 0:
        raise RuntimeError("pinned host allocation failed")
    buf = (C.c_uint8 * n).from_address(p.value)
    return np.frombuffer(buf, dtype=dtype).reshape(shape), p.value


def fill_normal(dst: np.ndarray, seed: int, scale: float = 1.0, chunk: int = 1 << 23):
    """Fills a (possibly huge) float32 array with N(0, scale): chunk k comes from PCG64 stream [seed, k], chunks are
    drawn by a pool of host threads (the generator releases the GIL), so a gigabyte takes a second, not ten."""
    from concurrent.futures import ThreadPoolExecutor
    flat = dst.reshape(-1)

    def one(k):
        i = k * chunk
        n = min(chunk, flat.size - i)
        np.random.default_rng([seed, k]).standard_normal(n, dtype=np.float32, out=flat[i:i + n])
        if scale != 1.0:
            flat[i:i + n] *= np.float32(scale)

    with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
        list(ex.map(one, range((flat.size + chunk - 1) // chunk)))


N_BLOCKS = 8  # the global batch is seeded in 8 row blocks, so that 1, 2, 4 and 8 ranks train on the same rows


def fill_global_batch_rows(x: np.ndarray, y: np.ndarray, first_row: int, gbatch: int, classes: int):
    """Rows [first_row, first_row + len(x)) of THE global batch: block k (gbatch / 8 rows) is drawn from seed 4000 + k
    (inputs) and 5000 + k (labels), whatever the number of ranks."""
    blk = gbatch // N_BLOCKS
    assert first_row % blk == 0 and x.shape[0] % blk == 0
    for j in range(x.shape[0] // blk):
        k = first_row // blk + j
        fill_normal(x[j * blk:(j + 1) * blk], seed=4000 + k)
        y[j * blk:(j + 1) * blk] = np.random.default_rng(5000 + k).integers(0, classes, size=blk, dtype=np.int32)


# ------------------------------------------------------------------------------------------ MLP workload
def mlp_flops_per_sample(dims):
    fwd = sum(2 * a * b for a, b in zip(dims[:-1], dims[1:]))
    dx = sum(2 * a * b for a, b in zip(dims[1:-1], dims[2:]))
    return fwd + fwd + dx  # forward, dW, dX (no dX for the first layer)


def build_mlp(aicf, dims, batch, global_batch, dp):
    """Two plans over one set of parameters (double-buffered inputs for the end-to-end loop); the
    device-resident timing replays the first one."""
    from aicf_cuda import DoubleBufferedStep, build_mlp_train_step
    vals, low = build_mlp_train_step(batch, dims, compute_dtype="bf16", global_batch=global_batch, data_parallel=dp, **ADAM)
    dbl = DoubleBufferedStep("dp_mlp", vals, low)
    return dbl, dbl.a, vals, low


def init_mlp_params(aicf, plan, dims, seed):
    """He-normal fp32 master weights (same seed on every rank => identical replicas), zero biases; bf16
    working copies made on the device by the cast kernel."""
    from aicf_cuda import _C
    from aicf_cuda._C import OpKind
    rng = np.random.default_rng(seed)
    for i in range(len(dims) - 1):
        w = np.empty((dims[i + 1], dims[i]), np.float32)
        rng.standard_normal(w.size, dtype=np.float32, out=w.reshape(-1))
        w *= np.float32(np.sqrt(2.0 / dims[i]))
        plan.tensor(f"{2 * i}.W").copy_from_host(w)
        _C.launch_by_id("cast_v0", OpKind.Cast, [plan.tensor(f"{2 * i}.W")], [plan.tensor(f"{2 * i}.W.lp")])
    _C.device_sync()


def host_lowering():
    """aicf_cuda's lowering (pure Python) loaded without the package's __init__, which would load the CUDA library:
    the host-only arm must not map libaicf_b200.so."""
    import importlib
    import types
    name = "aicf_cuda_hostonly"
    if name not in sys.modules:
        pkg = types.ModuleType(name)
        pkg.__path__ = [str(REPO / "ai-compiler-framework_b200" / "python" / "aicf_cuda")]
        sys.modules[name] = pkg
    return importlib.import_module(name + ".lowering")


def set_blas_threads():
    """All host cores for the BLAS behind NumPy, whatever OMP_NUM_THREADS says (torchrun exports 1). Returns the
    limiter (keep it alive) and the thread count in force."""
    cores = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        lim = threadpool_limits(limits=cores)
        return lim, max([i.get("num_threads", 1) for i in threadpool_info()] or [1])
    except Exception:
        return None, 1


class CpuMlpSample:
    """The NumPy fp32 port of the train step, cut down to the fraction b/G of one step: forward, loss and backward on
    b of the G rows, and the optimizer ops on the first b/G of the rows of every parameter tensor. Both parts scale
    linearly with the fraction, so b / seconds estimates the samples/s of the full step on these host cores."""

    def __init__(self, dims, b, gbatch):
        import oracle
        self.oracle, self.b, self.gbatch = oracle, b, gbatch
        vals, low = host_lowering().build_mlp_train_step(b, dims, compute_dtype="bf16", global_batch=gbatch, fuse_adam=False, **ADAM)
        params = oracle.mlp_params(dims, seed=4)
        x, y = oracle.mlp_batch(b, dims[0], dims[-1], seed=4)
        self.dtypes = {v.vid: v.dtype for v in vals}
        env = {}
        for v in vals:
            if v.name == "x":
                env[v.vid] = x
            elif v.name == "labels":
                env[v.vid] = y
            elif v.name in params:
                env[v.vid] = params[v.name]
            elif v.name.endswith(".W.lp"):
                env[v.vid] = oracle.cast(params[v.name[:-3]], "bf16")
            else:
                env[v.vid] = np.zeros(v.shape, np.int32 if v.dtype == "i32" else np.float32)
        self.env = env
        opt_names = ("adam_step", "step_inc")
        self.fb_ops = [it for it in low if it["op"] not in opt_names]
        self.opt_ops = [it for it in low if it["op"] in opt_names]
        # optimizer on the leading fraction of every tensor it touches (at least one row)
        frac = b / gbatch
        touched = {v for it in self.opt_ops for v in it["inputs"] + it["outputs"]}
        self.env_opt = {}
        for vid in touched:
            a = env[vid]
            rows = a.shape[0] if a.ndim else 1
            self.env_opt[vid] = a if a.size == 1 else np.ascontiguousarray(a[:max(1, int(round(rows * frac)))])
        self.opt_elements = sum(self.env_opt[it["inputs"][0]].size for it in self.opt_ops if it["op"] == "adam_step")

    def step(self) -> float:
        t0 = time.perf_counter()
        self.oracle.run_lowered(self.fb_ops, self.env, self.dtypes, np.float32)
        self.oracle.run_lowered(self.opt_ops, self.env_opt, self.dtypes, np.float32)
        return time.perf_counter() - t0

    def describe(self, n_timed: int) -> str:
        return (f"{n_timed} timed NumPy fp32 executions of the fraction {self.b}/{self.gbatch} of one step of the same lowered "
                f"graph: {self.b} rows through forward, softmax-CE and backward, Adam on that fraction of every parameter "
                f"tensor ({self.opt_elements} elements); samples/s = {self.b} / seconds")


def mlp_config(dims, gbatch, world, dp_mode, small):
    """The `config` object of the MLP line; the same for this backend's arm and the host arm."""
    return {"workload": "dp_captured_mlp" + ("_small" if small else ""), "layers": dims, "global_batch": gbatch,
            "per_gpu_batch": gbatch // world, "optimizer": "adam", "loss": "softmax_ce", "parallelism": f"dp{world}",
            "gradient_exchange": ("none" if world == 1 else "dp_adam_step over NVLink peer memory" if dp_mode == "fused"
                                  else "NCCL all-reduce"),
            "input_rows": f"rank r takes rows [r*b, (r+1)*b) of one global batch seeded per {gbatch // N_BLOCKS}-row block",
            "l2": "working set (>10 GB per step) far exceeds the 126 MB L2; no flush needed"}


def checksum64(t) -> int:
    """Sum of a device tensor's 32-bit words modulo 2^64: equal on two ranks iff (barring collisions) equal bits."""
    raw = t.numpy()
    return int(np.frombuffer(raw.tobytes(), dtype=np.uint32).sum(dtype=np.uint64))


def run_mlp(args, dist: Dist):
    import aicf_cuda
    lib = aicf_cuda.lib
    rank, local_rank, world = dist.rank, dist_env()[1], dist.world
    dims = SMALL_MLP_DIMS if args.small else MLP_DIMS
    gbatch = SMALL_MLP_BATCH if args.small else MLP_GLOBAL_BATCH
    batch = gbatch // world
    aicf_cuda._lib.check(lib.aicf_b200_set_device(local_rank), "set_device")
    # N > 1: this rank's threads, and the pinned staging buffers allocated below, stay on the NUMA node of its GPU.
    # At N = 1 the process keeps every core (the host arm of the same run uses them all).
    host_affinity = None
    if world > 1:
        from aicf_cuda import hostmem
        host_affinity = hostmem.bind_to_device_node(local_rank)
    if world > 1 and args.dp_mode == "nccl":
        from aicf_cuda import dp
        # NCCL prints its version banner on stdout at communicator creation; stdout carries the one JSON line only,
        # so file descriptor 1 points at stderr while the communicator comes up.
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dp.init_communicator(rank, world, dist.bcast_bytes)
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    dbl, plan, vals, low = build_mlp(aicf_cuda, dims, batch, gbatch, dp=(args.dp_mode if world > 1 else False))
    if world > 1 and args.dp_mode == "fused":
        dbl.connect(rank, world, dist.allgather)
    init_mlp_params(aicf_cuda, plan, dims, seed=4)

    # host inputs in pinned memory: rank r owns rows [r*batch, (r+1)*batch) of the one global batch
    x_host, _ = pinned_array(lib, (batch, dims[0]), np.float32, staging=True)
    y_host, _ = pinned_array(lib, (batch,), np.int32)
    fill_global_batch_rows(x_host, y_host, rank * batch, gbatch, dims[-1])
    x_dev, y_dev, loss_dev = plan.tensor("x"), plan.tensor("labels"), plan.tensor("loss")
    stream = plan.stream
    lib.aicf_b200_memcpy_h2d(x_dev.ptr, x_host.ctypes.data, x_host.nbytes, stream)
    lib.aicf_b200_memcpy_h2d(y_dev.ptr, y_host.ctypes.data, y_host.nbytes, stream)
    plan.sync()

    dbl.capture()
    ev = Events(lib)
    # ---- device-resident timing: K graph replays --------------------------------------------------
    plan.replay(args.warmup)
    plan.sync()
    dist.barrier()
    with ClockSampler(local_rank) as clocks:
        ev.start(stream)
        plan.replay(args.steps)
        ms = ev.stop_ms(stream)
        plan.sync()
    ms_fastest = -dist.max_float(-ms)
    ms = dist.max_float(ms)
    dist.barrier()
    loss_after = float(loss_dev.numpy()[0])
    steps_applied = args.warmup + args.steps

    # ---- checker leg (outside every timed region): the loss node against the logits it was computed from ----
    check = None
    if not args.no_check:
        import oracle
        from aicf_cuda import bf16_bits_to_f32
        z = bf16_bits_to_f32(plan.tensor("logits").numpy()).reshape(batch, dims[-1])
        want = float(np.mean(oracle.softmax_ce(z, y_host)[1])) if batch <= 8192 else float(np.mean(
            [np.mean(oracle.softmax_ce(z[i:i + 8192], y_host[i:i + 8192])[1]) for i in range(0, batch, 8192)]))
        check = {"what": f"mean softmax-CE loss of all {batch} rows recomputed in fp64 from the step's own logits",
                 "device": loss_after, "oracle": want, "ok": bool(abs(loss_after - want) <= 1e-5 * abs(want) + 1e-6)}

    # ---- data-parallel consistency: every replica holds the same weights; the loss is the global one ------
    dp_check = None
    if world > 1:
        names = [f"{2 * i}.W.lp" for i in range(len(dims) - 1)] + [f"{2 * i}.b" for i in range(len(dims) - 1)]
        mine = {"sums": [checksum64(plan.tensor(n)) for n in names], "wait_status": int(aicf_cuda._C.wait_status()), "loss": loss_after}
        every = dist.allgather(mine)
        dp_check = {"replicas_equal": all(e["sums"] == every[0]["sums"] for e in every), "tensors_compared": names,
                    "wait_status": [e["wait_status"] for e in every], "loss_per_rank": [e["loss"] for e in every],
                    "loss_global_mean": float(np.mean([e["loss"] for e in every])), "steps_applied": steps_applied,
                    "note": "loss_global_mean is comparable across N: every N trains on the same 65536 rows from the same "
                            "initial weights, so after the same number of steps it agrees with the N = 1 loss to bf16 accuracy"}

    # ---- end to end: host buffers in, loss out, every step ----------------------------------------------
    # DoubleBufferedStep.submit() = H2D of the step's pinned inputs on a copy stream, one graph replay, D2H of the
    # loss. The loss of step t is read on the host while step t+1 is in flight (one step of pipelining).
    def e2e_run(n):
        prev, last_loss = None, None
        for _ in range(n):
            slot = dbl.submit([x_host, y_host])
            if prev is not None:
                last_loss = float(dbl.result(prev)[0])
            prev = slot
        return float(dbl.result(prev)[0])

    e2e_run(max(2, min(args.warmup, 3)))
    dbl.sync()
    dist.barrier()
    e2e_steps = max(2, min(args.steps, 10))
    t0 = time.perf_counter()
    ev.start(stream)
    e2e_run(e2e_steps)
    e2e_ms = ev.stop_ms(stream)
    dbl.sync()
    e2e_ms = dist.max_float(max(e2e_ms, (time.perf_counter() - t0) * 1e3))
    dist.barrier()

    # ---- per-op device times of one eager step (event pair around every op, same stream) -----------------
    per_op = plan.profile()
    per_op = [a if a < b else b for a, b in zip(per_op, plan.profile())]
    kids = plan.kernel_ids()
    gemm_ms = sum(t for t, k in zip(per_op, kids) if k.startswith("gemm"))
    by_kid: dict[str, float] = {}
    for t, k in zip(per_op, kids):
        by_kid[k] = by_kid.get(k, 0.0) + t
    gemm_flops = mlp_flops_per_sample(dims) * batch
    peaks = measured_peaks()
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    status = aicf_cuda._C.wait_status()
    graph_kernels = int(plan.graph_kernel_nodes)
    dev_info = device_info(lib, local_rank)
    dbl.close()

    out = None
    if rank == 0:
        ms_step = ms / args.steps
        out = {
            "metric": "MLP train-step samples/s (captured graph replay)", "value": gbatch / (ms_step * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": mlp_config(dims, gbatch, world, args.dp_mode, args.small),
            "clocks": clocks.summary(), "device": dev_info,
            "e2e": {"value": gbatch / (e2e_ms / e2e_steps * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": int(x_host.nbytes + y_host.nbytes), "d2h_bytes_per_step": 4, "steps": e2e_steps,
                    "note": "every step: pinned host X (fp32) + labels copied in on a copy stream (double-buffered, overlaps the "
                            "previous replay), one graph replay, loss copied out and read by the host",
                    "host_affinity": host_affinity},
            "gpu_launches": graph_kernels * args.steps,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": None,
                         "kernel": "gemm_tcgen05_2cta_kernel", "peak_source": peaks["source"] + " (sustained cuBLAS bf16)",
                         "note": "algorithmic GEMM FLOPs of one step / summed GEMM op times of one eager step"},
            "phase_ms": {k: round(v, 4) for k, v in sorted(by_kid.items(), key=lambda kv: -kv[1])},
            "loss": loss_after, "steps_applied": steps_applied, "gemm_status": status,
            "ms_per_step_fastest_rank": ms_fastest / args.steps,
        }
        if check is not None:
            out["check"] = check
        if dp_check is not None:
            out["dp_check"] = dp_check
        if world == 1 and not args.no_kernels:
            out["kernels"] = run_kernel_suite(args)
        if world == 1 and not args.no_cpu:
            _lim, threads = set_blas_threads()
            cpu = CpuMlpSample(dims, 256 if args.small else 512, gbatch)
            cpu.step()
            secs = [cpu.step() for _ in range(5)]
            sec = statistics.median(secs)
            out["cpu_baseline"] = {"value": cpu.b / sec, "unit": "samples/s", "cores": threads, "kind": "port",
                                   "sample": cpu.describe(len(secs)), "seconds_per_sample_step": sec}
    return out


def run_mlp_reference(args, world: int):
    """NumPy fp32 execution of the same op graph on the host cores: W + K bounded sample steps (see CpuMlpSample)."""
    _lim, threads = set_blas_threads()
    dims = SMALL_MLP_DIMS if args.small else MLP_DIMS
    gbatch = SMALL_MLP_BATCH if args.small else MLP_GLOBAL_BATCH
    cpu = CpuMlpSample(dims, 256 if args.small else 512, gbatch)
    warm = max(args.warmup, 3)
    t_first = cpu.step()
    # whole run within a few minutes: if a sample step is slower than expected on this host, fewer timed steps
    budget_s = 150.0
    steps = int(max(1, min(args.steps, budget_s // max(t_first, 1e-3) - warm)))
    for _ in range(warm - 1):
        cpu.step()
    secs = [cpu.step() for _ in range(steps)]
    sec = statistics.mean(secs)
    value = cpu.b / sec
    return {"impl": "reference", "metric": "MLP train-step samples/s (captured graph replay)", "value": value, "unit": "samples/s",
            "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": sec * 1e3 * gbatch / cpu.b, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": mlp_config(dims, gbatch, world, args.dp_mode, args.small),
            "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": "port",
                             "sample": cpu.describe(steps) + "; the reference project has no CPU path and lacks bf16, softmax-CE and "
                                       "data parallelism, so the host arm is this port", "seconds_per_sample_step": sec},
            "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "ms_per_step is the sample step scaled to the full 65536-row step (seconds_per_sample_step x 65536 / rows)"}


def run_p2p_probe(args, dist: Dist):
    """Measured ceiling of the peer links for the exchange kernel: the stream probe (16-byte loads / stores, no
    arithmetic to speak of) reading from, and writing to, another rank's memory through the same IPC mappings the
    plans use. Every rank does the same thing at the same time (rank r talks to rank r+1), so each GPU carries one
    stream in and one stream out, as in the exchange. Reports GB/s per GPU and direction, max time over ranks."""
    import ctypes as C
    import aicf_cuda
    from aicf_cuda import Plan, Tensor, ValueSpec, dp
    from aicf_cuda.plan import ROLE_STATIC
    lib = aicf_cuda.lib
    rank, local_rank, world = dist.rank, dist_env()[1], dist.world
    if world < 2:
        raise SystemExit("p2p_probe needs at least 2 ranks (torchrun)")
    aicf_cuda._lib.check(lib.aicf_b200_set_device(local_rank), "set_device")
    n = 1 << 26  # 256 MiB per buffer
    vals = [ValueSpec(0, "window", (n,), "f32", ROLE_STATIC, persistent=True, peer_visible=True),
            ValueSpec(1, "scratch", (4,), "f32", ROLE_STATIC, persistent=True)]
    plan = Plan("p2p_probe", vals, [{"op": "grad_zero", "inputs": [1], "outputs": [1], "attrs": {}, "kernel_id": "grad_zero_v0"}])
    dp.connect_plans([plan], rank, world, dist.allgather)
    off = plan.tensor("window").ptr - plan.peer_pool_base(rank)
    window_of = lambda k: plan.peer_pool_base(k) + off
    local = [Tensor.zeros((n,)) for _ in range(2)]
    ev = Events(lib)

    def timed(reads, writes, ins, outs, in_flight, blocks):
        a = (C.c_void_p * reads)(*ins)
        b = (C.c_void_p * writes)(*outs)
        launch = lambda: aicf_cuda._lib.check(lib.aicf_b200_stream_probe(reads, writes, a, b, 4 * n, in_flight, blocks, 0), "stream_probe")
        for _ in range(3):
            launch()
        lib.aicf_b200_device_sync()
        dist.barrier()
        reps = 20
        ev.start(0)
        for _ in range(reps):
            launch()
        ms = dist.max_float(ev.stop_ms(0)) / reps
        dist.barrier()
        return ms

    right = (rank + 1) % world
    others = [(rank + j) % world for j in range(1, min(world, 5))]
    res = {}
    for in_flight, blocks in ((2, 8), (4, 8), (4, 16)):
        tag = f"inflight{in_flight}_blocks{blocks}"
        ms = timed(1, 1, [window_of(right)], [local[0].ptr], in_flight, blocks)
        res[f"pull_from_one_peer_{tag}"] = 4 * n / ms / 1e6
        ms = timed(1, 1, [local[0].ptr], [window_of(right)], in_flight, blocks)
        res[f"push_to_one_peer_{tag}"] = 4 * n / ms / 1e6
        ms = timed(len(others), 1, [window_of(k) for k in others], [local[0].ptr], in_flight, blocks)
        res[f"pull_from_{len(others)}_peers_{tag}"] = 4 * n * len(others) / ms / 1e6
        ms = timed(1, 1, [local[1].ptr], [local[0].ptr], in_flight, blocks)
        res[f"local_copy_{tag}"] = 2 * 4 * n / ms / 1e6
    plan.close()
    if rank != 0:
        return None
    best = max(v for k, v in res.items() if k.startswith("pull_from"))
    return {"metric": "peer-memory probe GB/s per GPU and direction (NVLink)", "value": best, "unit": "GB/s", "n_gpus": world,
            "steps": 20, "warmup": 3, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": "p2p_probe", "bytes_per_buffer": 4 * n,
                                                               "pattern": "every rank reads from / writes to rank+1 at the same time"},
            "gb_per_s": {k: round(v, 1) for k, v in res.items()}, "gpu_launches": 20 * 12}


def run_mlp_c1(args):
    """BASELINE config 1: fp32 MLP 784->256->10, batch 64, captured replay (launch/latency-bound; reports us/step)."""
    import aicf_cuda
    import oracle
    from aicf_cuda import Plan, _C, build_mlp_train_step
    dims, batch = [784, 256, 10], 64
    vals, low = build_mlp_train_step(batch, dims, compute_dtype="f32", **ADAM)
    plan = Plan("mlp_c1", vals, low)
    for name, w in oracle.mlp_params(dims, seed=0).items():
        plan.tensor(name).copy_from_host(w)
    x, y = oracle.mlp_batch(batch, dims[0], dims[-1], seed=0)
    plan.tensor("x").copy_from_host(x)
    plan.tensor("labels").copy_from_host(y)
    plan.capture()
    ev = Events(aicf_cuda.lib)
    reps = 200
    plan.replay(max(3, args.warmup) * 10)
    plan.sync()
    times = []
    with ClockSampler(0) as clocks:
        for _ in range(args.steps):
            ev.start(plan.stream)
            plan.replay(reps)
            times.append(ev.stop_ms(plan.stream) / reps)
    ms = statistics.mean(times)
    t0 = time.perf_counter()
    env, dtypes = {}, {}
    params = oracle.mlp_params(dims, seed=0)
    for v in vals:
        dtypes[v.vid] = v.dtype
        env[v.vid] = x if v.name == "x" else y if v.name == "labels" else params[v.name].copy() if v.name in params else \
            np.zeros(v.shape, np.int32 if v.dtype == "i32" else np.float32)
    cpu_steps = 50
    t0 = time.perf_counter()
    for _ in range(cpu_steps):
        oracle.run_lowered(low, env, dtypes, np.float32)
    cpu_s = (time.perf_counter() - t0) / cpu_steps
    flops = mlp_flops_per_sample(dims) * batch
    out = {"metric": "small MLP train-step samples/s (captured graph replay)", "value": batch / (ms * 1e-3), "unit": "samples/s",
           "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "us_per_step": ms * 1e3,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": "mlp_784_256_10_batch64", "kernels_per_step": plan.graph_kernel_nodes,
                      "l2": "3.3 MB working set: L2-resident by nature (latency-bound configuration)"},
           "clocks": clocks.summary(), "device": device_info(aicf_cuda.lib), "gpu_launches": plan.graph_kernel_nodes * reps * args.steps,
           "roofline": {"bound": "latency", "achieved": flops / (ms * 1e-3) / 1e12, "peak": None, "unit": "TFLOP/s", "frac": None,
                        "traffic": None, "note": f"{plan.graph_kernel_nodes} dependent kernels per step; time is launch + drain latency"},
           "cpu_baseline": {"value": batch / cpu_s, "unit": "samples/s", "cores": set_blas_threads()[1], "kind": "port",
                            "sample": f"{cpu_steps} NumPy fp32 steps of the same lowered graph (full configuration)"},
           "loss": float(plan.tensor("loss").numpy()[0]), "gemm_status": _C.wait_status()}
    plan.close()
    return out


# ------------------------------------------------------------------------------------------ single-kernel workloads
def _sample_rows(M, k, seed=11):
    edge = [0, 1, M - 2, M - 1]
    return np.unique(np.concatenate([edge, np.random.default_rng(seed).choice(M, size=min(k, M), replace=False)]))


def _verdict(what, err, tol):
    return {"what": what, "max_err": float(err), "tolerance": float(tol), "ok": bool(err <= tol)}


def kernel_case(w, *, small=False, size=0, rows=0, cols=0, dtype="f32", reduce_kind="sum", transb=False, want_check=True,
                probe=(0, 0)):
    """One single-kernel workload on a benchmark shape: device buffers, the launch closure `fn(stream)`, its algorithmic
    work, and `check()`, which reads a sample of the output back and compares it with the oracle (never timed)."""
    import oracle
    from aicf_cuda import _C, Tensor, bf16_bits_to_f32
    from aicf_cuda._C import OpKind
    peaks = measured_peaks()

    def host_normal(shape, scale, seed, dt="f32"):
        h = np.empty(shape, np.float32)
        fill_normal(h, seed, scale)
        return oracle.bf16_round(h) if dt == "bf16" else oracle.f16_round(h) if dt == "f16" else h

    def rows_of(t, sel):
        """Rows `sel` of a 2-D device tensor as float32 (one small copy per row, not the whole tensor)."""
        n = t.shape[1]
        out = np.empty((len(sel), n), np.float32)
        esz = t.nbytes // t.numel
        for j, r in enumerate(sel):
            v = Tensor((n,), t.dtype, ptr=t.ptr + int(r) * n * esz).numpy()
            out[j] = bf16_bits_to_f32(v) if t.dtype == "bf16" else v.astype(np.float32)
        return out

    case = {"check": None, "before": None}
    if w in ("gemm", "gemm_f32", "gemm_tf32x3"):
        n = size or (2048 if small else 8192 if w == "gemm" else 4096)
        dt = "bf16" if w == "gemm" else "f32"
        m = rows or n  # rows = M of a skinny product M x n x n (a small batch against square weights)
        hA, hB = host_normal((m, n), 0.577, 1, dt), host_normal((n, n), 0.577, 2, dt)  # U(-1,1) has sigma 0.577
        hb = host_normal((n,), 1.0, 3)
        A, B, bias = Tensor.from_numpy(hA, dt), Tensor.from_numpy(hB, dt), Tensor.from_numpy(hb)
        Cm = Tensor.empty((m, n), dt)
        kid = {"gemm": "gemm_bias_relu_bf16_tcgen05_out_bf16_v0", "gemm_f32": "gemm_bias_relu_f32_naive_v0",
               "gemm_tf32x3": "gemm_bias_relu_f32_3xtf32_v0"}[w]
        pay = struct.pack("<iii", 0, 1 if transb else 0, 1)
        fn = lambda st: _C.launch_by_id(kid, OpKind.GemmEpilogue, [A, B, bias], [Cm], 0x4750454C, pay, st)
        case.update(work=2.0 * m * n * n, unit="TFLOP/s", bound="tensor", peak=peaks["bf16_tflops"] if w == "gemm" else None,
                    metric=f"GEMM+bias+ReLU {dt} TFLOP/s" + (" (3xTF32 tensor-core path; 2*M*N*K counted once)" if w == "gemm_tf32x3" else ""),
                    cfg={"workload": f"gemm_bias_relu_{dt}" if w != "gemm_tf32x3" else "gemm_bias_relu_3xtf32_f32", "M": m, "N": n, "K": n,
                         "transB": bool(transb), "l2": "operands exceed L2 at 8192; smaller sizes are L2-resident by nature"})

        def check():
            sel = _sample_rows(m, 32)
            want = oracle.gemm_epilogue(hA[sel], hB, hb, False, bool(transb), True)
            err = np.max(np.abs(rows_of(Cm, sel) - want)) / max(np.max(np.abs(want)), 1e-30)
            return _verdict(f"{len(sel)} rows of C against fp64 on the same {dt} inputs, normwise", err, 2e-2 if dt == "bf16" else 1e-5)
        case["check"] = check
    elif w == "softmax":
        M, N = (4096, 4096) if small else (32768, 4096)
        M, N = rows or M, cols or N
        hX = host_normal((M, N), 3.0, 2, dtype)
        X, Y = Tensor.from_numpy(hX, dtype), Tensor.empty((M, N), dtype)
        fn = lambda st: _C.launch_by_id(f"softmax_lastdim_{dtype}_v0", OpKind.Softmax, [X], [Y], 0, b"", st)
        case.update(work=2.0 * X.nbytes, unit="GB/s", bound="hbm", peak=peaks["hbm_gbs"], metric=f"row softmax {dtype} HBM GB/s",
                    cfg={"workload": f"softmax_{dtype}", "rows": M, "cols": N, "l2": "read+write bytes exceed L2"})

        def check():
            sel = _sample_rows(M, 128)
            want, got = oracle.softmax(hX[sel]), rows_of(Y, sel)
            tol = 1e-5 if dtype == "f32" else 8e-3 if dtype == "bf16" else 1e-3
            err = np.max(np.abs(got - want) / (np.abs(want) + 1e-7 / tol))
            return _verdict(f"{len(sel)} rows against the fp64 oracle, relative", err, tol)
        case["check"] = check
    elif w in ("ln_fwd", "ln_bwd"):
        M, N = (4096, 4096) if small else (32768, 4096)
        M, N = rows or M, cols or N
        dt = dtype
        esz = 4 if dt == "f32" else 2
        hX = host_normal((M, N), 2.0, 2, dt)
        hG, hBt = host_normal((N,), 1.0, 3, dt), host_normal((N,), 0.1, 4, dt)
        X, Gm, Bt = Tensor.from_numpy(hX, dt), Tensor.from_numpy(hG, dt), Tensor.from_numpy(hBt, dt)
        Y, Mu, Rs = Tensor.empty((M, N), dt), Tensor.empty((M,), "f32"), Tensor.empty((M,), "f32")
        fwd = lambda st: _C.launch_by_id(f"layernorm_fwd_{dt}_v0", OpKind.LayerNormFwd, [X, Gm, Bt], [Y, Mu, Rs], 0, b"", st)
        if w == "ln_fwd":
            fn = fwd
            work = 2.0 * M * N * esz + 8.0 * M + 2.0 * N * esz

            def check():
                sel = _sample_rows(M, 128)
                want = oracle.layernorm_fwd(hX[sel], hG, hBt, np.float32(1e-5))[0]
                tol = 1e-5 if dt == "f32" else 8e-3 if dt == "bf16" else 1e-3
                err = np.max(np.abs(rows_of(Y, sel) - want) / (np.abs(want) + 1.0))
                return _verdict(f"{len(sel)} rows of y against the fp64 oracle, relative to |y| + 1", err, tol)
            case["check"] = check
        else:
            fwd(0)
            _C.device_sync()
            hdY = host_normal((M, N), 1.0, 5, dt)
            dY = Tensor.from_numpy(hdY, dt)
            dX, dG, dB = Tensor.empty((M, N), dt), Tensor.empty((N,), "f32"), Tensor.empty((N,), "f32")
            fn = lambda st: _C.launch_by_id(f"layernorm_bwd_{dt}_v0", OpKind.LayerNormBwd, [X, dY, Gm, Mu, Rs], [dX, dG, dB], 0, b"", st)
            work = 3.0 * M * N * esz + 8.0 * M + N * esz + 8.0 * N

            def check():
                sel = _sample_rows(M, 128)
                mu, rs = Mu.numpy()[sel], Rs.numpy()[sel]
                want = oracle.layernorm_bwd(hX[sel], hdY[sel], hG, mu, rs)[0]
                tol = 1e-5 if dt == "f32" else 8e-3 if dt == "bf16" else 1e-3
                err = np.max(np.abs(rows_of(dX, sel) - want) / (np.abs(want) + np.abs(want).max()))
                return _verdict(f"{len(sel)} rows of dx against the fp64 oracle, relative to |dx| + max|dx|", err, tol)
            case["check"] = check
        case.update(work=work, unit="GB/s", bound="hbm", peak=peaks["hbm_gbs"],
                    metric=f"layer norm {'forward' if w == 'ln_fwd' else 'backward (dx, dgamma, dbeta)'} {dt} HBM GB/s",
                    cfg={"workload": f"layernorm_{w[3:]}_{dt}", "rows": M, "cols": N, "l2": "read+write bytes exceed L2"})
    elif w == "reduce":
        M, N = (4096, 4096) if small else (32768, 4096)
        M, N = rows or M, cols or N
        hX = host_normal((M, N), 3.0, 2, dtype)
        X, O = Tensor.from_numpy(hX, dtype), Tensor.empty((M,), "f32")
        kid = f"reduce_{reduce_kind}_lastaxis_{dtype}_v0"
        kind = {"sum": OpKind.ReduceSum, "max": OpKind.ReduceMax, "mean": OpKind.ReduceMean}[reduce_kind]
        sch, pay = (0x5253554D, struct.pack("<q", -1)) if reduce_kind == "sum" else (0, b"")
        fn = lambda st: _C.launch_by_id(kid, kind, [X], [O], sch, pay, st)
        case.update(work=float(X.nbytes + 4 * M), unit="GB/s", bound="hbm", peak=peaks["hbm_gbs"],
                    metric=f"last-axis {reduce_kind} {dtype} HBM GB/s",
                    cfg={"workload": f"reduce_{reduce_kind}_{dtype}", "rows": M, "cols": N, "l2": "input exceeds L2"})

        def check():
            sel = _sample_rows(M, 512)
            want = oracle.reduce_lastaxis(hX[sel], reduce_kind)
            l1 = np.abs(hX[sel]).astype(np.float64).sum(axis=1) / (N if reduce_kind == "mean" else 1)
            err = np.max(np.abs(O.numpy()[sel] - want) / (l1 if reduce_kind != "max" else np.abs(want) + 1e-30))
            return _verdict(f"{len(sel)} rows against the fp64 oracle, relative to the row's sum of magnitudes", err, 1e-5)
        case["check"] = check
    elif w == "ce":
        B, Cn = (1024, 32000) if small else (8192, 32000)
        B, Cn = rows or B, cols or Cn
        hZ = host_normal((B, Cn), 2.0, 3)
        hL = np.random.default_rng(1).integers(0, Cn, B, dtype=np.int32)
        Z, L = Tensor.from_numpy(hZ), Tensor.from_numpy(hL)
        D, Lo, Am = Tensor.empty((B, Cn), "f32"), Tensor.empty((B,), "f32"), Tensor.empty((B,), "i32")
        fn = lambda st: _C.launch_by_id("softmax_ce_f32_i32_v0", OpKind.SoftmaxCE, [Z, L], [D, Lo, Am], 0, b"", st)
        case.update(work=2.0 * Z.nbytes + 12.0 * B, unit="GB/s", bound="hbm", peak=peaks["hbm_gbs"],
                    metric="softmax cross-entropy loss+grad f32 HBM GB/s",
                    cfg={"workload": "softmax_ce_f32", "rows": B, "classes": Cn, "l2": "read+write bytes exceed L2"})

        def check():
            sel = _sample_rows(B, 64)
            wd, wl, wa = oracle.softmax_ce(hZ[sel], hL[sel], scale=1.0 / B)
            e_d = np.max(np.abs(rows_of(D, sel) - wd) / (np.abs(wd) + 1e-7))
            e_l = np.max(np.abs(Lo.numpy()[sel] - wl) / (np.abs(wl) + 1e-1))
            exact = bool(np.array_equal(Am.numpy()[sel], wa))
            v = _verdict(f"{len(sel)} rows: gradient and loss against the fp64 oracle (relative), argmax exact", max(e_d, e_l), 1e-5)
            v["ok"] = v["ok"] and exact
            return v
        case["check"] = check
    elif w == "adam":
        n = (1 << 24) if small else (1 << 28)
        hP, hG = host_normal((n,), 0.02, 3), host_normal((n,), 1e-3, 4)
        P, G = Tensor.from_numpy(hP), Tensor.from_numpy(hG)
        M_, V_ = Tensor.zeros((n,)), Tensor.zeros((n,))
        step = Tensor.from_numpy(np.array([1], np.int32))
        pay = struct.pack("<fffffI", 3e-4, 0.9, 0.999, 1e-8, 0.01, 0)

        def fn(st):
            _C.launch_by_id("adam_step_f32_fused_v1", OpKind.AdamStep, [P, G, M_, V_, step], [P, M_, V_], 0x4D414441, pay, st)
        case.update(work=28.0 * n, unit="GB/s", bound="hbm", peak=peaks["hbm_gbs"], metric="fused Adam f32 HBM GB/s",
                    cfg={"workload": "adam_f32_wd", "elements": n, "l2": "7 streams of 1 GiB exceed L2"})

        def check_first_launch():
            """Runs the first launch (t = 1, m = v = 0) and compares 64 slices of 4096 elements of p, m, v."""
            fn(0)
            _C.device_sync()
            f = np.float32
            starts = np.unique(np.concatenate([[0, n - 4096], np.random.default_rng(5).integers(0, n // 4096, 62) * 4096]))
            worst = 0.0
            for s0 in starts:
                sl = slice(int(s0), int(s0) + 4096)
                wp, wm, wv = oracle.adam_step_fused(hP[sl], hG[sl], 0.0, 0.0, 1, f(3e-4), f(0.9), f(0.999), f(1e-8), weight_decay=f(0.01))
                for t, wnt, atol in ((P, wp, 1e-7), (M_, wm, 1e-9), (V_, wv, 1e-13)):
                    got = Tensor((4096,), "f32", ptr=t.ptr + int(s0) * 4).numpy()
                    worst = max(worst, float(np.max(np.abs(got - wnt) / (np.abs(wnt) + atol / 1e-5))))
            return _verdict(f"first step (t = 1): {len(starts)} slices of 4096 elements of p, m, v against the fp64 oracle, relative", worst, 1e-5)
        case["before"] = check_first_launch
    elif w == "stream_mix":
        # the ceiling for a streaming kernel with R input and W output arrays (rows = R, cols = W; default 4 + 3 = Adam's mix)
        import ctypes as C
        import aicf_cuda
        R, Wn = rows or 4, cols or 3
        n = (1 << 24) if small else (1 << 28)
        bufs = [Tensor.zeros((n,)) for _ in range(R + Wn)]
        ins = (C.c_void_p * R)(*[b.ptr for b in bufs[:R]])
        outs = (C.c_void_p * Wn)(*[b.ptr for b in bufs[R:]])

        def fn(st):
            aicf_cuda._lib.check(aicf_cuda.lib.aicf_b200_stream_probe(R, Wn, ins, outs, 4 * n, probe[0], probe[1], st), "stream_probe")
        case.update(work=4.0 * n * (R + Wn), unit="GB/s", bound="hbm", peak=peaks["hbm_gbs"],
                    metric=f"stream-mix probe: {R} arrays read, {Wn} written, HBM GB/s", keep=bufs,
                    cfg={"workload": f"stream_mix_{R}r{Wn}w_f32", "elements": n, "packets_in_flight": probe[0] or 2,
                         "blocks_per_sm": probe[1] or 8, "l2": f"{R + Wn} streams of {4 * n >> 20} MiB exceed L2"})
    else:
        raise SystemExit(f"unknown workload {w}")
    case["fn"] = fn
    if not want_check:
        case["check"] = case["before"] = None
    return case


def time_case(case, steps, warmup, device_index=0):
    """Times `reps` back-to-back launches captured in one CUDA graph (so that host launch latency does not pollute
    short kernels); reps is chosen so a timed region lasts about 2 ms. Returns the fields of a result entry."""
    import aicf_cuda
    from aicf_cuda import _C
    ev = Events(aicf_cuda.lib)
    fn = case["fn"]
    _C.trace_enable(False)
    check = case["before"]() if case.get("before") else None
    for _ in range(max(3, warmup)):
        fn(0)
    _C.device_sync()
    ev.start(0)
    fn(0)
    one = max(ev.stop_ms(0), 1e-3)
    reps = int(min(200, max(1, round(2.0 / one))))
    s = _C.graph_begin()
    for _ in range(reps):
        fn(s)
    _C.graph_end()
    for _ in range(3):
        _C.graph_launch()
    _C.device_sync()
    times = []
    with ClockSampler(device_index) as clocks:
        for _ in range(steps):
            ev.start(s)
            _C.graph_launch()
            times.append(ev.stop_ms(s) / reps)
    _C.graph_reset()
    if case.get("check"):
        check = case["check"]()
    ms = statistics.mean(times)
    achieved = case["work"] / (ms * 1e-3) / (1e12 if case["unit"] == "TFLOP/s" else 1e9)
    return {"ms": ms, "ms_min": min(times), "achieved": achieved, "reps": reps, "clocks": clocks.summary(), "check": check}


def run_kernel_workload(args):
    """GEMM TFLOP/s and softmax / CE / reduce / Adam GB/s on BASELINE's shapes (1 GPU)."""
    import aicf_cuda
    from aicf_cuda import _C
    peaks = measured_peaks()
    case = kernel_case(args.workload, small=args.small, size=args.size, rows=args.rows, cols=args.cols, dtype=args.dtype,
                       reduce_kind=args.reduce_kind, transb=args.transb, want_check=not args.no_check,
                       probe=(args.probe_in_flight, args.probe_blocks))
    r = time_case(case, args.steps, args.warmup)
    cfg = dict(case["cfg"], launches_per_timed_graph=r["reps"])
    out = {"metric": case["metric"], "value": r["achieved"], "unit": case["unit"], "n_gpus": 1, "steps": args.steps,
           "warmup": max(3, args.warmup), "ms_per_step": r["ms"], "ms_min": r["ms_min"], "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": cfg["workload"].split("_")[-1], "data": "synthetic", "config": cfg, "clocks": r["clocks"],
           "device": device_info(aicf_cuda.lib), "gpu_launches": args.steps * r["reps"],
           "roofline": {"bound": case["bound"], "achieved": r["achieved"], "peak": case["peak"], "unit": case["unit"],
                        "frac": (r["achieved"] / case["peak"]) if case["peak"] else None, "traffic": None, "peak_source": peaks["source"]},
           "gemm_status": _C.wait_status()}
    if r["check"] is not None:
        out["check"] = r["check"]
    return out


KERNEL_SUITE = [("gemm_8192_bf16", "gemm", dict(size=8192)), ("gemm_4096_bf16", "gemm", dict(size=4096)),
                ("gemm_1024_bf16", "gemm", dict(size=1024)), ("gemm_4096_f32", "gemm_f32", dict(size=4096)),
                ("softmax_f32", "softmax", dict(dtype="f32")),
                ("softmax_bf16", "softmax", dict(dtype="bf16")), ("softmax_ce_f32", "ce", {}),
                ("reduce_sum_f32", "reduce", dict(dtype="f32", reduce_kind="sum")),
                ("reduce_max_f32", "reduce", dict(dtype="f32", reduce_kind="max")),
                ("reduce_mean_bf16", "reduce", dict(dtype="bf16", reduce_kind="mean")), ("adam_f32_2p28", "adam", {}),
                # measured ceilings for the stream mixes above: 4 arrays read + 3 written (Adam), 1 + 1 (softmax, CE)
                # (launch shapes that measured best in a sweep of 1 / 2 / 4 packets in flight x 4 ... 1024 blocks per SM:
                # the rate keeps rising with the grid until every thread has one or two packets per array)
                ("ceiling_4_reads_3_writes", "stream_mix", dict(rows=4, cols=3, probe=(1, 1024))),
                ("ceiling_1_read_1_write", "stream_mix", dict(rows=1, cols=1, probe=(2, 1024)))]


def run_kernel_suite(args):
    """The other two parts of the metric on the benchmark shapes: name -> {value, unit, frac of the measured peak,
    algorithmic work, ms per launch, clocks during the timed launches, oracle check of a read-back sample}."""
    import gc
    out = {}
    for name, w, kw in KERNEL_SUITE:
        case = kernel_case(w, small=args.small, want_check=not args.no_check, **kw)
        r = time_case(case, steps=5, warmup=3)
        out[name] = {"value": r["achieved"], "unit": case["unit"], "frac": (r["achieved"] / case["peak"]) if case["peak"] else None,
                     "peak": case["peak"], "work": case["work"], "ms": r["ms"], "launches_timed": 5 * r["reps"],
                     "config": case["cfg"], "clocks": r["clocks"], "check": r["check"]}
        del case
        gc.collect()  # device buffers of the case go back before the next one allocates
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mlp")
    ap.add_argument("--small", action="store_true", help="reduced shapes (profiler captures)")
    ap.add_argument("--size", type=int, default=0)
    ap.add_argument("--rows", type=int, default=0, help="row count override for the softmax / ce / reduce / layer-norm workloads; M of the GEMM workloads (M x size x size)")
    ap.add_argument("--cols", type=int, default=0, help="row width override for the same workloads")
    ap.add_argument("--dtype", default="f32")
    ap.add_argument("--reduce-kind", default="sum")
    ap.add_argument("--transb", action="store_true")
    ap.add_argument("--probe-in-flight", type=int, default=0, help="stream_mix: 16-byte packets per array in flight per thread (1, 2, 4)")
    ap.add_argument("--probe-blocks", type=int, default=0, help="stream_mix: 256-thread blocks per SM (1-1024)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed NumPy baseline")
    ap.add_argument("--no-check", action="store_true", help="skip the oracle comparison of read-back samples (never timed)")
    ap.add_argument("--no-kernels", action="store_true", help="N = 1 MLP line without the single-kernel measurements")
    ap.add_argument("--dp-mode", default="fused", choices=["fused", "nccl"],
                    help="N > 1: gradient exchange fused with Adam over peer memory, or NCCL all-reduce + Adam")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    _, _, world = dist_env()
    if args.impl == "reference":
        rank = dist_env()[0]
        if rank != 0:
            return  # only rank 0 measures the host baseline; the others have nothing to do
        out = run_mlp_reference(args, max(world, args.gpus))  # host only: no process group, no CUDA library
        print(json.dumps(out), flush=True)
        return

    if args.workload == "mlp_c1":
        print(json.dumps(run_mlp_c1(args)), flush=True)
        return
    if args.workload not in ("mlp", "p2p_probe"):
        print(json.dumps(run_kernel_workload(args)), flush=True)
        return
    dist = Dist(world)
    try:
        out = run_p2p_probe(args, dist) if args.workload == "p2p_probe" else run_mlp(args, dist)
        if out is not None:
            print(json.dumps(out), flush=True)
    finally:
        dist.close()


if __name__ == "__main__":
    main()
