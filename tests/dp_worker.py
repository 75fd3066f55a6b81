"""Child process of tests/test_dp_gpu.py: one rank of a small data-parallel captured MLP on its own GPU."""
import os
import sys
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parents[1]
for p in (REPO, REPO / "ai-compiler-framework_b200" / "python"):
    sys.path.insert(0, str(p))


def main():
    rank, world, port, out_dir, dtype, mode = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5], sys.argv[6]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as td
    import aicf_cuda
    import oracle
    from aicf_cuda import Plan, _C, build_mlp_train_step, dp, f32_to_bf16_bits
    dims, gbatch, steps = [256, 512, 384, 64], 1024, 3
    td.init_process_group("gloo", rank=rank, world_size=world)
    aicf_cuda._lib.check(aicf_cuda.lib.aicf_b200_set_device(rank), "set_device")
    if mode != "fused":
        dp.init_from_torch_distributed()
    lo, hi = dp.shard_rows(gbatch, rank, world)
    vals, low = build_mlp_train_step(hi - lo, dims, compute_dtype=dtype, global_batch=gbatch, data_parallel=mode)
    plan = Plan(f"dp_rank{rank}", vals, low)
    if mode == "fused":
        dp.connect_plans_torch([plan])
    params = oracle.mlp_params(dims, seed=4)
    x, y = oracle.mlp_batch(gbatch, dims[0], dims[-1], seed=4)
    for v in vals:
        arr = x[lo:hi] if v.name == "x" else y[lo:hi] if v.name == "labels" else params.get(v.name)
        if arr is None and v.name.endswith(".W.lp"):
            arr = params[v.name[:-3]]
        if arr is not None:
            plan.tensor(v.vid).copy_from_host(f32_to_bf16_bits(arr) if v.dtype == "bf16" else arr)
    td.barrier()
    plan.run()          # one eager step (all_reduce on the side stream)
    plan.sync()
    first = dict(dW0_step1=plan.tensor("d_0.W").numpy(), W0_step1=plan.tensor("0.W").numpy(), loss_step1=plan.tensor("loss").numpy())
    plan.capture()      # then captured replays with the NCCL nodes inside the graph
    plan.replay(steps - 1)
    plan.sync()
    np.savez(Path(out_dir) / f"rank{rank}.npz", W0=plan.tensor("0.W").numpy(), W4=plan.tensor("4.W").numpy(),
             b4=plan.tensor("4.b").numpy(), dW0=plan.tensor("d_0.W").numpy(), loss=plan.tensor("loss").numpy(),
             step=plan.tensor("opt.step").numpy(), status=np.array([_C.wait_status()]), **first)
    plan.close()
    td.barrier()
    dp.finalize()
    td.destroy_process_group()


if __name__ == "__main__":
    main()
