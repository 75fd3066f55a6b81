"""Host-side logic of the data-parallel MLP step: batch sharding and communicator bootstrap.

One process per GPU. The data path is the library's NCCL communicator (all_reduce ops inside the plan);
torch.distributed - any backend, gloo is enough - is only the control plane that carries the 128-byte
communicator id from rank 0 to the others. The reference has no multi-device code (device hard-wired to 0,
src/python_bindings/bindings.cpp:123), so nothing here mirrors a reference interface.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

from ._lib import check, lib


def shard_rows(global_batch: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [start, stop) of the global batch owned by `rank`: contiguous equal blocks in rank order."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} / world {world}")
    if global_batch % world:
        raise ValueError(f"global batch {global_batch} is not divisible by {world} ranks")
    b = global_batch // world
    return rank * b, (rank + 1) * b


def loss_scale(global_batch: int) -> float:
    """Scale applied to the softmax-CE gradient on every rank: 1/global batch, so that the SUM of the
    shard gradients equals the single-device mean-loss gradient."""
    return 1.0 / float(global_batch)


def init_communicator(rank: int, world: int, bcast_bytes) -> None:
    """Creates the NCCL communicator. `bcast_bytes(b)` must return rank 0's bytes on every rank."""
    if world == 1:
        check(lib.aicf_b200_dp_init(0, 1, None), "dp_init")
        return
    buf = (C.c_uint8 * 128)()
    if rank == 0:
        check(lib.aicf_b200_dp_unique_id(buf), "dp_unique_id")
    uid = bcast_bytes(bytes(buf) if rank == 0 else None)
    if not isinstance(uid, (bytes, bytearray)) or len(uid) != 128:
        raise RuntimeError("communicator id broadcast failed")
    check(lib.aicf_b200_dp_init(rank, world, (C.c_uint8 * 128).from_buffer_copy(uid)), "dp_init")


def init_from_torch_distributed() -> Tuple[int, int]:
    """Bootstrap from an initialised torch.distributed process group; returns (rank, world)."""
    import torch.distributed as td
    rank, world = td.get_rank(), td.get_world_size()

    def bcast(b):
        box = [b]
        td.broadcast_object_list(box, src=0)
        return box[0]

    init_communicator(rank, world, bcast)
    return rank, world


def connect_plans(plans, rank: int, world: int, allgather) -> None:
    """Lets every plan's dp_adam_step ops reach the other ranks' gradient and weight buffers.
    `allgather(obj)` must return the list of every rank's `obj` in rank order (for instance
    torch.distributed.all_gather_object). All ranks must pass their plans in the same order."""
    for plan in plans:
        handles = allgather(plan.peer_handle())
        plan.open_peers(rank, world, handles)


def connect_plans_torch(plans) -> None:
    import torch.distributed as td
    rank, world = td.get_rank(), td.get_world_size()

    def gather(obj):
        out = [None] * world
        td.all_gather_object(out, obj)
        return out

    connect_plans(plans, rank, world, gather)


def finalize() -> None:
    check(lib.aicf_b200_dp_finalize(), "dp_finalize")
