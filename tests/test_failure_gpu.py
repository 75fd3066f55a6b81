"""Failure detection without faulting a GPU: a data-parallel exchange whose peer never shows up must give up
after its bounded wait, report through the status word, leave the device usable and touch nothing."""
import numpy as np
import pytest

from aicf_cuda import _C, Plan, Tensor, ValueSpec
from aicf_cuda.plan import ROLE_PARAM, ROLE_STATIC

pytestmark = pytest.mark.gpu


def test_dp_exchange_gives_up_when_a_rank_never_arrives(gpu):
    n = 4096
    vals = [ValueSpec(0, "0.b", (n,), "f32", ROLE_PARAM, peer_visible=True),
            ValueSpec(1, "d_0.b", (n,), "f32", ROLE_STATIC, persistent=True, peer_visible=True),
            ValueSpec(2, "opt.m.0.b", (n,), "f32", persistent=True), ValueSpec(3, "opt.v.0.b", (n,), "f32", persistent=True),
            ValueSpec(4, "opt.step", (1,), "i32", persistent=True)]
    low = [{"op": "dp_adam_step", "inputs": [0, 1, 2, 3, 4], "outputs": [0, 2, 3], "attrs": {"lr": 0.1, "slot": 0},
            "kernel_id": "dp_adam_step_f32_p2p_v0"}]
    plan = Plan("lonely_rank", vals, low)
    silent = Tensor.zeros((plan.peer_pool_bytes // 4,), "f32")  # stands in for rank 1's pool: its flags never move
    plan.open_peers_raw(0, 2, [0, silent.ptr])
    p0 = np.linspace(-1, 1, n, dtype=np.float32)
    plan.tensor("0.b").copy_from_host(p0)
    plan.tensor("d_0.b").copy_from_host(np.ones(n, np.float32))
    plan.tensor("opt.step").copy_from_host(np.array([1], np.int32))
    assert _C.wait_status(clear=True) == 0
    plan.run()
    with pytest.raises(RuntimeError, match="exchange expired"):
        plan.sync()  # returns after the two bounded waits (~2 s each), not never, and reports what happened
    status = _C.wait_status(clear=True)
    assert (status >> 17) & 3 == 1, f"status word {status:#x}: the ready-phase timeout must be reported"
    assert np.array_equal(plan.tensor("0.b").numpy(), p0), "work that depended on the missing rank must be skipped"
    assert not silent.numpy()[2048:].any(), "nothing may be written into the absent rank's tensors"
    # the device and the library are still usable
    x = Tensor.from_numpy(np.array([-1.0, 2.0], np.float32))
    _C.launch_by_id("relu_f32_v0", _C.OpKind.EltwiseRelu, [x], [x])
    _C.device_sync()
    assert list(x.numpy()) == [0.0, 2.0] and _C.wait_status() == 0
    plan.close()
