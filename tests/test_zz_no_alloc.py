"""aicf_b200_colsum_f32_noalloc: the column sum for callers that cannot allocate device memory (its
partial sums live in a fixed array inside the library image). Checked through the C ABI against the
workspace-using entry point it mirrors, on two calls in a row that share the built-in array.

Collected last on purpose (file name): a failure here cannot hide the result of any other test."""
import ctypes as C
import struct

import numpy as np
import pytest

import aicf_cuda
from aicf_cuda import Tensor
from aicf_cuda._C import OpKind
from util import by_id

pytestmark = pytest.mark.gpu
RSUM = 0x5253554D


def noalloc(x: Tensor, out: Tensor, rows: int, cols: int) -> int:
    rc = aicf_cuda.lib.aicf_b200_colsum_f32_noalloc(x.ptr, out.ptr, rows, cols, 0)
    aicf_cuda.lib.aicf_b200_device_sync()
    return rc


def test_matches_the_workspace_entry_point_on_two_calls_in_a_row(gpu):
    rng = np.random.default_rng(17)
    # both shapes split the rows over many blocks, so both really go through the scratch array; the second
    # call uses fewer columns and other data, so stale partials from the first would show up
    for rows, cols in [(8192, 1024), (5000, 520)]:
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        X = Tensor.from_numpy(x)
        want_t, got_t = Tensor.zeros((cols,)), Tensor.from_numpy(np.full(cols, np.nan, np.float32))
        need = aicf_cuda.lib.aicf_b200_query_workspace(b"reduce_sum_keep_lastdim_f32_v0", int(OpKind.ReduceSum),
                                                       aicf_cuda._C_ctypes._build_descs([X], "x")[0], 1, None)
        assert 0 < need <= 512 * 1024, "the case must exercise scratch memory and fit the built-in array"
        by_id("reduce_sum_keep_lastdim_f32_v0", OpKind.ReduceSum, [X], [want_t], RSUM, struct.pack("<q", 0))
        assert noalloc(X, got_t, rows, cols) == 0, aicf_cuda.lib.aicf_b200_last_error().decode()
        got, want = got_t.numpy(), want_t.numpy()
        l1 = np.abs(x).astype(np.float64).sum(axis=0)
        assert (np.abs(got.astype(np.float64) - want) <= 1e-5 * l1).all()          # the suite's reduction tolerance
        assert (np.abs(got.astype(np.float64) - x.astype(np.float64).sum(axis=0)) <= 1e-5 * l1).all()
        assert np.array_equal(got, want), "same kernels, same split, same order: identical bits"


def test_rejects_shapes_beyond_the_built_in_scratch_and_bad_arguments(gpu):
    rows, cols = 4096, 70000  # two row splits x 70000 columns x 4 B = 547 KiB > 512 KiB
    X, O = Tensor.empty((rows, cols)), Tensor.empty((cols,))
    assert noalloc(X, O, rows, cols) == 1
    msg = aicf_cuda.lib.aicf_b200_last_error().decode()
    assert "needs 560000 bytes" in msg and "524288" in msg
    assert noalloc(X, O, 0, cols) == 1
    assert aicf_cuda.lib.aicf_b200_colsum_f32_noalloc(None, O.ptr, 4, 4, 0) == 1


def test_small_inputs_that_need_no_scratch_still_work(gpu):
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    O = Tensor.empty((4,))
    assert noalloc(Tensor.from_numpy(x), O, 3, 4) == 0
    assert np.array_equal(O.numpy(), x.sum(axis=0))
