"""GPU: blk_softmax_noalloc, the softmax entry point that performs no device
allocation, against the plan-based entry point (blk_softmax_run).

It exists for hosts that cannot call cudaMalloc when they need the operator --
a runtime that owns all device memory through its own arena, a plugin inside
someone else's pool, a caller that must not stall other streams (cudaMalloc
and cudaFree synchronise the device).  The chunk table lives in a fixed device array that all calls
share and that keeps the previous call's contents, so the test makes two calls
in a row with different batches and checks each against the plan path.

Collected last (file name) so that a run stopping at the first failure has
already run every other test; it also passes alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import O, assert_probs_close
from blockedattention_b200 import _lib as L
from blockedattention_b200.plan import SoftmaxPlan, dtype_code

pytestmark = pytest.mark.gpu


def call_noalloc(x, out, rows, cols, H, scale=1.0):
    rows = np.ascontiguousarray(rows, np.int64); cols = np.ascontiguousarray(cols, np.int64)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        return L.lib.blk_softmax_noalloc(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), L.i64(rows), L.i64(cols),
                                         len(rows), H, dtype_code(x.dtype), C.c_float(scale), C.c_void_p(stream))


def test_noalloc_matches_plan_path_on_two_calls_in_a_row(cuda_device):
    dev = cuda_device
    batches = [
        (torch.float16, 3, [37, 11, 300, 5], [25, 3, 33, 2047], 1.0),     # first call sets the table up
        (torch.bfloat16, 2, [8, 200], [9000, 64], 0.5),                   # shorter table over the stale one
        (torch.float32, 5, [64, 1, 0, 33], [64, 1, 7, 99], 2.0),
    ]
    for dtype, H, rows, cols, scale in batches:
        D = int((np.asarray(rows) * np.asarray(cols)).sum())
        g = torch.Generator().manual_seed(D)
        X = torch.randn((H, D), generator=g).to(dtype)
        x = X.to(dev)
        ref = SoftmaxPlan(rows, cols, H, dtype, device=dev).run(x, scale=scale)
        out = torch.full_like(x, float("nan"))
        assert call_noalloc(x, out, rows, cols, H, scale) == L.BLK_OK, L.lib.blk_last_error()
        torch.cuda.synchronize()
        # the plan path runs the pipelined kernel, this entry point the one-window-per-CTA kernel: same fp32
        # arithmetic up to the order of the row sums, so results agree to a unit in the last place
        ulp = {torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7, torch.float32: 2.0 ** -21}[dtype]
        assert float((out.float() - ref.float()).abs().max()) <= ulp
        assert_probs_close(out, O.block_softmax(X, rows, cols, scale=scale), "no-alloc vs oracle")
        # in place as well; by now the module is loaded and the table's address resolved, so the device's free
        # memory as the driver reports it (cudaMemGetInfo sees every allocation of the process, the library's
        # own included, unlike torch's allocator statistics) must not move across the call
        free_before = torch.cuda.mem_get_info(dev)[0]
        assert call_noalloc(x, x, rows, cols, H, scale) == L.BLK_OK
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before, "the call changed the device's free memory"
        assert torch.equal(x, out), "in place gives the same bits as out of place"


def test_noalloc_rejects_what_it_cannot_hold(cuda_device):
    dev = cuda_device
    x = torch.zeros((1, 16), dtype=torch.float16, device=dev)
    # 70000 one-row blocks of rows longer than a chunk: more chunks than the built-in table holds
    rows = np.ones(70000, np.int64); cols = np.full(70000, 9000, np.int64)
    rc = call_noalloc(x, x, rows, cols, 1)
    assert rc == L.BLK_ERR_UNSUPPORTED and b"65536" in L.lib.blk_last_error()
    assert call_noalloc(x, x, [-1], [4], 1) == L.BLK_ERR_INVALID
    assert call_noalloc(x, x, [], [], 1) == L.BLK_OK           # empty batch: nothing to do


def test_noalloc_refuses_a_capturing_stream(cuda_device):
    # its table comes from temporary host memory, so a recorded call would replay a dangling copy: it must refuse
    # and leave the capture intact
    dev = cuda_device
    rows, cols = [4, 9], [16, 33]
    x = torch.randn((2, 4 * 16 + 9 * 33), device=dev).half()
    out = torch.empty_like(x)
    assert call_noalloc(x, out, rows, cols, 2) == L.BLK_OK          # resolves the table's address outside capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        graph.capture_begin()
        try:
            rc = call_noalloc(x, out, rows, cols, 2)
            msg = L.lib.blk_last_error()
        finally:
            graph.capture_end()
    assert rc == L.BLK_ERR_UNSUPPORTED and b"captured" in msg
    torch.cuda.synchronize()
    want = out.clone()
    assert call_noalloc(x, out, rows, cols, 2) == L.BLK_OK          # still usable afterwards
    torch.cuda.synchronize()
    assert torch.equal(out, want)
