"""GPU: the allocation-free KNNConv entry point.

`fovi_knnconv_forward_bcn_static` serves callers that may not allocate device memory where they
run a layer (a serving or real-time loop whose memory was fixed at start-up, a plug-in callback
whose host owns the allocator): the repacked activations live in a 32 MiB array inside the library
instead of a buffer obtained from an allocator.  This file is collected last on purpose, so a run
that stops at the first failure has already been through every other test.

Checked here, calling through the C ABI with raw pointers: the result equals the ordinary entry
points' (fovi_pack_points + fovi_knnconv_forward) on two calls in a row with different inputs and
batch sizes (the array is reused and keeps the previous call's contents), for both input layouts a
plan can ask for, and a batch too large for the array is refused with a clear message.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import synth_images, kaiming_weight
from oracle import fovi_oracle as oracle

pytestmark = pytest.mark.gpu


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _static_forward(lib, plan, x, wt, bias, relu):
    B = x.shape[0]
    y = torch.empty((B, plan.n_out, plan.c_out), dtype=torch.float32, device="cuda")
    rc = lib.fovi_knnconv_forward_bcn_static(plan._h, C.c_void_p(x.data_ptr()), 0, C.c_void_p(wt.data_ptr()),
                                             C.c_void_p(bias.data_ptr()), C.c_void_p(y.data_ptr()), 0, B, int(relu), _stream())
    assert rc == 0, (rc, lib.fovi_last_cuda_error())
    return y


def _check_two_calls(ops, lib, plan, w, c_in, n_in, batches, tables):
    wt = plan.pack_weights(torch.from_numpy(w).cuda())
    bias = torch.from_numpy(np.random.RandomState(9).standard_normal(plan.c_out).astype(np.float32)).cuda()
    for call, B in enumerate(batches):
        x = torch.from_numpy(synth_images(20 + call, (B, c_in, n_in)) - np.float32(0.5)).cuda()
        want = plan.forward(ops.pack_points(x, plan), wt, bias, relu=True, out_dtype=torch.float32, batch=B)
        got = _static_forward(lib, plan, x, wt, bias, relu=True)
        plan.check()
        # same kernels on the same packed values: identical bits (tolerance of the other tests: 1e-2 rel-L2)
        assert torch.equal(got, want), (call, float((got - want).abs().max()))
        # ... and the oracle on the same bf16-rounded operands (first rows; the tensor-core tests' bar)
        r = min(B, 2)
        xr = x[:r].to(torch.bfloat16).float().cpu().numpy()
        wr = torch.from_numpy(w).to(torch.bfloat16).float().numpy()
        ref = oracle.knnconv_forward_closed_form(xr, tables[0], tables[1].astype(np.int64), plan.V, wr, bias.cpu().numpy(), relu=True)
        assert np.abs(got[:r].permute(0, 2, 1).cpu().numpy() - ref).max() < 2e-3 * max(1.0, np.abs(ref).max())


def test_static_scratch_matches_regular_entry_points(golden):
    from fovi_b200 import ops
    from fovi_b200._lib import lib
    assert lib.fovi_static_scratch_bytes() == 32 << 20
    # pair layout (c_in = 3): ragged batch first, then a larger one that reuses and overwrites the array
    g = golden("config1.npz")
    V, n_in = int(g["V"]), int(g["n_in"])
    plan = ops.KnnConvPlan(g["knn_idx_pad"], g["tap"], n_in, V, 3, 64, group=1)   # the C entry point under test takes the plain plan
    _check_two_calls(ops, lib, plan, kaiming_weight(np.random.RandomState(1), 64, 3, V), 3, n_in, (5, 130), (g["knn_idx_pad"], g["tap"]))
    # channels-last layout (c_in = 64)
    t = golden("config3_tables.npz")
    V = int(t["l1_V"])
    plan = ops.KnnConvPlan(t["l1_knn_idx_pad"], t["l1_tap"], 1023, V, 64, 192)
    _check_two_calls(ops, lib, plan, kaiming_weight(np.random.RandomState(2), 192, 64, V), 64, 1023, (3, 2), (t["l1_knn_idx_pad"], t["l1_tap"]))


def test_static_scratch_rejects_oversized_batch(golden):
    from fovi_b200 import ops
    from fovi_b200._lib import lib
    t = golden("config3_tables.npz")
    plan = ops.KnnConvPlan(t["l1_knn_idx_pad"], t["l1_tap"], 1023, int(t["l1_V"]), 64, 192)
    B = (32 << 20) // (1023 * 64 * 2) + 1                   # one image more than the array holds
    dummy = torch.zeros(16, device="cuda")
    rc = lib.fovi_knnconv_forward_bcn_static(plan._h, C.c_void_p(dummy.data_ptr()), 0, C.c_void_p(dummy.data_ptr()), None,
                                             C.c_void_p(dummy.data_ptr()), 0, B, 0, _stream())
    assert rc == 2
    assert b"static scratch holds" in lib.fovi_last_cuda_error()
