"""GPU: the failure path of the tensor-core KNNConv kernels.  A wait that runs out must surface as a status the host
reads (FOVI_ERR_DEVICE_TIMEOUT), with nothing faulted: the same plan then computes correct results.  The wait is made to
run out by a diagnostic launch whose producer issues no loads and whose wait limit is a few thousand attempts."""
import numpy as np
import pytest
import torch

from conftest import kaiming_weight
from oracle import fovi_oracle as oracle

pytestmark = pytest.mark.gpu
FOVI_ERR_DEVICE_TIMEOUT = 6   # include/fovi_b200.h


def _random_tables(rs, n_in, n_out, K, V):
    idx = rs.randint(0, n_in, size=(K, n_out)).astype(np.int64)
    idx[rs.rand(K, n_out) < 0.2] = n_in   # pads
    tap = rs.randint(0, V, size=(n_out, K)).astype(np.int64)
    return idx, tap


# (c_in, c_out, B): the three single-CTA operand modes and the CTA-pair kernel (c_in multiple of 64, B > 128)
@pytest.mark.parametrize("c_in,c_out,B", [(3, 64, 5), (16, 32, 5), (64, 64, 5), (64, 64, 200)])
def test_wait_timeout_is_reported_and_context_survives(c_in, c_out, B):
    from fovi_b200 import ops
    from fovi_b200._lib import FoviError
    rs = np.random.RandomState(c_in + B)
    n_in, n_out, K, V = 300, 120, 9, 9
    idx, tap = _random_tables(rs, n_in, n_out, K, V)
    plan = ops.KnnConvPlan(idx, tap, n_in, V, c_in, c_out)
    assert plan.tc_supported
    x = rs.randn(B, c_in, n_in).astype(np.float32)
    w = kaiming_weight(rs, c_out, c_in, V)
    wt = plan.pack_weights(torch.from_numpy(w).cuda())
    xp = ops.pack_points(torch.from_numpy(x).cuda(), plan)

    plan.selftest_wait_timeout(xp, wt, batch=B)
    with pytest.raises(FoviError) as e:
        plan.check()
    assert e.value.status == FOVI_ERR_DEVICE_TIMEOUT and "wait site" in str(e.value)
    plan.check()                                 # the status word was cleared by the failing check

    y = plan.forward(xp, wt, out_dtype=torch.float32, batch=B)
    plan.check()
    ref = oracle.knnconv_forward(x, idx, tap, V, w)
    y = y.permute(0, 2, 1).cpu().numpy()
    err = np.linalg.norm(y - ref) / np.linalg.norm(ref)
    assert err < 1e-2, err
