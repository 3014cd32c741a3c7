"""A bounded device wait that really runs out, and the recovery afterwards.

Every wait inside the GEMM kernels (on a shared-memory barrier fed by TMA copies or by the tensor core) gives up after a
limited number of polls, raises a status word, lets the other roles of the CTA leave, drains what is in flight, frees its
tensor memory and returns.  mi8_test_wait_fault makes the producer leave out the loads of one pipeline item, so the roles
waiting for those bytes time out - nothing traps, faults or spins for ever.  The test checks what the host sees (the error
contract of the reference is "report and stop", src/common/logging.h:100-140): the launch returns, mi8_poll_status reports
MI8_ERR_DEVICE with a 10x code, and after mi8_workspace_init + mi8_clear_status the next call is bit-exact again."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n,tile", [(48, 512, 384, 0), (200, 1024, 256, 0), (300, 1024, 512, 512)])
def test_wait_runs_out_and_the_library_recovers(cuda_device, oracle, m, k, n, tile):
    from marian_dev_b200 import ops
    from marian_dev_b200.binding import check, lib
    L = lib()
    rng = np.random.default_rng(m + n)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.01).astype(np.float32)
    bt, qb = oracle.prepare_b(w)
    want = oracle.affine(a, bt, qb, bias, 1.0, False)
    aq = ops.prepareA(torch.from_numpy(a).to(cuda_device))
    b = ops.prepareB(torch.from_numpy(w).to(cuda_device))
    bias_t = torch.from_numpy(bias).to(cuda_device)
    ws = ops.default_workspace(cuda_device)
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    try:
        L.mi8_test_wait_fault(1, 1 << 12)            # the second K block of every CTA never arrives; give up after 4096 polls
        out = ops.multiply(aq, b, bias_t, tile_m=tile)
        torch.cuda.synchronize()                      # the kernel returned by itself
    finally:
        L.mi8_test_wait_fault(-1, 0)
    status = ops.poll_status()
    assert status in (101, 102, 103, 104), f"expected a bounded-wait status word, got {status}"
    import ctypes
    v = ctypes.c_int(0)
    assert L.mi8_poll_status(ctypes.byref(v)) == 6    # MI8_ERR_DEVICE until the word is cleared
    # recovery: clear the workspace and the status word, then the same call is exact (tensor memory was released:
    # a leaked allocation would make this launch wait for columns that never come back)
    check(L.mi8_workspace_init(ws.ptr, ws.nbytes, torch.cuda.current_stream().cuda_stream))
    ops.clear_status()
    out = ops.multiply(aq, b, bias_t, tile_m=tile)
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    assert np.array_equal(out.cpu().numpy(), want)
    for _ in range(3):                                # and stays exact
        out = ops.multiply(aq, b, bias_t)
    torch.cuda.synchronize()
    assert ops.poll_status() == 0 and np.array_equal(out.cpu().numpy(), want)
