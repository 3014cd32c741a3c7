"""The no-allocation multiply (mi8_multiply_i8_static), called through the C ABI.

Some callers cannot give the library a workspace because they cannot allocate device memory at the
point of the call (Marian's arena already owns it; a latency-critical thread must not trigger
cudaMalloc's device synchronisation).  For them the split-K scratch is a fixed array inside the
library.  This test runs the entry point twice in a row on shapes that really split K, so the second
call meets the first call's leftovers in the shared array, and compares with the regular entry point
bit for bit (the tolerance of the other parity tests is exact equality as well).  It is collected
last so that a failure here cannot hide another test's result in a run that stops at the first failure.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n", [(8, 2048, 1024), (16, 4096, 512), (64, 2048, 2048), (300, 512, 640)])
def test_static_scratch_matches_workspace_entry_point(cuda_device, m, k, n):
    from marian_dev_b200 import multiply_plan, ops
    from marian_dev_b200.binding import MI8_F32, check, lib
    torch.manual_seed(m * 31 + n)
    a = torch.randn(m, k, device=cuda_device)
    w = torch.randn(k, n, device=cuda_device) * 0.02
    bias = torch.randn(n, device=cuda_device) * 0.01
    aq = ops.prepareA(a)
    b = ops.prepareB(w)
    want = ops.multiply(aq, b, bias, 1.0, True)                      # regular entry point, caller-owned workspace
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for _ in range(2):                                                # two calls in a row share the built-in array
        out = torch.full((m, n), float("nan"), device=cuda_device)
        check(lib().mi8_multiply_i8_static(aq.data.data_ptr(), b.data.data_ptr(), m, n, k, aq.quant_mult.data_ptr(),
                                           b.quant_mult.data_ptr(), 1.0, bias.data_ptr(), 1, out.data_ptr(), MI8_F32, stream))
        outs.append(out)
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    for out in outs:
        assert np.array_equal(out.cpu().numpy(), want.cpu().numpy())
    if (m, k, n) != (300, 512, 640):
        assert multiply_plan(m, n, k)["splits"] > 1, "the case is meant to exercise the split-K scratch"


def test_static_scratch_rejects_oversized_shapes(cuda_device):
    from marian_dev_b200.binding import MI8_F32, lib
    m, k, n = 64, 4096, 8320                                         # split-K plan: 65 tiles x 32 KiB = 2.03 MiB of accumulation buffers
    aq = torch.zeros(m * k + 4, dtype=torch.int8, device=cuda_device)
    bt = torch.zeros(n * k + 4, dtype=torch.int8, device=cuda_device)
    q = torch.ones(2, device=cuda_device)
    out = torch.zeros(m, n, device=cuda_device)
    rc = lib().mi8_multiply_i8_static(aq.data_ptr(), bt.data_ptr(), m, n, k, q.data_ptr(), q[1:].data_ptr(), 1.0, None, 0,
                                      out.data_ptr(), MI8_F32, torch.cuda.current_stream().cuda_stream)
    assert rc == 4                                                    # MI8_ERR_WORKSPACE
    assert lib().mi8_strerror(rc) == b"workspace missing or too small"
    assert lib().mi8_multiply_i8_static(None, None, 4, 8, 64, None, None, 1.0, None, 0, None, 0, None) == 1
