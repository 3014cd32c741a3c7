"""The no-allocation multiply (mi8_multiply_i8_static), called through the C ABI.

Some callers cannot give the library a workspace because they cannot allocate device memory at the
point of the call (Marian's arena already owns it; a latency-critical thread must not trigger
cudaMalloc's device synchronisation).  For them the split-K scratch is a fixed array inside the
library.  This test runs the entry point twice in a row on shapes that really split K, so the second
call meets the first call's leftovers in the shared array, and compares with the regular entry point
and with the CPU checker bit for bit (the tolerance of the other parity tests is exact equality as well),
with and without a bias and with fp16 output.  It is collected
last so that a failure here cannot hide another test's result in a run that stops at the first failure.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n", [(8, 2048, 1024), (16, 4096, 512), (64, 2048, 2048), (300, 512, 640)])
@pytest.mark.parametrize("with_bias,out_dtype", [(True, torch.float32), (False, torch.float32), (True, torch.float16)])
def test_static_scratch_matches_workspace_entry_point(cuda_device, oracle, m, k, n, with_bias, out_dtype):
    from marian_dev_b200 import multiply_plan, ops
    from marian_dev_b200.binding import MI8_F16, MI8_F32, check, lib
    rng = np.random.default_rng(m * 31 + n)
    a_np = rng.standard_normal((m, k)).astype(np.float32)
    w_np = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias_np = (rng.standard_normal(n) * 0.01).astype(np.float32) if with_bias else None
    a = torch.from_numpy(a_np).to(cuda_device)
    bias = torch.from_numpy(bias_np).to(cuda_device) if with_bias else None
    aq = ops.prepareA(a)
    b = ops.prepareB(torch.from_numpy(w_np).to(cuda_device))
    want = ops.multiply(aq, b, bias, 1.0, True, out_dtype=out_dtype)     # regular entry point, caller-owned workspace
    # ... which itself must be what the CPU checker computes, so this test stands on its own
    bt, qb = oracle.prepare_b(w_np)
    checker = oracle.affine(a_np, bt, qb, bias_np, 1.0, True)
    if out_dtype == torch.float16:
        checker = checker.astype(np.float16)
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for _ in range(2):                                                # two calls in a row share the built-in array
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device=cuda_device)
        check(lib().mi8_multiply_i8_static(aq.data.data_ptr(), b.data.data_ptr(), m, n, k, aq.quant_mult.data_ptr(),
                                           b.quant_mult.data_ptr(), 1.0, bias.data_ptr() if with_bias else None, 1, out.data_ptr(),
                                           MI8_F32 if out_dtype == torch.float32 else MI8_F16, stream))
        outs.append(out)
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    assert np.array_equal(want.cpu().numpy(), checker)
    for out in outs:
        assert np.array_equal(out.cpu().numpy(), want.cpu().numpy())
        assert np.array_equal(out.cpu().numpy(), checker)
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
    # arguments are checked before anything is queued: a misaligned operand or an unknown output type is refused outright
    st = torch.cuda.current_stream().cuda_stream
    assert lib().mi8_multiply_i8_static(aq.data_ptr() + 1, bt.data_ptr(), 8, 256, 2048, q.data_ptr(), q[1:].data_ptr(), 1.0, None, 0,
                                        out.data_ptr(), MI8_F32, st) == 2
    assert lib().mi8_multiply_i8_static(aq.data_ptr(), bt.data_ptr(), 8, 256, 2048, q.data_ptr(), q[1:].data_ptr(), 1.0, None, 0,
                                        out.data_ptr(), 7, st) == 1
