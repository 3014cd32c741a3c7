"""Parity of the CUDA kernels (called through the C ABI) against the CPU oracle: bit-exact for the
abs-max, the int8 quantisation, the int32 accumulators and - because both sides round the same
two fp32 operations - the dequantised outputs as well (the tolerance the path asks for is 1e-5
relative; the assertion below is the stricter exact one, with the 1e-5 check kept beside it)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5  # relative error allowed for dequantised outputs


def _ops():
    from marian_dev_b200 import ops
    return ops


def _assert_healthy():
    assert _ops().poll_status() == 0


@pytest.mark.parametrize("n", [1, 3, 4, 17, 1024, 4099, 256 * 512, 1 << 22])
def test_max_absolute_and_quantize(cuda_device, oracle, n):
    ops = _ops()
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32) * 3
    n_pad = ((n + 3) // 4) * 4
    xt = torch.zeros(n_pad, dtype=torch.float32, device=cuda_device)
    xt[:n] = torch.from_numpy(x).to(cuda_device)
    ws = ops.default_workspace(cuda_device)
    from marian_dev_b200.binding import check, lib
    absmax = torch.zeros(1, dtype=torch.float32, device=cuda_device)
    qm = torch.zeros(1, dtype=torch.float32, device=cuda_device)
    check(lib().mi8_max_absolute_f32(xt.data_ptr(), n, absmax.data_ptr(), qm.data_ptr(), ws.ptr, ws.nbytes,
                                     torch.cuda.current_stream().cuda_stream))
    q = torch.zeros(n_pad + 16, dtype=torch.int8, device=cuda_device)
    check(lib().mi8_quantize_f32_i8(xt.data_ptr(), n, qm.data_ptr(), q.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert absmax.item() == np.abs(x).max()
    assert np.float32(qm.item()) == oracle.quant_mult(x)
    want = oracle.quantize(x, oracle.quant_mult(x))
    assert np.array_equal(q[:n].cpu().numpy(), want)
    assert int(q[n:].abs().sum()) == 0  # nothing written past the end
    # the workspace counters are back to zero
    assert int(ws.buf[:16640].to(torch.int32).sum()) == 0
    _assert_healthy()


def test_quantize_edge_cases(cuda_device, oracle):
    ops = _ops()
    # all-zero tensor: multiplier defined as 1
    z = torch.zeros(64, 64, device=cuda_device)
    zq = ops.prepareA(z)
    torch.cuda.synchronize()
    assert zq.quant_mult.item() == 1.0 and int(zq.data.abs().sum()) == 0
    # ties round to even, +-max maps to +-127, -128 never appears
    vals = np.array([127.0, -127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, -126.5, 63.49999, 1e-9] + [0.0] * 4,
                    dtype=np.float32).reshape(1, 16)
    t = torch.from_numpy(vals).to(cuda_device)
    tq = ops.prepareA(t)
    torch.cuda.synchronize()
    assert tq.quant_mult.item() == 1.0
    assert np.array_equal(tq.data.cpu().numpy(), oracle.quantize(vals, np.float32(1.0)))
    assert tq.data.min().item() >= -127
    _assert_healthy()


@pytest.mark.parametrize("k,n", [(512, 2048), (1024, 1024), (256, 1536), (96, 40)])
def test_prepare_b(cuda_device, oracle, k, n):
    ops = _ops()
    rng = np.random.default_rng(k * 7 + n)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    b = ops.prepareB(torch.from_numpy(w).to(cuda_device))
    torch.cuda.synchronize()
    bt, qb = oracle.prepare_b(w)
    assert np.float32(b.quant_mult.item()) == qb
    assert np.array_equal(b.data.cpu().numpy(), bt)
    assert b.shape == (k, n)
    # an [N,K] weight (tied embedding used with transB) is only quantised
    b2 = ops.prepareB(torch.from_numpy(np.ascontiguousarray(w.T)).to(cuda_device), w_is_nk=True)
    torch.cuda.synchronize()
    assert np.array_equal(b2.data.cpu().numpy(), bt) and b2.shape == (k, n)
    _assert_healthy()


def _run_affine(cuda_device, oracle, m, k, n, relu, with_bias, seed, out_dtype=torch.float32, tile_m=0, splits=0,
                scale=1.0):
    ops = _ops()
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.01).astype(np.float32) if with_bias else None
    bt, qb = oracle.prepare_b(w)
    want, want_acc, want_aq, want_qa = oracle.affine(a, bt, qb, bias, scale, relu, want_acc=True)

    b = ops.prepareB(torch.from_numpy(w).to(cuda_device))
    aq = ops.prepareA(torch.from_numpy(a).to(cuda_device))
    acc = torch.full((m, n), -7, dtype=torch.int32, device=cuda_device)
    guard = 64
    out_buf = torch.full((m * n + guard,), float("nan"), dtype=out_dtype, device=cuda_device)
    out = ops.multiply(aq, b, torch.from_numpy(bias).to(cuda_device) if with_bias else None, scale, relu,
                       out=out_buf[:m * n].view(m, n), out_dtype=out_dtype, acc_out=acc, tile_m=tile_m, splits=splits)
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    assert np.array_equal(aq.data.cpu().numpy(), want_aq)
    assert np.float32(aq.quant_mult.item()) == want_qa
    got_acc = acc.cpu().numpy()
    assert np.array_equal(got_acc, want_acc), f"int32 accumulators differ at {np.argwhere(got_acc != want_acc)[:5]}"
    got = out.float().cpu().numpy()
    if out_dtype == torch.float32:
        denom = np.maximum(np.abs(want), 1e-30)
        assert np.all(np.abs(got - want) <= REL_TOL * np.maximum(denom, np.abs(want).max() * 1e-3))
        assert np.array_equal(got, want)  # both sides round identically, so in fact bit-exact
    else:
        assert np.array_equal(got, want.astype(np.float16).astype(np.float32))
    assert bool(torch.isnan(out_buf[m * n:].float()).all())  # canary behind the output untouched
    ws = ops.default_workspace(cuda_device)
    # counters and split-K accumulation buffers are zero again (bytes 16640..20736 hold abs-max partials)
    assert int(ws.buf[:16640].view(torch.int32).abs().sum()) == 0
    assert int(ws.buf[20736:].view(torch.int32).abs().max()) == 0
    return got


def test_config1_single_affine(cuda_device, oracle):
    """X[256,512] ~ N(0,1), W[512,2048] ~ N(0,0.02), bias ~ N(0,0.01), ReLU, seed 0."""
    _run_affine(cuda_device, oracle, 256, 512, 2048, True, True, 0)


@pytest.mark.parametrize("m", [1, 2, 5, 8, 16, 17, 31, 32, 33, 64, 100, 128, 130, 256, 257, 512, 1000])
def test_affine_m_sweep(cuda_device, oracle, m):
    _run_affine(cuda_device, oracle, m, 512, 384, bool(m % 2), bool(m % 3), 100 + m)


@pytest.mark.parametrize("n", [8, 40, 128, 136, 264, 1000])
@pytest.mark.parametrize("k", [64, 128, 192, 512, 1040])
def test_affine_ragged_nk(cuda_device, oracle, n, k):
    _run_affine(cuda_device, oracle, 24, k, n, True, True, n * 13 + k)


@pytest.mark.parametrize("splits", [1, 2, 4, 8])
@pytest.mark.parametrize("m,tile_m", [(8, 16), (64, 64), (200, 256)])
def test_split_k_bit_identical(cuda_device, oracle, splits, m, tile_m):
    _run_affine(cuda_device, oracle, m, 1024, 640, False, True, 7, tile_m=tile_m, splits=splits)


@pytest.mark.parametrize("tile_m", [16, 32, 64, 128, 256])
def test_every_tile_width(cuda_device, oracle, tile_m):
    # more activation rows than one tile, so several tiles along M run in every configuration
    _run_affine(cuda_device, oracle, 300, 256, 384, True, True, tile_m, tile_m=tile_m)


def test_persistent_schedule_many_tiles(cuda_device, oracle):
    # 32 x 16 = 512 tiles on 148 CTAs: every CTA walks several tiles and both accumulator buffers
    _run_affine(cuda_device, oracle, 4096, 256, 4096, True, True, 11)


@pytest.mark.parametrize("m,k,n", [(512, 1024, 1024), (300, 256, 384), (777, 208, 333), (129, 128, 130), (1, 64, 8)])
def test_cta_pair_kernel(cuda_device, oracle, m, k, n):
    """tile_m = 512 selects the two-CTA kernel (256 x 256 tile per cluster): ragged M, odd numbers of
    128-row weight tiles (the second CTA of the last pair has no rows), K that is not a multiple of 128."""
    _run_affine(cuda_device, oracle, m, k, n, True, True, m + k + n, tile_m=512)


def test_cta_pair_kernel_many_tiles(cuda_device, oracle):
    # 16 x 16 = 256 pair tiles on 74 clusters: every pair walks several tiles and both accumulator buffers
    _run_affine(cuda_device, oracle, 4096, 256, 4096, False, True, 12, tile_m=512)
    _run_affine(cuda_device, oracle, 2100, 1024, 1000, True, False, 13, out_dtype=torch.float16, tile_m=512)


@pytest.mark.parametrize("tile_m", [0, 64, 128, 256, 512])
def test_rows_from_keeps_whole_tiles_below(cuda_device, oracle, tile_m):
    """Equal words: tiles wholly below the row limit keep the sentinel, every other row is computed; unequal
    words: everything is computed.  Covers the single-CTA and the two-CTA kernel."""
    ops = _ops()
    m, k, n = 1100, 256, 520
    rng = np.random.default_rng(tile_m + 5)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.01).astype(np.float32)
    bt, qb = oracle.prepare_b(w)
    want = oracle.affine(a, bt, qb, bias, 1.0, False, want_acc=True)[0]
    b = ops.prepareB(torch.from_numpy(w).to(cuda_device))
    aq = ops.prepareA(torch.from_numpy(a).to(cuda_device))
    bias_t = torch.from_numpy(bias).to(cuda_device)
    from marian_dev_b200 import multiply_plan
    plan = multiply_plan(m, n, k, tile_m, 0)
    tm = 256 if plan["tile_m"] == 512 else plan["tile_m"]
    words = torch.tensor([7, 7, 8], dtype=torch.int32, device=cuda_device)
    for limit in (0, 300, 777, m):
        out = torch.full((m, n), 12345.0, dtype=torch.float32, device=cuda_device)
        ops.multiply_rows_from(aq, b, bias_t, out, words[0:1], words[1:2], limit, tile_m=tile_m)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        kept = (limit // tm) * tm      # whole tiles below the limit
        assert np.all(got[:kept] == 12345.0)
        assert np.array_equal(got[kept:], want[kept:])
        out.fill_(12345.0)
        ops.multiply_rows_from(aq, b, bias_t, out, words[0:1], words[2:3], limit, tile_m=tile_m)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want)
    assert ops.poll_status() == 0


@pytest.mark.parametrize("m,k,n", [(512, 1024, 1024), (512, 4096, 1024), (1, 64, 8), (16, 512, 384), (33, 208, 333), (64, 1024, 4096),
                                   (200, 256, 640), (77, 1040, 136), (512, 512, 1152)])
def test_multiply_quantises_its_activation(cuda_device, oracle, m, k, n):
    """mi8_multiply_f32_slot: PrepareA inside the GEMM kernel from a pre-reduced abs-max; accumulators and
    outputs equal the oracle's (and so the two-call route's) bit for bit; ragged M, N and K."""
    ops = _ops()
    rng = np.random.default_rng(m * 3 + k + n)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.01).astype(np.float32)
    bt, qb = oracle.prepare_b(w)
    want, want_acc, _want_aq, want_qa = oracle.affine(a, bt, qb, bias, 1.0, True, want_acc=True)
    b = ops.prepareB(torch.from_numpy(w).to(cuda_device))
    a_t = torch.from_numpy(a).to(cuda_device)
    slot = a_t.abs().max().reshape(1).view(torch.int32).clone()       # bit pattern of max|a|
    acc = torch.full((m, n), -7, dtype=torch.int32, device=cuda_device)
    qa = torch.zeros(1, device=cuda_device)
    out = ops.multiply_from_slot(a_t, slot, b, torch.from_numpy(bias).to(cuda_device), 1.0, True, acc_out=acc, qa_out=qa)
    assert out is not None
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    assert np.float32(qa.item()) == want_qa
    assert np.array_equal(acc.cpu().numpy(), want_acc)
    assert np.array_equal(out.cpu().numpy(), want)


def test_multiply_from_slot_declines_large_shapes(cuda_device):
    ops = _ops()
    a = torch.randn(4096, 256, device=cuda_device)
    b = ops.prepareB(torch.randn(256, 4096, device=cuda_device) * 0.02)
    slot = a.abs().max().reshape(1).view(torch.int32).clone()
    assert ops.multiply_from_slot(a, slot, b) is None


def test_int8_mma_peak_measurement(cuda_device):
    """The measurement aid runs, raises no device status and reports a plausible tensor-pipe rate (above what the
    full GEMM reaches, below the nominal 4.5 POPS of the part)."""
    ops = _ops()
    tops = ops.measure_int8_peak(2048)
    assert ops.poll_status() == 0
    assert 500.0 < tops < 4600.0


def test_fp16_output_and_scale(cuda_device, oracle):
    _run_affine(cuda_device, oracle, 96, 512, 256, False, True, 5, out_dtype=torch.float16, scale=0.125)
    _run_affine(cuda_device, oracle, 96, 512, 256, True, False, 6, scale=2.0)


def test_repeated_calls_share_workspace(cuda_device, oracle):
    a = _run_affine(cuda_device, oracle, 8, 1024, 1024, False, True, 3)
    for _ in range(3):
        b = _run_affine(cuda_device, oracle, 8, 1024, 1024, False, True, 3)
        assert np.array_equal(a, b)


def test_operator_surface(cuda_device, oracle):
    """affine / dot / affineWithReluDropout on [..., K] inputs, float semantics of the reference's
    own operator tests (src/tests/units/operator_tests.cpp:618-659) within int8 precision."""
    ops = _ops()
    rng = np.random.default_rng(21)
    x = rng.standard_normal((3, 7, 256)).astype(np.float32)
    w = (rng.standard_normal((256, 128)) * 0.05).astype(np.float32)
    bias = (rng.standard_normal(128) * 0.1).astype(np.float32)
    xt, bt_, biast = (torch.from_numpy(v).to(cuda_device) for v in (x, w, bias))
    W = ops.prepareB(bt_)
    bt, qb = oracle.prepare_b(w)
    y = ops.affine(xt, W, biast)
    y2 = ops.dot(xt, W, scale=0.5)
    y3 = ops.affineWithReluDropout(xt, W, biast)
    torch.cuda.synchronize()
    assert y.shape == (3, 7, 128)
    assert np.array_equal(y.cpu().numpy(), oracle.affine(x, bt, qb, bias))
    assert np.array_equal(y2.cpu().numpy(), oracle.affine(x, bt, qb, None, 0.5))
    assert np.array_equal(y3.cpu().numpy(), oracle.affine(x, bt, qb, bias, 1.0, True))
    ref = np.maximum(x @ w + bias, 0)
    assert np.abs(y3.cpu().numpy() - ref).max() < 0.05 * np.abs(ref).max()
    _assert_healthy()


def test_argument_errors(cuda_device):
    ops = _ops()
    from marian_dev_b200.binding import Mi8Error
    W = ops.prepareB(torch.randn(64, 32, device=cuda_device))
    with pytest.raises(Mi8Error):
        ops.affine(torch.randn(4, 64, device=cuda_device).double(), W, None)
    with pytest.raises(Mi8Error):
        ops.affine(torch.randn(4, 48, device=cuda_device), W, None)  # inner dimension mismatch
    with pytest.raises(Mi8Error):
        ops.affine(torch.randn(4, 64), W, None)  # host tensor: there is no CPU path
    with pytest.raises(Mi8Error):
        ops.affineWithReluDropout(torch.randn(4, 64, device=cuda_device), W, None, 0.1)
    Wbad = ops.prepareB(torch.randn(40, 32, device=cuda_device))  # K = 40 is not a multiple of 16
    with pytest.raises(Mi8Error):
        ops.affine(torch.randn(4, 40, device=cuda_device), Wbad, None)
    _assert_healthy()


def test_against_committed_golden_vectors(cuda_device):
    """The GPU path must hash to the committed fixtures (tests/golden/affine_golden.json): quantised
    weights and activations, both multipliers, the int32 accumulators and the fp32 outputs."""
    import json
    import os
    from tests.golden.make_golden import cases, digest, inputs
    ops = _ops()
    want = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "affine_golden.json")))
    for name, spec in cases().items():
        a, w, bias = inputs(spec)
        m, n = spec["m"], spec["n"]
        b = ops.prepareB(torch.from_numpy(w).to(cuda_device))
        aq = ops.prepareA(torch.from_numpy(a).to(cuda_device))
        acc = torch.empty((m, n), dtype=torch.int32, device=cuda_device)
        out = ops.multiply(aq, b, torch.from_numpy(bias).to(cuda_device) if bias is not None else None, spec["scale"],
                           spec["relu"], acc_out=acc)
        torch.cuda.synchronize()
        got = {"bt": b.data.cpu().numpy(), "qb": b.quant_mult.cpu().numpy(), "aq": aq.data.cpu().numpy(),
               "qa": aq.quant_mult.cpu().numpy(), "acc": acc.cpu().numpy(), "out": out.cpu().numpy()}
        for key, arr in got.items():
            assert digest(arr) == want[name]["sha256"][key], f"{name}: {key} differs from the committed fixture"
    _assert_healthy()


def test_kernel_times_facility(cuda_device):
    """mi8_kernel_times_begin / _end attribute device time to the kernels launched in between."""
    import ctypes
    from marian_dev_b200.binding import Mi8KernelTime, check, lib
    ops = _ops()
    L = lib()
    a = torch.randn(64, 256, device=cuda_device)
    b = ops.prepareB(torch.randn(256, 128, device=cuda_device) * 0.02)
    check(L.mi8_kernel_times_begin())
    for _ in range(3):
        ops.affine(a, b, None)
    buf = (Mi8KernelTime * 16)()
    n = ctypes.c_int(0)
    check(L.mi8_kernel_times_end(buf, 16, ctypes.byref(n)))
    got = {r.name.decode(): (r.launches, r.total_us) for r in buf[:n.value]}
    gemm = [v for k, v in got.items() if "mi8_gemm_kernel" in k]
    assert gemm and gemm[0][0] == 3 and gemm[0][1] > 0
    assert sum(v[0] for v in got.values()) == 9          # abs-max, quantise, GEMM per affine
    # off again: nothing is recorded
    ops.affine(a, b, None)
    check(L.mi8_kernel_times_begin())
    check(L.mi8_kernel_times_end(buf, 16, ctypes.byref(n)))
    assert n.value == 0


@pytest.mark.parametrize("m,k,n", [(4096, 4096, 32000), (1, 4096, 32000), (4096, 512, 512), (1024, 1024, 32000), (4096, 4096, 4096)])
def test_sweep_corner_shapes_at_full_size(cuda_device, oracle, m, k, n):
    """The largest and the skinniest shapes of the affine sweep at their real sizes (two-CTA kernel, split-K and
    weight-streaming plans included): int32 accumulators and fp32 outputs equal the checker's, bit for bit."""
    ops = _ops()
    oracle.set_threads(oracle.max_threads())
    try:
        rng = np.random.default_rng(m + k + n)
        a = rng.standard_normal((m, k)).astype(np.float32)
        w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
        bias = (rng.standard_normal(n) * 0.01).astype(np.float32)
        bt, qb = oracle.prepare_b(w)
        want, want_acc, _aq, want_qa = oracle.affine(a, bt, qb, bias, 1.0, True, want_acc=True)
        b = ops.prepareB(torch.from_numpy(w).to(cuda_device))
        aq = ops.prepareA(torch.from_numpy(a).to(cuda_device))
        acc = torch.empty((m, n), dtype=torch.int32, device=cuda_device)
        out = ops.multiply(aq, b, torch.from_numpy(bias).to(cuda_device), 1.0, True, acc_out=acc)
        torch.cuda.synchronize()
        assert ops.poll_status() == 0
        assert np.float32(aq.quant_mult.item()) == want_qa
        assert np.array_equal(acc.cpu().numpy(), want_acc)
        assert np.array_equal(out.cpu().numpy(), want)
    finally:
        oracle.set_threads(1)
