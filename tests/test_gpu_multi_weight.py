"""mi8_multiply_i8_multi through the C ABI: one quantised activation against two or three converted weights of the same
shape in one launch (Wk|Wv of an attention block, Wq|Wk|Wv of the encoder, the SSRU's W|Wf).  Every output must equal,
bit for bit, what the CPU checker computes for that weight alone: every tile width the plan picks (skinny rows, one wave,
persistent schedules, the two-CTA kernel), with and without bias, fp32 and fp16 output, ReLU."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(cuda_device, oracle, m, k, n_each, count, with_bias, relu=False, out_dtype=torch.float32, seed=0):
    from marian_dev_b200 import ops
    from marian_dev_b200.binding import MI8_F16, MI8_F32, check, lib
    rng = np.random.default_rng(seed + m * 13 + k + n_each * 7 + count)
    a = rng.standard_normal((m, k)).astype(np.float32)
    ws_np = [(rng.standard_normal((k, n_each)) * (0.02 * (i + 1))).astype(np.float32) for i in range(count)]   # different multipliers
    biases = [(rng.standard_normal(n_each) * 0.01).astype(np.float32) if (with_bias and i != 0) or with_bias == "all" else None
              for i in range(count)]
    aq = ops.prepareA(torch.from_numpy(a).to(cuda_device))
    wq = [ops.prepareB(torch.from_numpy(w).to(cuda_device)) for w in ws_np]
    stacked = torch.cat([w.data.reshape(-1) for w in wq]).contiguous()                # the matrices one behind the other
    assert stacked.data_ptr() % 16 == 0
    bias_t = [torch.from_numpy(b).to(cuda_device) if b is not None else None for b in biases]
    outs = [torch.full((m, n_each), float("nan"), dtype=out_dtype, device=cuda_device) for _ in range(count)]
    vp = ctypes.c_void_p
    qb = (vp * 3)(*[w.quant_mult.data_ptr() for w in wq])
    bp = (vp * 3)(*[b.data_ptr() if b is not None else None for b in bias_t])
    cp = (vp * 3)(*[o.data_ptr() for o in outs])
    wsp = ops.default_workspace(cuda_device)
    rc = lib().mi8_multiply_i8_multi(aq.data.data_ptr(), stacked.data_ptr(), m, n_each, k, count, aq.quant_mult.data_ptr(), qb, 1.0, bp,
                                     int(relu), cp, MI8_F32 if out_dtype == torch.float32 else MI8_F16, wsp.ptr, wsp.nbytes,
                                     torch.cuda.current_stream().cuda_stream)
    check(rc)
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    for i in range(count):
        bt, qbi = oracle.prepare_b(ws_np[i])
        want = oracle.affine(a, bt, qbi, biases[i], 1.0, relu)            # quantises `a` like prepareA, then the exact product
        got = outs[i].cpu().numpy()
        if out_dtype == torch.float16:
            want = want.astype(np.float16)
        assert np.array_equal(got, want), f"matrix {i} of {count} differs (max abs diff {np.abs(got.astype(np.float64) - want).max()})"


@pytest.mark.parametrize("m", [1, 16, 40, 64, 200, 512, 1100])
@pytest.mark.parametrize("count", [2, 3])
def test_multi_weight_matches_checker(cuda_device, oracle, m, count):
    _run(cuda_device, oracle, m, 256, 128, count, with_bias=True)


@pytest.mark.parametrize("m,k,n_each,count", [(512, 1024, 1024, 2), (2600, 1024, 1024, 3), (700, 512, 256, 2), (33, 1024, 384, 3)])
def test_multi_weight_decoder_shapes(cuda_device, oracle, m, k, n_each, count):
    """Wk|Wv at the benchmark's decoder width, Wq|Wk|Wv over an encoder-sized activation (the two-CTA kernel, whose two
    CTAs can sit in different matrices), the SSRU pair (first matrix without bias)."""
    _run(cuda_device, oracle, m, k, n_each, count, with_bias="all" if count == 3 else True)


def test_multi_weight_fp16_relu(cuda_device, oracle):
    _run(cuda_device, oracle, 96, 256, 256, 2, with_bias="all", relu=True, out_dtype=torch.float16)


def test_multi_weight_rejects_ragged_width(cuda_device):
    from marian_dev_b200.binding import MI8_F32, lib
    vp = ctypes.c_void_p
    t = torch.zeros(1 << 16, dtype=torch.int8, device=cuda_device)
    f = torch.ones(4, device=cuda_device)
    o = torch.zeros(8 * 192, device=cuda_device)
    qb = (vp * 3)(f.data_ptr(), f.data_ptr(), None)
    cp = (vp * 3)(o.data_ptr(), o.data_ptr(), None)
    rc = lib().mi8_multiply_i8_multi(t.data_ptr(), t.data_ptr(), 8, 96, 64, 2, f.data_ptr(), qb, 1.0, None, 0, cp, MI8_F32, None, 0, None)
    assert rc == 3    # MI8_ERR_UNSUPPORTED: 96 is not a multiple of 128
    assert lib().mi8_multiply_i8_multi(t.data_ptr(), t.data_ptr(), 8, 128, 64, 4, f.data_ptr(), qb, 1.0, None, 0, cp, MI8_F32, None, 0, None) == 1
