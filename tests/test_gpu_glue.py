"""The decode-step glue kernels (through the C ABI) against the CPU checker's fixed-order float
restatement: bit-exact.  An int8 pipeline amplifies a one-ulp difference in LayerNorm or softmax to a
full quantisation step within two affines, so "close" is not good enough for these ops."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from marian_dev_b200.binding import check, lib
    return lib(), check


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _dev(a, cuda_device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)


def test_det_exp_log_match_libm_closely(oracle):
    xs = np.concatenate([np.linspace(-87, 5, 2001), [-100.0, 0.0, -1e-6, 1e-6]]).astype(np.float32)
    got = np.array([oracle.L.mo_det_expf(float(x)) for x in xs], np.float32)
    want = np.exp(xs.astype(np.float64))
    ok = want > 1e-37
    assert np.max(np.abs(got[ok] - want[ok]) / want[ok]) < 4e-7
    ys = np.concatenate([np.logspace(-20, 20, 2001), [1.0, 2.0, 0.5]]).astype(np.float32)
    gl = np.array([oracle.L.mo_det_logf(float(y)) for y in ys], np.float32)
    wl = np.log(ys.astype(np.float64))
    assert np.max(np.abs(gl - wl) / np.maximum(1.0, np.abs(wl))) < 4e-7


@pytest.mark.parametrize("rows,dim", [(1, 64), (7, 256), (33, 1024), (5, 4096)])
@pytest.mark.parametrize("with_resid", [True, False])
def test_add_layernorm_bit_exact(cuda_device, oracle, rows, dim, with_resid):
    L, check = _lib()
    rng = np.random.default_rng(rows * dim)
    a = rng.standard_normal((rows, dim)).astype(np.float32) * 3
    r = rng.standard_normal((rows, dim)).astype(np.float32) if with_resid else None
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    b = (0.1 * rng.standard_normal(dim)).astype(np.float32)
    want = oracle.add_layernorm(a, r, g, b, 1e-6)
    ad, gd, bd = _dev(a, cuda_device), _dev(g, cuda_device), _dev(b, cuda_device)
    rd = _dev(r, cuda_device) if with_resid else None
    out = torch.empty(rows, dim, device=cuda_device)
    rowmax = torch.zeros(rows, device=cuda_device)
    slot = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    check(L.mi8g_add_layernorm(ad.data_ptr(), rd.data_ptr() if with_resid else None, gd.data_ptr(), bd.data_ptr(), 1e-6, rows, dim,
                               out.data_ptr(), rowmax.data_ptr(), slot.data_ptr(), _stream()))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)
    assert np.array_equal(rowmax.cpu().numpy(), np.abs(want).max(axis=1))
    assert slot.view(torch.float32).item() == np.abs(want).max()
    # and it is a LayerNorm: close to the float64 formula
    y = a.astype(np.float64) + (r.astype(np.float64) if with_resid else 0)
    ref = (y - y.mean(1, keepdims=True)) / np.sqrt(y.var(1, keepdims=True) + 1e-6) * g + b
    assert np.abs(want - ref).max() < 1e-4


@pytest.mark.parametrize("mode,rows,batch,length,heads,dh", [
    (0, 12, 3, 1, 2, 32), (0, 12, 3, 9, 2, 32), (0, 64, 16, 45, 16, 64), (0, 8, 2, 70, 8, 64),
    (1, 12, 3, 7, 2, 32), (1, 64, 16, 33, 16, 64), (2, 3 * 11, 3, 11, 4, 64), (2, 2 * 40, 2, 40, 8, 32),
    (2, 2 * 136, 2, 136, 16, 64), (2, 5 * 3, 5, 3, 2, 32), (2, 1, 1, 1, 2, 64),
    # cross-attention with several beams per sentence, at the decode benchmark's size among them
    (1, 8 * 5, 5, 40, 8, 32), (1, 2 * 7, 7, 130, 16, 64), (1, 4 * 128, 128, 36, 16, 64), (1, 3 * 9, 9, 1, 4, 64)])
def test_attention_bit_exact(cuda_device, oracle, mode, rows, batch, length, heads, dh):
    L, check = _lib()
    rng = np.random.default_rng(rows * length + mode)
    dim = heads * dh
    q = rng.standard_normal((rows, dim)).astype(np.float32)
    kv_rows = length * rows if mode == 0 else batch * length
    k = rng.standard_normal((kv_rows, dim)).astype(np.float32)
    v = rng.standard_normal((kv_rows, dim)).astype(np.float32)
    mask = None
    if mode != 0:
        lens = rng.integers(1, length + 1, size=batch)
        mask = np.where(np.arange(length)[None, :] < lens[:, None], 0.0, -99999999.0).astype(np.float32)
    want = oracle.attention1(q, k, v, mask, rows, heads, dh, length, batch, mode)
    qd, kd, vd = _dev(q, cuda_device), _dev(k, cuda_device), _dev(v, cuda_device)
    md = _dev(mask, cuda_device) if mask is not None else None
    out = torch.empty(rows, dim, device=cuda_device)
    slot = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    check(L.mi8g_attention1(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), md.data_ptr() if md is not None else None, rows, heads, dh,
                            length, batch, mode, out.data_ptr(), slot.data_ptr(), _stream()))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)
    assert slot.view(torch.float32).item() == np.abs(want).max()
    # sanity against a float64 softmax attention for one row
    r0 = rows - 1
    grp = r0 % batch if mode == 1 else (r0 // length if mode == 2 else 0)
    idx = [p * rows + r0 for p in range(length)] if mode == 0 else [grp * length + p for p in range(length)]
    for h in range(heads):
        sl = slice(h * dh, (h + 1) * dh)
        z = (k[idx][:, sl].astype(np.float64) @ q[r0, sl].astype(np.float64)) / np.sqrt(dh)
        if mask is not None:
            z = z + mask[grp]
        w = np.exp(z - z.max()); w /= w.sum()
        assert np.abs(want[r0, sl] - w @ v[idx][:, sl].astype(np.float64)).max() < 1e-4


@pytest.mark.parametrize("rows,vocab,k", [(3, 512, 1), (8, 32000, 4), (5, 1000, 8), (2, 300, 3), (7, 5000, 3), (4, 4100, 8), (3, 32000, 1), (3, 1001, 2), (2, 130, 8),
                                           (600, 32000, 4)])
def test_lse_topk_and_merge_bit_exact(cuda_device, oracle, rows, vocab, k):
    L, check = _lib()
    rng = np.random.default_rng(vocab + k)
    logits = rng.standard_normal((rows, vocab)).astype(np.float32)
    logits[0, 5] = logits[0, 3] = logits[0].max() + 1.0      # an exact tie: the smaller index must win
    prev = rng.standard_normal(rows).astype(np.float32)
    prev[-1] = -np.inf                                        # a dummy hypothesis slot
    cs_w, cw_w = oracle.lse_topk(logits, k, prev)
    ld, pd = _dev(logits, cuda_device), _dev(prev, cuda_device)
    cs = torch.empty(rows, k, device=cuda_device)
    cw = torch.empty(rows, k, dtype=torch.int32, device=cuda_device)
    check(L.mi8g_lse_topk(ld.data_ptr(), rows, vocab, k, pd.data_ptr(), cs.data_ptr(), cw.data_ptr(), _stream()))
    torch.cuda.synchronize()
    assert np.array_equal(cs.cpu().numpy(), cs_w)
    assert np.array_equal(cw.cpu().numpy(), cw_w)
    if k > 1:
        assert cw_w[0, 0] == 3 and cw_w[0, 1] == 5
    ref = logits.astype(np.float64) - np.log(np.exp(logits.astype(np.float64)).sum(1, keepdims=True))
    assert np.abs(cs_w[:-1, 0] - (ref[:-1].max(1) + prev[:-1])).max() < 1e-4
    # merge: treat the rows as `rows` beams of ONE sentence
    os_, ob, ow = (torch.empty(k, device=cuda_device), torch.empty(k, dtype=torch.int32, device=cuda_device),
                   torch.empty(k, dtype=torch.int32, device=cuda_device))
    check(L.mi8g_nbest_merge(cs.data_ptr(), cw.data_ptr(), rows, 1, vocab, k, os_.data_ptr(), ob.data_ptr(), ow.data_ptr(), _stream()))
    torch.cuda.synchronize()
    cands = sorted(((-float(cs_w[j, c]), j * vocab + int(cw_w[j, c])) for j in range(rows) for c in range(k) if cs_w[j, c] != -np.inf))
    for n in range(min(k, len(cands))):
        assert os_[n].item() == np.float32(-cands[n][0])
        assert ob[n].item() == cands[n][1] // vocab and ow[n].item() == cands[n][1] % vocab


def test_embed_and_quantize_slot(cuda_device, oracle):
    L, check = _lib()
    rng = np.random.default_rng(4)
    vocab, dim, rows, S = 100, 128, 24, 6
    wemb = rng.standard_normal((vocab, dim)).astype(np.float32)
    from marian_dev_b200.model import sinusoidal_table
    pos = sinusoidal_table(16, dim)
    words = rng.integers(0, vocab, rows).astype(np.int32)
    scale = float(np.sqrt(np.float32(dim)))
    want = oracle.embed(wemb, words, pos, S, scale, rows)
    wd, pd, idd = _dev(wemb, cuda_device), _dev(pos, cuda_device), _dev(words, cuda_device)
    out = torch.empty(rows, dim, device=cuda_device)
    slot = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    check(L.mi8g_embed(wd.data_ptr(), idd.data_ptr(), pd.data_ptr(), S, scale, rows, dim, out.data_ptr(), None, slot.data_ptr(), _stream()))
    q = torch.empty(rows * dim + 16, dtype=torch.int8, device=cuda_device)
    qm = torch.zeros(1, device=cuda_device)
    check(L.mi8g_quantize_slot(out.data_ptr(), rows * dim, slot.data_ptr(), q.data_ptr(), qm.data_ptr(), _stream()))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)
    assert np.float32(qm.item()) == oracle.quant_mult(want)
    assert np.array_equal(q[:rows * dim].cpu().numpy().reshape(rows, dim), oracle.quantize(want, oracle.quant_mult(want)))
    # zero embedding at the first decoder step
    want0 = oracle.embed(wemb, None, pos[3:4], 0, scale, rows)
    check(L.mi8g_embed(wd.data_ptr(), None, pd[3:].data_ptr(), 0, scale, rows, dim, out.data_ptr(), None, None, _stream()))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want0)


@pytest.mark.parametrize("rows,vocab,k,dim", [(512, 32000, 4, 1024), (64, 1000, 4, 64), (5, 300, 1, 128), (130, 777 * 4, 8, 256), (33, 129, 3, 64)])
def test_fused_output_layer_bit_exact(cuda_device, oracle, rows, vocab, k, dim):
    """int8 GEMM with the log-sum-exp / top-k reduction inside its write-back + the block merge: candidates and the
    (optional) logits equal the checker's affine followed by its log-softmax / top-k, bit for bit; ragged vocabularies,
    row counts that are not a multiple of 128, k up to 8."""
    L, check = _lib()
    from marian_dev_b200 import ops
    rng = np.random.default_rng(rows + vocab + k)
    a = rng.standard_normal((rows, dim)).astype(np.float32)
    wemb = (rng.standard_normal((vocab, dim)) * 0.05).astype(np.float32)       # [vocab, dim]: already N x K
    bias = (rng.standard_normal(vocab) * 0.1).astype(np.float32)
    prev = rng.standard_normal(rows).astype(np.float32)
    bt, qb = oracle.prepare_b(wemb, w_is_nk=True)
    logits_w = oracle.affine(a, bt, qb, bias, 1.0, False)
    logits_w = logits_w[0] if isinstance(logits_w, tuple) else logits_w
    cs_w, cw_w = oracle.lse_topk(logits_w, k, prev)
    wq = ops.prepareB(torch.from_numpy(wemb).to(cuda_device), w_is_nk=True)
    aq = ops.prepareA(torch.from_numpy(a).to(cuda_device))
    nbytes = L.mi8g_output_scratch_bytes(rows, vocab)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=cuda_device)
    logits = torch.full((rows, vocab), float("nan"), device=cuda_device)
    cs = torch.empty(rows, k, device=cuda_device)
    cw = torch.empty(rows, k, dtype=torch.int32, device=cuda_device)
    bd, pd = _dev(bias, cuda_device), _dev(prev, cuda_device)
    check(L.mi8g_output_topk(aq.data.data_ptr(), aq.quant_mult.data_ptr(), wq.data.data_ptr(), wq.quant_mult.data_ptr(), rows, vocab, dim,
                             bd.data_ptr(), k, pd.data_ptr(), scratch.data_ptr(), nbytes, logits.data_ptr(), cs.data_ptr(), cw.data_ptr(),
                             _stream()))
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    assert np.array_equal(logits.cpu().numpy(), logits_w)
    assert np.array_equal(cw.cpu().numpy(), cw_w)
    assert np.array_equal(cs.cpu().numpy(), cs_w)
    # without the logits copy: same candidates
    cs2 = torch.empty_like(cs)
    cw2 = torch.empty_like(cw)
    check(L.mi8g_output_topk(aq.data.data_ptr(), aq.quant_mult.data_ptr(), wq.data.data_ptr(), wq.quant_mult.data_ptr(), rows, vocab, dim,
                             bd.data_ptr(), k, pd.data_ptr(), scratch.data_ptr(), nbytes, None, cs2.data_ptr(), cw2.data_ptr(), _stream()))
    torch.cuda.synchronize()
    assert torch.equal(cs2, cs) and torch.equal(cw2, cw)
