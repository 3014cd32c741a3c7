"""The cluster GEMM through the C ABI (mi8g_affine_slot, mi8g_affine_slot_add_layernorm): one launch that quantises the fp32
activation from its abs-max slot inside the kernel (the CTAs of a cluster share the quantised tile through distributed shared
memory) and, in its second form, applies the residual add + LayerNorm to the result with the per-row sums exchanged between
the CTAs of the cluster.  Both must equal, bit for bit, what the CPU checker computes for prepareA + multiply (+ LayerNorm):
every tile width and cluster size, ragged row counts, K = 128 ... 4096, with and without bias / residual, ReLU, the abs-max
outputs and the row maxima."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(cuda_device, oracle, m, k, n, with_bias, seed=0, scale_a=1.0):
    from marian_dev_b200 import ops
    rng = np.random.default_rng(seed + 31 * m + k + 7 * n)
    a = (rng.standard_normal((m, k)) * scale_a).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.03).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.05).astype(np.float32) if with_bias else None
    wq = ops.prepareB(torch.from_numpy(w).to(cuda_device))
    bt, qb = oracle.prepare_b(w)
    ad = torch.from_numpy(a).to(cuda_device)
    slot = torch.tensor([np.abs(a).max()], dtype=torch.float32, device=cuda_device)     # the bit pattern of max|a|
    bd = torch.from_numpy(bias).to(cuda_device) if with_bias else None
    return a, bias, bt, qb, ad, slot, wq, bd


def _affine(cuda_device, oracle, m, k, n, with_bias=True, relu=False, tile=0, cluster=0, seed=0):
    from marian_dev_b200 import ops
    from marian_dev_b200.binding import check, lib
    a, bias, bt, qb, ad, slot, wq, bd = _setup(cuda_device, oracle, m, k, n, with_bias, seed)
    out = torch.full((m, n), float("nan"), device=cuda_device)
    canary = torch.full((64,), 7.0, device=cuda_device)
    amax = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    check(lib().mi8g_affine_slot(ad.data_ptr(), slot.data_ptr(), wq.data.data_ptr(), wq.quant_mult.data_ptr(), m, n, k, 1.0,
                                 bd.data_ptr() if bd is not None else None, int(relu), out.data_ptr(), amax.data_ptr(), tile, cluster,
                                 torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    want = oracle.affine(a, bt, qb, bias, 1.0, relu)
    got = out.cpu().numpy()
    assert np.array_equal(got, want), f"max abs diff {np.abs(got.astype(np.float64) - want).max()}"
    assert amax.view(torch.float32).item() == np.abs(want).max()
    assert torch.all(canary == 7.0)


@pytest.mark.parametrize("m,k,n", [(512, 1024, 1024), (512, 1024, 4096), (512, 4096, 1024), (256, 1024, 4096), (37, 512, 512),
                                   (200, 1024, 2048), (1, 128, 128), (130, 256, 384), (64, 2048, 1024), (300, 1024, 1280)])
def test_cluster_affine_matches_checker(cuda_device, oracle, m, k, n):
    _affine(cuda_device, oracle, m, k, n, with_bias=True, relu=(n == 4096))


@pytest.mark.parametrize("tile", [32, 64, 128])
@pytest.mark.parametrize("cluster", [1, 2, 4, 8])
def test_cluster_affine_every_plan(cuda_device, oracle, tile, cluster):
    _affine(cuda_device, oracle, 150, 1024, 1024, with_bias=(cluster != 2), tile=tile, cluster=cluster, seed=tile + cluster)
    _affine(cuda_device, oracle, 97, 384, 1024, with_bias=True, relu=True, tile=tile, cluster=cluster, seed=tile * cluster)   # fewer K blocks than CTAs


def test_cluster_affine_many_waves(cuda_device, oracle):
    """More clusters than the device holds at once (they run in waves), rows not a multiple of the tile."""
    _affine(cuda_device, oracle, 1500, 1024, 1024, tile=32)
    _affine(cuda_device, oracle, 1111, 512, 2048, tile=64, relu=True)


def test_cluster_affine_rejects_unsupported(cuda_device):
    from marian_dev_b200.binding import lib
    f = torch.zeros(1 << 16, device=cuda_device)
    q = torch.zeros(1 << 16, dtype=torch.int8, device=cuda_device)
    s = torch.cuda.current_stream().cuda_stream
    L = lib()
    assert L.mi8g_affine_slot(f.data_ptr(), f.data_ptr(), q.data_ptr(), f.data_ptr(), 8, 192, 128, 1.0, None, 0, f.data_ptr(), None, 0, 0, s) != 0   # N % 128
    assert L.mi8g_affine_slot(f.data_ptr(), f.data_ptr(), q.data_ptr(), f.data_ptr(), 8, 128, 192, 1.0, None, 0, f.data_ptr(), None, 0, 0, s) != 0   # K % 128
    assert L.mi8g_affine_slot(f.data_ptr(), f.data_ptr(), q.data_ptr(), f.data_ptr(), 8, 128, 8192, 1.0, None, 0, f.data_ptr(), None, 0, 0, s) != 0  # K > 4096
    assert L.mi8g_affine_slot(f.data_ptr(), f.data_ptr(), q.data_ptr(), f.data_ptr(), 8, 384, 128, 1.0, None, 0, f.data_ptr(), None, 0, 2, s) != 0   # 3 tiles, cluster 2
    assert L.mi8g_affine_slot_add_layernorm(f.data_ptr(), f.data_ptr(), q.data_ptr(), f.data_ptr(), 8, 2048, 128, 1.0, None, None, f.data_ptr(),
                                            f.data_ptr(), 1e-6, f.data_ptr(), None, None, None, s) != 0                                            # row wider than a cluster


@pytest.mark.parametrize("m,k,n", [(512, 1024, 1024), (512, 4096, 1024), (100, 512, 512), (33, 1024, 1024), (1, 128, 128), (77, 256, 384),
                                   (600, 1024, 1024)])
@pytest.mark.parametrize("with_resid", [True, False])
def test_cluster_affine_layernorm_matches_checker(cuda_device, oracle, m, k, n, with_resid):
    from marian_dev_b200 import ops
    from marian_dev_b200.binding import check, lib
    a, bias, bt, qb, ad, slot, wq, bd = _setup(cuda_device, oracle, m, k, n, True, seed=5, scale_a=2.0)
    rng = np.random.default_rng(m + n)
    resid = rng.standard_normal((m, n)).astype(np.float32) if with_resid else None
    g = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    b = (0.1 * rng.standard_normal(n)).astype(np.float32)
    want = oracle.add_layernorm(oracle.affine(a, bt, qb, bias, 1.0, False), resid, g, b, 1e-6)
    rd = torch.from_numpy(resid).to(cuda_device) if with_resid else None
    gd, betad = torch.from_numpy(g).to(cuda_device), torch.from_numpy(b).to(cuda_device)
    out = torch.full((m, n), float("nan"), device=cuda_device)
    rowmax = torch.full((m + 8,), -1.0, device=cuda_device)
    s1 = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    s2 = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    check(lib().mi8g_affine_slot_add_layernorm(ad.data_ptr(), slot.data_ptr(), wq.data.data_ptr(), wq.quant_mult.data_ptr(), m, n, k, 1.0,
                                               bd.data_ptr(), rd.data_ptr() if with_resid else None, gd.data_ptr(), betad.data_ptr(), 1e-6,
                                               out.data_ptr(), rowmax.data_ptr(), s1.data_ptr(), s2.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert ops.poll_status() == 0
    got = out.cpu().numpy()
    assert np.array_equal(got, want), f"max abs diff {np.abs(got.astype(np.float64) - want).max()}"
    rm = rowmax.cpu().numpy()
    assert np.array_equal(rm[:m], np.abs(want).max(axis=1))
    assert np.all(rm[m:] == -1.0)                                  # nothing written behind the last row
    assert s1.view(torch.float32).item() == np.abs(want).max()
    assert s2.view(torch.float32).item() == np.abs(want).max()


def test_cluster_affine_repeated_launches_agree(cuda_device, oracle):
    """Back-to-back launches under programmatic dependent launch, alternating shapes: no stale shared-memory state."""
    for i in range(6):
        _affine(cuda_device, oracle, 512 if i % 2 else 96, 1024, 1024 if i % 3 else 4096, seed=i)
