"""Parity of the packed8avx512 CUDA path (through the C ABI of include/marian_packed8.h): bit-exact against the
fixtures the reference's own compiled mjdgemm wrote, against that library itself where the run has it, and
against the CPU checker on shapes the reference does not instantiate."""
import os

import numpy as np
import pytest
import torch

from oracle.oracle import Packed8Item, Packed8Oracle, RefMjdgemm
from tests.test_packed8_oracle import GOLDEN, _gen, _same_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def chk():
    o = Packed8Oracle()
    o.set_threads(os.cpu_count() or 1)
    return o


def _p8():
    from marian_dev_b200 import packed8
    return packed8


def _healthy():
    from marian_dev_b200 import ops
    assert ops.poll_status() == 0


def _gpu_affine(dev, a, item, bias, relu=False, **kw):
    p8 = _p8()
    w = p8.Packed8Weight(item.packed, item.K, item.N, device=dev)
    at = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    bt = torch.from_numpy(bias).to(dev) if bias is not None else None
    aq, sa, za, su = p8.quantize_rows(at)
    c, acc = p8.multiply(aq, sa, za, su, w, bt, relu=relu, want_acc=True, **kw)
    torch.cuda.synchronize()
    _healthy()
    return c.cpu().numpy(), acc.cpu().numpy(), (aq.cpu().numpy(), sa.cpu().numpy(), za.cpu().numpy(), su.cpu().numpy()), w


def test_stored_reference_outputs(cuda_device):
    g = np.load(GOLDEN)
    item = Packed8Item(g["full_packed"], 512, 512)
    c, _, _, _ = _gpu_affine(cuda_device, g["full_a"], item, g["full_bias"])
    assert _same_bits(c, g["full_c_bias"])
    c, _, _, _ = _gpu_affine(cuda_device, g["full_a"], item, None)
    assert _same_bits(c, g["full_c_nobias"])


def test_hashed_reference_outputs(cuda_device, chk):
    g = np.load(GOLDEN)
    ran = 0
    for line in g["hashed_cases"]:
        seed, M, N, K, h_in, h_packed, h_out = str(line).split()
        w, a, bias = _gen.inputs(int(seed), int(M), int(K), int(N))
        if _gen.sha(w, a, bias) != h_in:
            continue
        item = chk.prepare_b(w)
        assert _gen.sha(item.packed) == h_packed
        p8 = _p8()
        wt = p8.Packed8Weight(item.packed, item.K, item.N, device=cuda_device)
        c = p8.gemmInt8Packed(torch.from_numpy(a).to(cuda_device), wt, torch.from_numpy(bias).to(cuda_device))
        torch.cuda.synchronize()
        _healthy()
        assert _gen.sha(c.cpu().numpy()) == h_out, (M, N, K)
        ran += 1
    if ran == 0:
        pytest.skip("seeded inputs differ under this NumPy")


def test_unpack_and_row_quantisation_bit_exact(cuda_device, chk):
    w, a, bias = _gen.inputs(11, 37, 768, 160)
    a[5] = 0.0
    a[6] = -2.5
    item = chk.prepare_b(w)
    c, acc, (aq, sa, za, su), wt = _gpu_affine(cuda_device, a, item, bias)
    assert np.array_equal(wt.bt.cpu().numpy(), chk.unpack_bt(item))
    oq, osa, oza, osu = chk.quantize_rows(a)
    assert np.array_equal(aq, oq) and _same_bits(sa, osa) and np.array_equal(za, oza) and np.array_equal(su, osu)
    oc, oacc = chk.affine(a, item, bias, want_acc=True)
    assert np.array_equal(acc, oacc)
    assert _same_bits(c, oc)


@pytest.mark.parametrize("M,N,K", [(1, 512, 512), (4, 1024, 1024), (57, 4096, 1024), (200, 1024, 4096), (300, 3072, 1024),
                                   (512, 512, 8192), (1000, 1024, 512), (16, 32000, 512), (2100, 4096, 1024)])
@pytest.mark.parametrize("relu", [False, True])
def test_against_checker_on_reference_shapes(cuda_device, chk, M, N, K, relu):
    w, a, bias = _gen.inputs(M + N + K, M, K, N)
    item = chk.prepare_b(w)
    c, acc, _, _ = _gpu_affine(cuda_device, a, item, bias, relu=relu)
    oc, oacc = chk.affine(a, item, bias, relu=relu, want_acc=True)
    assert np.array_equal(acc, oacc)
    assert _same_bits(c, oc)
    try:
        ref = RefMjdgemm()
    except FileNotFoundError:
        return
    if ref.isa() in (5, 6) and not relu:
        assert _same_bits(c, ref.gemm(a, item, bias))


@pytest.mark.parametrize("tile_m,splits", [(16, 0), (32, 0), (64, 0), (128, 0), (256, 0), (512, 0), (0, 2), (0, 4), (64, 8)])
def test_every_tile_width_and_split(cuda_device, chk, tile_m, splits):
    # tile_m 512 = the two-CTA kernel (tcgen05.mma.cta_group::2 with an unsigned activation operand)
    w, a, bias = _gen.inputs(77, 130, 1024, 288)
    item = chk.prepare_b(w)
    c, acc, _, _ = _gpu_affine(cuda_device, a, item, None, tile_m=tile_m, splits=splits)
    oc, oacc = chk.affine(a, item, None, want_acc=True)
    assert np.array_equal(acc, oacc)
    assert _same_bits(c, oc)


def test_one_call_entry_and_argument_checks(cuda_device, chk):
    from marian_dev_b200.binding import lib
    p8 = _p8()
    w, a, bias = _gen.inputs(5, 8, 256, 64)
    item = chk.prepare_b(w)
    wt = p8.Packed8Weight(item.packed, 256, 64, device=cuda_device)
    at, bt = torch.from_numpy(a).to(cuda_device), torch.from_numpy(bias).to(cuda_device)
    c = p8.gemmInt8Packed(at, wt, bt)
    torch.cuda.synchronize()
    assert _same_bits(c.cpu().numpy(), chk.affine(a, item, bias))
    assert p8.gemmInt8Packed(at[:0], wt, bt).shape == (0, 64)
    L = lib()
    out = torch.empty((300, 300), dtype=torch.int8, device=cuda_device)
    assert L.mi8p_unpack_b(wt.item.data_ptr(), 300, 64, out.data_ptr(), None) == 3       # K % 256 != 0: unsupported
    assert L.mi8p_unpack_b(None, 256, 64, out.data_ptr(), None) == 1
    assert L.mi8p_gemm_int8_packed(at.data_ptr(), wt.bt.data_ptr(), wt.scale_b.data_ptr(), wt.zp_b.data_ptr(), wt.off_b.data_ptr(),
                                   None, c.data_ptr(), 8, 64, 256, None, 0, None, 0, None) != 0   # no scratch
    _healthy()


@pytest.mark.parametrize("K,N", [(256, 32), (512, 512), (1024, 96), (1536, 256)])
def test_weight_conversion_bit_exact_and_container_round_trip(cuda_device, chk, tmp_path, K, N):
    from marian_dev_b200 import binary_io as bio
    p8 = _p8()
    rng = np.random.default_rng(K + N)
    w = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    w[:, 3] = 0.25                                            # a constant column
    w[:, 5] = np.abs(w[:, 5])                                 # a one-sided column
    want = chk.prepare_b(w)
    got = p8.prepareB(torch.from_numpy(w).to(cuda_device))
    torch.cuda.synchronize()
    _healthy()
    assert np.array_equal(got.item.cpu().numpy(), want.packed)          # weights, scales, zero points, column offsets
    assert np.array_equal(got.bt.cpu().numpy(), chk.unpack_bt(want))
    # marian-conv --gemm-type packed8avx512, then load: the affine on the loaded item equals the checker's
    items = bio.convert({"encoder_l1_ffn_W1": w, "encoder_l1_ffn_b1": np.zeros((1, N), np.float32)}, "type: transformer\n",
                        gemm_type="packed8avx512", device=cuda_device)
    path = str(tmp_path / "model.bin")
    bio.save_items(path, items)
    _, params = bio.items_to_params(bio.load_items(path), device=cuda_device)
    wt = params["encoder_l1_ffn_W1"]
    assert isinstance(wt, p8.Packed8Weight) and params["encoder_l1_ffn_b1"].dtype == np.float32
    a = rng.standard_normal((9, K)).astype(np.float32)
    c = p8.gemmInt8Packed(torch.from_numpy(a).to(cuda_device), wt)
    torch.cuda.synchronize()
    assert _same_bits(c.cpu().numpy(), chk.affine(a, want, None))
    from marian_dev_b200.binding import lib
    assert lib().mi8p_prepare_b_f32(got.item.data_ptr(), 100, 32, got.item.data_ptr(), None) == 3


def test_row_shards_need_no_exchange(cuda_device, chk):
    from marian_dev_b200 import parallel
    p8 = _p8()
    w, a, bias = _gen.inputs(123, 301, 512, 256)
    item = chk.prepare_b(w)
    wt = p8.Packed8Weight(item.packed, 512, 256, device=cuda_device)
    bt = torch.from_numpy(bias).to(cuda_device)
    whole = p8.gemmInt8Packed(torch.from_numpy(a).to(cuda_device), wt, bt).cpu().numpy()
    for world in (2, 3, 8):
        parts = []
        for rank in range(world):
            r0, r1 = parallel.shard_rows(301, rank, world)
            parts.append(parallel.sharded_packed8_affine(torch.from_numpy(a[r0:r1]).to(cuda_device), wt, bt).cpu().numpy())
        assert _same_bits(np.concatenate(parts), whole)
    _healthy()
