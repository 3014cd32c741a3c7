"""CPU tests of the packed8avx512 checker: pinned against the reference's own compiled mjdgemm when
oracle/_ref holds it, and always against the fixtures that library produced."""
import hashlib
import importlib.util
import os

import numpy as np
import pytest

from oracle.oracle import Packed8Item, Packed8Oracle, RefMjdgemm

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "packed8_golden.npz")

_spec = importlib.util.spec_from_file_location("make_packed8_golden", os.path.join(ROOT, "tests", "golden", "make_packed8_golden.py"))
_gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_gen)


def _same_bits(x, y):
    return np.array_equal(np.ascontiguousarray(x).view(np.uint32), np.ascontiguousarray(y).view(np.uint32))


@pytest.fixture(scope="module")
def chk():
    o = Packed8Oracle()
    o.set_threads(os.cpu_count() or 1)
    return o


def _reference_or_skip():
    try:
        ref = RefMjdgemm()
    except FileNotFoundError:
        pytest.skip("oracle/_ref/libref_mjdgemm.so not built (needs the reference tree: make -C oracle ref)")
    if ref.isa() not in (5, 6):
        pytest.skip("this host does not take the reference's AVX-512 route")
    return ref


def test_restatement_matches_the_stored_reference_outputs(chk):
    g = np.load(GOLDEN)
    item = Packed8Item(g["full_packed"], 512, 512)
    assert _same_bits(chk.affine(g["full_a"], item, g["full_bias"]), g["full_c_bias"])
    assert _same_bits(chk.affine(g["full_a"], item, None), g["full_c_nobias"])


def test_restatement_matches_the_hashed_reference_outputs(chk):
    g = np.load(GOLDEN)
    ran = 0
    for line in g["hashed_cases"]:
        seed, M, N, K, h_in, h_packed, h_out = str(line).split()
        w, a, bias = _gen.inputs(int(seed), int(M), int(K), int(N))
        if _gen.sha(w, a, bias) != h_in:
            continue   # this NumPy draws other random numbers than the one that wrote the fixture
        item = chk.prepare_b(w)
        assert _gen.sha(item.packed) == h_packed
        assert _gen.sha(chk.affine(a, item, bias)) == h_out
        ran += 1
    if ran == 0:
        pytest.skip("seeded inputs differ under this NumPy")


def test_block_order_round_trip(chk):
    rng = np.random.default_rng(3)
    b = rng.integers(-64, 64, size=(512, 96), dtype=np.int8)
    packed = chk.pack_b(b)
    # element (k, n) sits at [k/256][n/32][(k%256)/4][n%32][k%4]
    blocks = packed.reshape(2, 3, 64, 32, 4)
    assert blocks[1, 2, 5, 7, 3] == b[256 + 5 * 4 + 3, 64 + 7]
    tail = np.zeros(12 * 96, np.int8)
    bt = chk.unpack_bt(Packed8Item(np.concatenate([packed, tail]), 512, 96))
    assert np.array_equal(bt, b.T)


def test_row_statistics_and_edge_rows(chk):
    a = np.zeros((4, 256), np.float32)
    a[1] = 0.75                      # constant row: the reference divides by zero, here the range is widened to [0, 0.75]
    a[2] = np.linspace(-2, 6, 256)
    a[3] = -np.linspace(0, 3, 256)
    aq, sa, za, su = chk.quantize_rows(a)
    assert sa[0] == 1.0 and za[0] == 255 and np.all(aq[0] == 255)
    assert np.all(aq[1] == 255) and za[1] == 0 and np.isclose(sa[1], 0.75 / 255)
    assert aq[2].min() == 0 and aq[2].max() >= 254      # the zero point is truncated, not rounded
    assert su.tolist() == aq.astype(np.int64).sum(1).tolist()
    # dequantised rows come back within one step (half a step of rounding, up to one of clipping at the low end)
    deq = (aq.astype(np.float32) - za[:, None]) * sa[:, None]
    assert np.all(np.abs(deq - a) <= sa[:, None] + 1e-6)


def test_affine_is_close_to_float_and_m0(chk):
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((256, 64)) * 0.05).astype(np.float32)
    a = rng.standard_normal((9, 256)).astype(np.float32)
    bias = rng.standard_normal(64).astype(np.float32)
    item = chk.prepare_b(w)
    c, acc = chk.affine(a, item, bias, want_acc=True)
    assert np.abs(c - (a @ w + bias)).max() < 0.05
    assert acc.dtype == np.int32
    assert _same_bits(chk.affine(a, item, bias, relu=True), np.maximum(c, 0))
    assert chk.affine(np.zeros((0, 256), np.float32), item, bias).shape == (0, 64)


@pytest.mark.parametrize("N,K", [(512, 512), (1024, 512), (512, 1024), (3072, 1024), (8192, 512)])
def test_against_the_compiled_reference(chk, N, K):
    ref = _reference_or_skip()
    rng = np.random.default_rng(N + K)
    for M in (1, 7, 49, 100):
        w, a, bias = _gen.inputs(int(rng.integers(1 << 30)), M, K, N)
        item = chk.prepare_b(w)
        assert np.array_equal(ref.pack_b(np.ascontiguousarray(chk.unpack_bt(item).T)), item.packed[:K * N])
        assert _same_bits(chk.affine(a, item, bias), ref.gemm(a, item, bias))
        assert _same_bits(chk.affine(a, item, None), ref.gemm(a, item, None))
