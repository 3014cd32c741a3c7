"""CPU tests: the two restatements of the reference path agree with each other and with the
known-answer vectors available for it.

No test in the reference uses an intgemm-typed operand, so the only reference-held vectors that
apply are the float operator contracts of src/tests/units/operator_tests.cpp:508-534,618-659
(dot / affine / affineWithReluDropout on small integer-valued matrices).  Those inputs are exactly
representable after quantisation when the largest magnitude maps to 127 without rounding, which the
cases below arrange, so the int8 path must reproduce the float answers to within float rounding.
"""
import json
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_c_and_numpy_restatements_agree(oracle):
    rng = np.random.default_rng(0)
    for (m, k, n) in [(1, 64, 8), (7, 128, 24), (256, 512, 2048), (33, 1040, 136)]:
        a = rng.standard_normal((m, k)).astype(np.float32)
        w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
        bias = (rng.standard_normal(n) * 0.01).astype(np.float32)
        bt_c, qb_c = oracle.prepare_b(w)
        bt_n, qb_n = O.numpy_prepare_b(w)
        assert qb_c == qb_n and np.array_equal(bt_c, bt_n)
        for relu in (False, True):
            out_c, acc_c, aq_c, qa_c = oracle.affine(a, bt_c, qb_c, bias, 0.5, relu, want_acc=True)
            out_n, acc_n, aq_n, qa_n = O.numpy_affine(a, bt_n, qb_n, bias, 0.5, relu)
            assert qa_c == qa_n
            assert np.array_equal(aq_c, aq_n) and np.array_equal(acc_c, acc_n)
            assert np.array_equal(out_c, out_n)


def test_threads_do_not_change_results(oracle):
    rng = np.random.default_rng(1)
    a = rng.integers(-127, 128, (37, 256)).astype(np.int8)
    b = rng.integers(-127, 128, (50, 256)).astype(np.int8)
    oracle.set_threads(1)
    r1 = oracle.multiply_i32(a, b)
    oracle.set_threads(4)
    r4 = oracle.multiply_i32(a, b)
    oracle.set_threads(1)
    assert np.array_equal(r1, r4)
    assert np.array_equal(r1, a.astype(np.int64) @ b.astype(np.int64).T)


def test_multiply_routes_agree_with_exact_integer_product(oracle):
    """The vectorised routes of the checker's int8 multiply (AVX512-VNNI with the +128 shift, AVX2 with 16-bit
    widening) and the portable loop all equal the exact integer product, extreme values and ragged K included."""
    rng = np.random.default_rng(3)
    best = oracle.set_isa(-1)
    try:
        for (m, k, n) in [(7, 208, 33), (33, 1040, 130), (5, 64, 1), (1, 16, 3), (9, 4096, 17)]:
            a = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
            bt = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
            a[0, :] = 127
            bt[0, :] = -127
            want = a.astype(np.int64) @ bt.astype(np.int64).T
            for isa in range(best + 1):
                assert oracle.set_isa(isa) == isa
                for threads in (1, 3):
                    oracle.set_threads(threads)
                    assert np.array_equal(oracle.multiply_i32(a, bt).astype(np.int64), want), (m, k, n, isa, threads)
    finally:
        oracle.set_isa(-1)
        oracle.set_threads(1)


def test_quantise_rounding_and_saturation(oracle):
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, 127.0, -127.0, 300.0, -300.0, 0.49999997], dtype=np.float32)
    want = np.array([0, 2, 2, 0, -2, -2, 126, 127, -127, 127, -127, 0], dtype=np.int8)
    assert np.array_equal(oracle.quantize(x, np.float32(1.0)), want)
    assert np.array_equal(O.numpy_quantize(x, np.float32(1.0)), want)
    assert oracle.quant_mult(np.zeros(8, np.float32)) == 1.0
    assert O.numpy_quant_mult(np.zeros(8, np.float32)) == 1.0
    assert oracle.quant_mult(np.array([-2.0, 1.0], np.float32)) == np.float32(127.0) / np.float32(2.0)


def test_reference_float_operator_vectors(oracle):
    """Known answers shaped like the reference's operator tests: small integer matrices whose
    quantisation is exact, so the int8 path must return the float product."""
    a = np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9], [10, 11, 12]], dtype=np.float32)       # 4 x 3
    b = np.array([[1, 2], [3, 4], [5, 6]], dtype=np.float32)                               # 3 x 2
    bias = np.array([2, 3], dtype=np.float32)
    # scale both so max|.| = 127 exactly: the multipliers become 1 and nothing is rounded
    a_s, b_s = a * np.float32(127.0 / 12.0), b * np.float32(127.0 / 6.0)
    # pad K to a multiple of 4 with zeros (does not change the product)
    a_p = np.zeros((4, 4), np.float32); a_p[:, :3] = a_s
    b_p = np.zeros((4, 2), np.float32); b_p[:3] = b_s
    bt, qb = oracle.prepare_b(b_p)
    out = oracle.affine(a_p, bt, qb, bias, 1.0, False)
    want = a_s @ b_s + bias
    assert np.allclose(out, want, rtol=2e-2, atol=0)
    out_relu = oracle.affine(-a_p, bt, qb, bias, 1.0, True)
    assert np.array_equal(out_relu, np.maximum(oracle.affine(-a_p, bt, qb, bias, 1.0, False), 0))


def test_sat16_emulation_matches_exact_on_small_values(oracle):
    rng = np.random.default_rng(3)
    a = rng.integers(-20, 21, (5, 64)).astype(np.int8)
    b = rng.integers(-20, 21, (9, 64)).astype(np.int8)
    assert np.array_equal(oracle.multiply_i32(a, b, sat16=True), oracle.multiply_i32(a, b))
    # and saturates where the exact path does not
    a[:] = 127
    b[:] = 127
    assert (oracle.multiply_i32(a, b, sat16=True) < oracle.multiply_i32(a, b)).all()


def test_golden_fixtures(oracle):
    """Committed fixtures (tests/golden/make_golden.py): inputs are regenerated from the seed, the
    oracle's outputs must hash to the committed digests."""
    path = os.path.join(GOLDEN, "affine_golden.json")
    if not os.path.exists(path):
        pytest.skip("golden fixtures not generated")
    from tests.golden.make_golden import cases, digest, run_case
    want = json.load(open(path))
    for name, spec in cases().items():
        got = run_case(oracle, spec)
        assert {k: digest(v) for k, v in got.items()} == want[name]["sha256"], name
