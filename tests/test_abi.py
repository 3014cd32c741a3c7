"""CPU tests of the boundary: the shared object loads, exports every symbol the header declares,
and its host-side logic (planning, argument checks, status text) behaves without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols(header="marian_i8.h", prefix="mi8_"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(" + prefix + r"[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import marian_dev_b200 as pkg
    from marian_dev_b200.binding import EXPORTS
    assert os.path.exists(pkg.LIB_PATH), "build the library first (python __graft_entry__.py)"
    L = ctypes.CDLL(pkg.LIB_PATH)
    declared = _declared_symbols()
    assert declared, "no declarations parsed from the header"
    for sym in declared:
        assert hasattr(L, sym), f"{sym} declared in include/marian_i8.h but not exported"
    assert sorted(EXPORTS) == declared
    from marian_dev_b200.binding import DECODE_EXPORTS
    declared_decode = _declared_symbols("marian_i8_decode.h", "mi8[dg]_")
    assert declared_decode
    for sym in declared_decode:
        assert hasattr(L, sym), f"{sym} declared in include/marian_i8_decode.h but not exported"
    assert sorted(DECODE_EXPORTS) == declared_decode
    from marian_dev_b200.binding import PACKED8_EXPORTS
    declared_p8 = _declared_symbols("marian_packed8.h", "mi8p_")
    assert declared_p8
    for sym in declared_p8:
        assert hasattr(L, sym), f"{sym} declared in include/marian_packed8.h but not exported"
    assert sorted(PACKED8_EXPORTS) == declared_p8
    from marian_dev_b200.binding import MEASURE_EXPORTS
    declared_measure = _declared_symbols("marian_i8_measure.h", "mi8d?_")
    assert declared_measure
    for sym in declared_measure:
        assert hasattr(L, sym), f"{sym} declared in include/marian_i8_measure.h but not exported"
    assert sorted(MEASURE_EXPORTS) == declared_measure


def test_strerror_and_version():
    from marian_dev_b200.binding import lib
    L = lib()
    assert L.mi8_version() >= 100
    assert L.mi8_strerror(0) == b"ok"
    texts = {L.mi8_strerror(i) for i in range(8)}
    assert len(texts) == 8 and b"unknown status" not in texts
    assert L.mi8_strerror(99) == b"unknown status"


@pytest.mark.parametrize("m,expect_tile", [(1, 16), (16, 16), (17, 32), (64, 64), (65, 32), (128, 32), (200, 32), (512, 32), (1024, 64), (2048, 128)])
def test_plan_tile_choice(m, expect_tile):
    from marian_dev_b200 import multiply_plan
    p = multiply_plan(m, 1024, 1024)
    assert p["tile_m"] == expect_tile
    assert p["n_tiles"] == 8 and p["m_tiles"] == (m + expect_tile - 1) // expect_tile
    assert 1 <= p["splits"] <= 8
    assert p["grid"] <= p["sm_count"]
    assert p["smem_bytes"] <= 227 * 1024


def test_plan_cta_pair_choice():
    """Enough 128 x 256 tiles for every SM and K >= 1024: the two-CTA kernel (reported as tile 512) with
    tiles of 256 x 256 per cluster; shorter K or too few tiles stay on the single-CTA kernel."""
    from marian_dev_b200 import multiply_plan
    p = multiply_plan(8192, 4096, 1024)
    assert p["tile_m"] == 512 and p["splits"] == 1 and p["n_tiles"] == 16 and p["m_tiles"] == 32
    assert p["grid"] % 2 == 0 and p["grid"] <= p["sm_count"] and p["smem_bytes"] <= 227 * 1024
    assert multiply_plan(8192, 4096, 512)["tile_m"] == 256
    assert multiply_plan(512, 4096, 1024)["tile_m"] == 128
    assert multiply_plan(300, 384, 256, 512)["tile_m"] == 512      # forced
    assert multiply_plan(300, 384, 256, 512)["n_tiles"] == 2


def test_plan_covers_k_without_empty_splits():
    from marian_dev_b200 import multiply_plan
    for k in (64, 128, 192, 1040, 4096):
        for splits in (1, 2, 3, 5, 8):
            kb = (k + 127) // 128
            if splits > kb:
                with pytest.raises(Exception):
                    multiply_plan(8, 256, k, 0, splits)
                continue
            p = multiply_plan(8, 256, k, 0, splits)
            per = (kb + p["splits"] - 1) // p["splits"]
            assert (p["splits"] - 1) * per < kb <= p["splits"] * per


def test_plan_rejects_bad_arguments():
    from marian_dev_b200 import Mi8Error, multiply_plan
    for bad in [(0, 8, 64), (8, 0, 64), (8, 8, 0)]:
        with pytest.raises(Mi8Error):
            multiply_plan(*bad)
    with pytest.raises(Mi8Error):
        multiply_plan(8, 8, 64, 48, 0)  # tile width that does not exist


def test_workspace_size_bound():
    from marian_dev_b200.binding import lib
    L = lib()
    upper = L.mi8_workspace_bytes(0, 0, 0)
    for (m, n, k) in [(1, 512, 512), (16, 1024, 1024), (512, 32000, 1024), (4096, 4096, 4096), (8, 256, 4096)]:
        assert L.mi8_workspace_bytes(m, n, k) <= upper


def test_null_and_misaligned_arguments_are_rejected_before_any_launch():
    from marian_dev_b200.binding import lib
    L = lib()
    assert L.mi8_multiply_i8(None, None, 4, 8, 64, None, None, 1.0, None, 0, None, 0, None, None, 0, None) == 1
    assert L.mi8_multiply_i8(16, 32, 4, 8, 40, 48, 64, 1.0, None, 0, 80, 0, None, None, 0, None) == 2   # K % 16
    assert L.mi8_multiply_i8(17, 32, 4, 8, 64, 48, 64, 1.0, None, 0, 80, 0, None, None, 0, None) == 2   # pointer
    assert L.mi8_multiply_i8(16, 32, 4, 8, 64, 48, 64, 1.0, None, 0, 80, 7, None, None, 0, None) == 1   # dtype
    assert L.mi8_multiply_i8(16, 32, 0, 8, 64, 48, 64, 1.0, None, 0, 80, 0, None, None, 0, None) == 0   # M = 0 is a no-op
    assert L.mi8_max_absolute_f32(None, 16, None, None, None, 0, None) == 1
    assert L.mi8_max_absolute_f32(16, 16, None, None, None, 0, None) == 4                                # no workspace
    assert L.mi8_workspace_init(None, 0, None) == 4
    assert L.mi8_prepare_a_f32(16, -1, 8, 32, 48, 64, 1 << 20, None) == 1


def test_new_entry_points_reject_bad_arguments_before_any_launch():
    """Argument checks of the entry points without a reference counterpart run on the host: no device is needed."""
    from marian_dev_b200.binding import lib
    L = lib()
    # mi8_multiply_f32_slot: null pointers, K % 16, misaligned activation, bad dtype; M = 0 is a no-op
    assert L.mi8_multiply_f32_slot(None, None, None, None, 4, 8, 64, None, 1.0, None, 0, None, 0, None, None) == 1
    assert L.mi8_multiply_f32_slot(16, 32, None, 48, 4, 8, 40, 64, 1.0, None, 0, 80, 0, None, None) == 2
    assert L.mi8_multiply_f32_slot(20, 32, None, 48, 4, 8, 64, 64, 1.0, None, 0, 80, 0, None, None) == 2
    assert L.mi8_multiply_f32_slot(16, 32, None, 48, 4, 8, 64, 64, 1.0, None, 0, 80, 9, None, None) == 1
    assert L.mi8_multiply_f32_slot(16, 32, None, 48, 0, 8, 64, 64, 1.0, None, 0, 80, 0, None, None) == 0
    # a shape that does not give every CTA one tile is declined (MI8_ERR_UNSUPPORTED), not launched
    assert L.mi8_multiply_f32_slot(16, 32, None, 48, 8192, 8192, 64, 64, 1.0, None, 0, 80, 0, None, None) == 3
    # mi8_multiply_i8_rows_from: the two device words are mandatory, the row limit cannot be negative
    assert L.mi8_multiply_i8_rows_from(16, 32, 4, 8, 64, 48, 64, 1.0, None, 0, 80, 0, None, 0, None, None, None, 0, 0) == 1
    assert L.mi8_multiply_i8_rows_from(16, 32, 4, 8, 64, 48, 64, 1.0, None, 0, 80, 0, None, 0, None, 96, 112, -1, 0) == 1
    # mi8_measure_int8_peak: iteration count and output pointer
    assert L.mi8_measure_int8_peak(0, None, None) == 1
    # fused output layer: scratch too small, k out of range
    assert L.mi8g_output_scratch_bytes(512, 32000) == 512 * 250 * 18 * 4
    assert L.mi8g_output_topk(16, 32, 48, 64, 8, 256, 64, 80, 4, None, 96, 16, None, 112, 128, None) == 4
    assert L.mi8g_output_topk(16, 32, 48, 64, 8, 256, 64, 80, 9, None, 96, 1 << 20, None, 112, 128, None) == 1
