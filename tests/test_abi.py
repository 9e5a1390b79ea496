"""CPU: the C-ABI library loads, exports every symbol the header declares, and
rejects contract violations on the host before any launch (so these calls are
safe without a GPU)."""
from __future__ import annotations

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "escha_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(escha_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    from escha_mlx_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 15
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names, "binding lists a symbol the header does not declare"


def test_version():
    from escha_mlx_b200 import _lib
    assert _lib.lib.escha_version() == 1


def test_host_side_validation_raises_value_error():
    from escha_mlx_b200._lib import check, lib
    fake = ctypes.c_void_p(0x1000)  # aligned, never dereferenced: validation fails first
    with pytest.raises(ValueError, match="K=4"):
        check(lib.escha_decode_tiles(fake, 4, 128, 128, None, fake, None))
    with pytest.raises(ValueError, match="multiples of 16"):
        check(lib.escha_decode_tiles(fake, 2, 100, 128, None, fake, None))
    with pytest.raises(ValueError, match="multiples of 128"):
        check(lib.escha_coded_gemv(fake, fake, None, 1, 256, 144, 2, 1, 0.5, None, 0, fake, None))
    with pytest.raises(ValueError, match="at least one row"):
        check(lib.escha_coded_gemv(fake, fake, None, 0, 256, 128, 2, 1, 0.5, None, 0, fake, None))
    with pytest.raises(ValueError, match="NULL"):
        check(lib.escha_coded_gemv(None, fake, None, 1, 256, 128, 2, 1, 0.5, None, 0, fake, None))
    with pytest.raises(ValueError, match="16-byte aligned"):
        check(lib.escha_scaled_had(ctypes.c_void_p(0x1004), fake, None, 1, 128, 0.5, fake, None))
    with pytest.raises(ValueError, match="divisible by 128"):
        check(lib.escha_scaled_had(fake, fake, None, 1, 192, 0.5, fake, None))
    with pytest.raises(ValueError, match="does not divide"):
        check(lib.escha_gemv_ref(fake, fake, None, None, 0, None, 1, 128, 128, 2, 3, fake, fake, None))
    with pytest.raises(ValueError, match="workspace"):
        check(lib.escha_coded_gemv(fake, fake, None, 1, 512, 128, 2, 2, 0.5, fake, 16, fake, None))
    with pytest.raises(ValueError, match="rows per job"):
        check(lib.escha_moe_group_rows(fake, 8, 4, 5, fake, 100, None, None))
    # host tables of the joint int8 launch: plain arrays, no alignment demanded of the tables
    tab = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    widths = (ctypes.c_int * 2)(64, 24)
    with pytest.raises(ValueError, match="1..4 linears"):
        check(lib.escha_w8a16_many(fake, 5, tab, tab, widths, 128, 1, tab, None))
    with pytest.raises(ValueError, match="multiple of 64"):
        check(lib.escha_w8a16_many(fake, 2, tab, tab, widths, 96, 1, tab, None))
    with pytest.raises(ValueError, match="multiples of 16"):
        check(lib.escha_w8a16_many(fake, 2, tab, tab, widths, 128, 1, tab, None))


def test_pure_helpers():
    from escha_mlx_b200._lib import lib
    assert lib.escha_moe_jobs_bound(512, 256, 8) == (512 + 256 * 7) // 8
    assert lib.escha_moe_jobs_bound(8, 256, 8) == 8
    # 4096x4096: 32 output blocks -> floor(3*148/32) = 13 splits fill a 148-SM part's
    # 444 resident-CTA slots without exceeding them
    assert lib.escha_coded_gemv_splits(4096, 4096, 1, 148) == 13
    assert lib.escha_coded_gemv_splits(5120, 17408, 1, 148) == 3
    assert lib.escha_coded_gemv_splits(17408, 5120, 1, 148) == 11
    assert lib.escha_coded_gemv_splits(5120, 17408 * 4, 1, 148) == 1
    # never fewer than two 128-channel blocks per split
    assert lib.escha_coded_gemv_splits(512, 128, 1, 148) == 2
    assert lib.escha_coded_gemv_workspace_bytes(1, 4096, 1, 8) == 0
    assert lib.escha_coded_gemv_workspace_bytes(1, 4096, 4, 8) == (1 << 20) + 4 * 32 * 8 * 128 * 4
