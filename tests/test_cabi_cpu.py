"""CPU checks of the C-ABI library: it loads, exports every function include/qagg.h declares, the layout helpers
agree with the oracle, and compute entry points fail loudly (never silently fall back) when there is no CUDA device."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from cntk_b200 import build
    build.build()
    from cntk_b200 import lib as L
    return L


def declared_functions():
    text = open(os.path.join(ROOT, "include", "qagg.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qagg_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_all_exported(lib):
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib.raw(), n), f"libqagg.so does not export {n}"
    assert sorted(lib.EXPORTS) == names, "cntk_b200.lib.EXPORTS is out of date with include/qagg.h"


def test_layout_helpers_match_oracle(lib, oracle_port):
    for M in (0, 1, 7, 31, 32, 33, 64, 70, 1000, 2048, 9304, 50000):
        for bits in (1, 2, 4, 8, 16, 32):
            assert lib.packed_col_bytes(M, bits) == oracle_port.packed_col_bytes(M, bits)
            assert lib.packed_bytes(M, 13, bits) == 13 * oracle_port.packed_col_bytes(M, bits)
    for N in (0, 1, 3, 8, 9, 429, 2048, 50000):
        for K in (1, 2, 3, 8, 16):
            for r in range(K):
                assert lib.stripe(N, r, K) == oracle_port.stripe(N, r, K)


def test_bad_arguments(lib):
    with pytest.raises(lib.QaggError):
        lib.packed_col_bytes(10, 3)
    with pytest.raises(lib.QaggError):
        lib.stripe(10, 4, 4)
    with pytest.raises(lib.QaggError):
        lib.quantize(16, 16, 16, 16, 8, 8, 5, True)
    assert "power of two" in lib.last_error()
    with pytest.raises(lib.QaggError):
        lib.stream_wait_selftest(10, 0)        # no status word
    with pytest.raises(lib.QaggError):
        lib.stream_wait_selftest(0, 16)        # at least one poll


def test_no_cpu_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(lib.QaggError) as e:
        lib.quantize(16, 16, 16, 16, 8, 8, 1, True)
    assert "qagg error -2" in str(e.value)
    with pytest.raises(lib.QaggError):
        lib.Comm.create(None, 0, 1, 0)
    with pytest.raises(lib.QaggError) as e:
        lib.stream_wait_selftest(10, 16)       # valid arguments, but no device to launch on
    assert "qagg error -2" in str(e.value)
