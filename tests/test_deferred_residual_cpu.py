"""The deferred form of the error-feedback residual (what the streaming quantize kernel keeps between steps) restated in
numpy and checked against the oracle on CPU: keeping v = gradient + residual and the column's two reconstruction values,
and forming v - (v >= 0 ? val1 : val0) only when the state is next read, gives the oracle's residual bit for bit, step
after step; the packed bit of a value is (v >= 0) and needs no range; the count of rows below the threshold is the number
of zero bits.  Reference arithmetic: Source/Math/ColumnQuantizer.h:100-125 (1 bit, threshold 0),
Source/Math/ValueQuantizer.h:131-141 (Unquantize)."""
import numpy as np
import pytest

F = np.float32


def levels_1bit(lower, upper):
    """Unquantize(0), Unquantize(1) for Nbits = 1: ufactor = (upper - lower) / 2 (0 below 1e-36), (q + 0.5) * ufactor + lower."""
    rng = F(upper) - F(lower)
    ufactor = np.where(rng < F(1e-36), F(0), F(0.5) * rng).astype(F)
    return (F(0.5) * ufactor + F(lower)).astype(F), (F(1.5) * ufactor + F(lower)).astype(F)


def unpack_bits(packed_col, M):
    words = packed_col[8:].view(np.uint32)
    Q = words.size
    rows = np.arange(M)
    return ((words[rows % Q] >> (rows // Q).astype(np.uint32)) & 1).astype(bool)


@pytest.mark.parametrize("M,N", [(2048, 5), (291, 7), (70, 3), (33, 2), (1, 4)])
def test_deferred_state_reproduces_the_oracle_residual(oracle_port, M, N):
    rng = np.random.default_rng(1234 + M)
    C = oracle_port.packed_col_bytes(M, 1)
    res = np.zeros((N, M), F)           # oracle: plain residual
    v_state = np.zeros((N, M), F)       # deferred state: quantized value ...
    val0 = np.zeros(N, F)               # ... and the two reconstruction values per column (all zero = zero residual)
    val1 = np.zeros(N, F)
    for step in range(6):
        g = (rng.standard_normal((N, M)) * 1e-3).astype(F)
        if step == 2:
            g[0, :] = 0.0               # an all-zero column
        if step == 3:
            g[1 % N, :] = -np.abs(g[1 % N, :])  # an all-negative column
        # what the streaming kernel does when it reads the state
        r_read = (v_state - np.where(v_state >= 0, val1[:, None], val0[:, None])).astype(F)
        assert np.array_equal(r_read.view(np.uint32), res.view(np.uint32)), f"step {step}: residual read from the deferred state differs"
        v = (g + r_read).astype(F)
        # the oracle's step
        packed = np.zeros(N * C, np.uint8)
        oracle_port.quantize(g, res, res, packed, 1, True)
        cols = packed.reshape(N, C)
        for j in range(N):
            bits = unpack_bits(cols[j], M)
            assert np.array_equal(bits, v[j] >= 0), f"step {step} column {j}: the bit is (v >= 0), whatever the range"
            n0 = int(M - bits.sum())
            assert n0 == int((v[j] < 0).sum()), "rows below the threshold = zero bits"
            lower, upper = cols[j][:8].view(F)
            val0[j], val1[j] = levels_1bit(lower, upper)
        v_state = v
    # export: the plain residual of the last step
    r_final = (v_state - np.where(v_state >= 0, val1[:, None], val0[:, None])).astype(F)
    assert np.array_equal(r_final.view(np.uint32), res.view(np.uint32))
