"""CPU checks that pin the oracle: the plain-C restatement (oracle/qagg_oracle.c) must reproduce the
fixtures that tests/golden/make_golden.py wrote from the reference's own headers, the known answers
obtained from those headers, and -- when the reference-built library is present -- its output directly."""
import json
import os
import struct
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402

from oracle import exchange as ox  # noqa: E402

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def digests():
    with open(os.path.join(GOLD, "golden_digests.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def small():
    return np.load(os.path.join(GOLD, "golden_small.npz"))


def test_input_generator_has_not_drifted(digests):
    for (rows, cols, low, high, seed) in mg.UNIT_CASES:
        got = [mg.sha(mg.uniform_input(rows, cols, low, high, seed + it)) for it in range(mg.ITERS)]
        assert got == digests["inputs"][f"{rows}x{cols}_seed{seed}"], "numpy input stream changed; regenerate fixtures"


@pytest.mark.parametrize("case", mg.UNIT_CASES, ids=lambda c: f"{c[0]}x{c[1]}")
def test_port_reproduces_reference_unit_grid(oracle_port, digests, case):
    rows, cols, low, high, seed = case
    for bits in mg.BITS:
        for zero_thr in ((False, True) if bits == 1 else (False,)):
            key = f"{rows}x{cols}_seed{seed}_b{bits}_z{int(zero_thr)}"
            d, _ = mg.run_unit_case(oracle_port, rows, cols, low, high, seed, bits, zero_thr)
            assert d == digests["unit"][key], key


def test_port_matches_full_small_arrays(oracle_port, small):
    rows, cols, low, high, seed = mg.UNIT_CASES[0]
    for bits in (1, 2, 4):
        for zero_thr in ((False, True) if bits == 1 else (False,)):
            key = f"{rows}x{cols}_seed{seed}_b{bits}_z{int(zero_thr)}"
            keep = []
            mg.run_unit_case(oracle_port, rows, cols, low, high, seed, bits, zero_thr, keep)
            for it, (g, p, r, o) in enumerate(keep):
                np.testing.assert_array_equal(g, small[f"{key}_it{it}_in"])
                np.testing.assert_array_equal(p, small[f"{key}_it{it}_packed"])
                np.testing.assert_array_equal(r, small[f"{key}_it{it}_res"])
                np.testing.assert_array_equal(o, small[f"{key}_it{it}_out"])


def test_port_reproduces_config1_round_trip(oracle_port, digests):
    """2048 x 2048, N(0, 0.01^2), seed 0 + step, 1 bit, ten error-feedback steps (first three checked here to
    keep the CPU suite short; the GPU suite checks all ten)."""
    be = oracle_port
    for zero_thr in (True, False):
        res = np.zeros((2048, 2048), np.float32)
        out = np.zeros((2048, 2048), np.float32)
        packed = np.zeros(2048 * be.packed_col_bytes(2048, 1), np.uint8)
        for step in range(3):
            g = mg.normal_input(2048, 2048, 0.01, step)
            exp = digests["config1"][f"z{int(zero_thr)}"][step]
            assert mg.sha(g) == exp["in"]
            be.quantize(g, res, res, packed, 1, zero_thr)
            be.unquantize(packed, out, 1, add=False)
            assert mg.sha(packed) == exp["packed"]
            assert mg.sha(res) == exp["residual"]
            assert mg.sha(out) == exp["out"]


def test_conservation_invariant(oracle_port):
    """in + prevResidual + prevOut == newResidual + newOut within (hi - lo) * 1e-4
    (Tests/UnitTests/MathTests/MatrixQuantizerTests.cpp:327-338)."""
    be = oracle_port
    for (rows, cols, low, high, seed) in mg.UNIT_CASES:
        for bits in (1, 2, 4, 8):
            res = np.zeros((cols, rows), np.float32)
            out = np.zeros((cols, rows), np.float32)
            packed = np.zeros(cols * be.packed_col_bytes(rows, bits), np.uint8)
            for it in range(mg.ITERS):
                g = mg.uniform_input(rows, cols, low, high, seed + it)
                lhs = g + res + (out if it > 0 else 0)
                be.quantize(g, res, res, packed, bits, True)
                be.unquantize(packed, out, bits, add=(it > 0))
                assert np.max(np.abs(lhs - (res + out))) <= (high - low) * 1e-4


def _words(packed_col):
    return [struct.unpack("<I", packed_col[8 + 4 * w: 12 + 4 * w].tobytes())[0] for w in range((len(packed_col) - 8) // 4)]


def test_known_answers_from_reference_headers(oracle_port):
    be = oracle_port
    assert be.packed_col_bytes(70, 1) == 20 and be.packed_col_bytes(2048, 1) == 264
    # all-zero column, M = 70, 1 bit, zero threshold: range collapses, every real row's bit is 1, padding bits 0
    g = np.zeros((1, 70), np.float32)
    r = np.zeros((1, 70), np.float32)
    p = np.zeros(20, np.uint8)
    be.quantize(g, r, r, p, 1, True)
    assert struct.unpack("<ff", p[:8].tobytes()) == (0.0, 0.0)
    assert _words(p) == [0x00FFFFFF, 0x007FFFFF, 0x007FFFFF]
    assert not r.any()
    o = np.ones((1, 70), np.float32)
    be.unquantize(p, o, 1, add=False)
    assert not o.any()
    # M = 64, 4 bits, ramp: lower/upper = -/+ 4 * sqrt(sum v^2 / M); nibble k of word w is the level of row w + 8k
    g = ((np.arange(64, dtype=np.float32) - np.float32(31.5)) * np.float32(0.01)).reshape(1, 64)
    r = np.zeros((1, 64), np.float32)
    p = np.zeros(be.packed_col_bytes(64, 4), np.uint8)
    be.quantize(g, r, r, p, 4, True)
    lo, hi = struct.unpack("<ff", p[:8].tobytes())
    assert abs(hi - 0.738918) < 1e-6 and lo == -hi
    assert _words(p) == [0x99876554, 0xA9876654, 0xA9876654, 0xA9877654, 0xA9877654, 0xA9887654, 0xA9887654, 0xA9987655]
    # M = 64, 1 bit, mean threshold, ramp around 0.5
    g = (np.float32(0.5) + (np.arange(64, dtype=np.float32) - np.float32(31.5)) * np.float32(0.01)).reshape(1, 64)
    r = np.zeros((1, 64), np.float32)
    p = np.zeros(be.packed_col_bytes(64, 1), np.uint8)
    be.quantize(g, r, r, p, 1, False)
    lo, hi = struct.unpack("<ff", p[:8].tobytes())
    assert abs(lo - 0.18) < 1e-6 and abs(hi - 0.82) < 1e-6
    assert _words(p) == [0xFFFF0000, 0xFFFF0000]


def test_stripe_partition(oracle_port):
    for N in (0, 1, 3, 7, 8, 9, 429, 2048, 50000):
        for K in (1, 2, 3, 4, 8):
            covered = 0
            for r in range(K):
                s, n = ox.stripe(N, r, K)
                assert (s, n) == oracle_port.stripe(N, r, K)
                assert s == covered
                covered += n
            assert covered == N


@pytest.mark.parametrize("K", [1, 2, 3, 4, 8])
def test_exchange_restatement_matches_fixtures(oracle_port, digests, K):
    for bits in (1, 2, 4):
        for zero_thr in ((True, False) if bits == 1 else (True,)):
            for self_quant in (True, False):
                key = f"K{K}_b{bits}_z{int(zero_thr)}_s{int(self_quant)}"
                assert mg.run_exchange(oracle_port, K, bits, zero_thr, self_quant) == digests["exchange"][key], key


def test_exchange_all_ranks_agree_and_v2_identity(oracle_port):
    K = 3
    st = ox.ExchangeState(mg.EXCHANGE_SHAPES, K)
    grads = mg.exchange_inputs(K, 0)
    ox.aggregate_step(oracle_port, st, grads, 1)
    for i in range(len(mg.EXCHANGE_SHAPES)):
        for r in range(1, K):
            np.testing.assert_array_equal(grads[0][i], grads[r][i])
    st1 = ox.ExchangeState(mg.EXCHANGE_SHAPES, 1)
    g1 = mg.exchange_inputs(1, 0)
    keep = [a.copy() for a in g1[0]]
    assert ox.aggregate_step(oracle_port, st1, g1, 1, v2_identity_at_k1=True) is None
    for a, b in zip(g1[0], keep):
        np.testing.assert_array_equal(a, b)


def test_port_equals_reference_build_directly(oracle_port, oracle_ref):
    """Random shapes incl. odd row counts, all-zero columns, NaN-free extremes: byte-identical outputs."""
    rng = np.random.default_rng(7)
    for trial in range(40):
        M = int(rng.integers(1, 300))
        N = int(rng.integers(1, 20))
        bits = int(rng.choice([1, 2, 4, 8, 16, 32]))
        zero_thr = bool(rng.integers(0, 2))
        scale = float(10.0 ** rng.integers(-6, 2))
        res_a = np.zeros((N, M), np.float32)
        res_b = np.zeros((N, M), np.float32)
        for it in range(3):
            g = (rng.standard_normal((N, M)) * scale).astype(np.float32)
            if trial % 5 == 0:
                g[rng.integers(0, N)] = 0.0
            pa = np.zeros(N * oracle_port.packed_col_bytes(M, bits), np.uint8)
            pb = np.zeros_like(pa)
            oracle_port.quantize(g, res_a, res_a, pa, bits, zero_thr)
            oracle_ref.quantize(g, res_b, res_b, pb, bits, zero_thr)
            np.testing.assert_array_equal(pa, pb)
            np.testing.assert_array_equal(res_a.view(np.uint32), res_b.view(np.uint32))
            oa = np.full((N, M), 0.25, np.float32)
            ob_ = np.full((N, M), 0.25, np.float32)
            oracle_port.unquantize(pa, oa, bits, add=bool(it % 2))
            oracle_ref.unquantize(pb, ob_, bits, add=bool(it % 2))
            np.testing.assert_array_equal(oa.view(np.uint32), ob_.view(np.uint32))


@pytest.mark.parametrize("K", [1, 2, 3, 8])
def test_column_subset_replay_equals_full_exchange(oracle_port, K):
    """aggregate_columns (what the full-size and multi-GPU checks replay for sampled columns) reproduces aggregate_step
    column for column: aggregates, residuals, stripe residuals and packed columns, over three error-feedback steps."""
    rng = np.random.default_rng(11 + K)
    shapes = [(70, 19), (33, 5), (128, 1), (5, 16)]
    for bits, zero_thr, self_q in ((1, True, True), (1, False, True), (4, True, True), (1, True, False)):
        st = ox.ExchangeState(shapes, K)
        sub_res = [[np.zeros((N, M), np.float32) for (M, N) in shapes] for _ in range(K)]
        sub_sres = [np.zeros((N, M), np.float32) for (M, N) in shapes]  # indexed by global column
        for step in range(3):
            grads = [[(rng.standard_normal((N, M)) * 1e-2).astype(np.float32) for (M, N) in shapes] for _ in range(K)]
            keep = [[a.copy() for a in grads[r]] for r in range(K)]
            packed = ox.aggregate_step(oracle_port, st, grads, bits, zero_thr, self_q)
            for i, (M, N) in enumerate(shapes):
                C = oracle_port.packed_col_bytes(M, bits)
                for owner in range(K):
                    cols = [c for c in range(N) if ox.owner_of(c, N, K) == owner]
                    s, n = ox.stripe(N, owner, K)
                    assert cols == list(range(s, s + n))
                    if not cols:
                        continue
                    g = [keep[r][i][cols] for r in range(K)]
                    res = [np.ascontiguousarray(sub_res[r][i][cols]) for r in range(K)]
                    sres = np.ascontiguousarray(sub_sres[i][cols])
                    out, pk = ox.aggregate_columns(oracle_port, owner, g, res, sres, bits, zero_thr, self_q)
                    for r in range(K):
                        sub_res[r][i][cols] = res[r]
                        np.testing.assert_array_equal(res[r].view(np.uint32), st.res[r][i][cols].view(np.uint32))
                        np.testing.assert_array_equal(out.view(np.uint32), grads[r][i][cols].view(np.uint32))
                    sub_sres[i][cols] = sres
                    if K > 1:
                        np.testing.assert_array_equal(sres.view(np.uint32), st.sres[owner][i].view(np.uint32))
                    np.testing.assert_array_equal(pk, packed[0][i][s * C:(s + n) * C])


# ---- ElemType = double --------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def oracle_port_f64():
    from oracle import backend
    backend.build()
    return backend.OracleBackendF64()


def test_double_port_reproduces_reference_unit_grid(oracle_port_f64):
    """The C port's double instantiation against digests made by the reference's own headers with ElemType = double
    (tests/golden/golden_digests_f64.json): ten shape/range cases x bits {1..64} x both 1-bit modes x 5 iterations."""
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_digests_f64.json")) as f:
        want = json.load(f)["unit"]
    got = mg.unit_digests_f64(oracle_port_f64)
    assert got.keys() == want.keys()
    for k in want:
        assert got[k] == want[k], k


def test_double_layout(oracle_port_f64):
    # QuantizedColumn<double>::QuantizedColumnSize: two doubles + 64-bit words (Source/Math/QuantizedMatrix.h:42-47)
    assert oracle_port_f64.packed_col_bytes(70, 1) == 16 + 8 * 2
    assert oracle_port_f64.packed_col_bytes(2048, 1) == 16 + 8 * 32
    assert oracle_port_f64.packed_col_bytes(64, 4) == 16 + 8 * 4
    assert oracle_port_f64.packed_col_bytes(10, 64) == 16 + 8 * 10
    # an all-zero column: range collapses, every real row's bit is 1, padding bits stay 0; word w holds rows w, w + Q, ...
    g = np.zeros((1, 70), np.float64)
    r = np.zeros((1, 70), np.float64)
    p = np.zeros(oracle_port_f64.packed_col_bytes(70, 1), np.uint8)
    oracle_port_f64.quantize(g, r, r, p, 1, True)
    lo, hi = struct.unpack("<dd", p[:16].tobytes())
    assert lo == 0.0 and hi == 0.0
    assert list(np.frombuffer(p[16:].tobytes(), dtype="<u8")) == [(1 << 35) - 1, (1 << 35) - 1]
    assert not r.any()


def test_double_port_equals_reference_build_directly(oracle_port_f64):
    from oracle import backend
    if not backend.have_ref():
        pytest.skip("oracle/_ref/libqagg_ref.so not present")
    ref = backend.RefBackendF64()
    rng = np.random.default_rng(9)
    for trial in range(30):
        M = int(rng.integers(1, 300))
        N = int(rng.integers(1, 12))
        bits = int(rng.choice([1, 2, 4, 8, 16, 32, 64]))
        zero_thr = bool(rng.integers(0, 2))
        scale = float(10.0 ** rng.integers(-6, 2))
        ra = np.zeros((N, M), np.float64)
        rb = np.zeros((N, M), np.float64)
        for it in range(3):
            g = rng.standard_normal((N, M)) * scale
            pa = np.zeros(N * oracle_port_f64.packed_col_bytes(M, bits), np.uint8)
            pb = np.zeros_like(pa)
            oracle_port_f64.quantize(g, ra, ra, pa, bits, zero_thr)
            ref.quantize(g, rb, rb, pb, bits, zero_thr)
            np.testing.assert_array_equal(pa, pb)
            np.testing.assert_array_equal(ra.view(np.uint64), rb.view(np.uint64))
            oa = np.full((N, M), 0.25)
            ob_ = np.full((N, M), 0.25)
            oracle_port_f64.unquantize(pa, oa, bits, add=bool(it % 2))
            ref.unquantize(pb, ob_, bits, add=bool(it % 2))
            np.testing.assert_array_equal(oa.view(np.uint64), ob_.view(np.uint64))


def test_learner_update_restatement_known_answers(oracle_port):
    """oracle_sgd_update (Matrix::MomentumSGDUpdate, Source/Math/Matrix.cpp:1681-1698 over ScaleAndAdd :5415-5429), on numbers
    whose results can be written down: the three forms of the smoothed-gradient update, the fused multiply-add (one
    rounding: 1 + 2^-24 * 2^-1 cannot come out of a separate multiply and add), and the parameter step."""
    f = np.float32
    # momentum == 1: smoothed += alpha * g;  alpha = unitGain * lr = 0.5 * 0.5
    w, g, s = np.array([10.0], f), np.array([8.0], f), np.array([1.0], f)
    oracle_port.sgd_update(w, g, s, 0.5, 1.0, 0.5)
    assert s[0] == 3.0 and w[0] == 7.0
    # momentum == 0: smoothed = alpha * g (the old value is not read: NaN does not spread)
    w, g, s = np.array([10.0], f), np.array([8.0], f), np.array([np.nan], f)
    oracle_port.sgd_update(w, g, s, 0.25, 0.0, 1.0)
    assert s[0] == 2.0 and w[0] == 8.0
    # otherwise: smoothed = (smoothed + (alpha / momentum) * g) * momentum
    w, g, s = np.array([10.0], f), np.array([4.0], f), np.array([2.0], f)
    oracle_port.sgd_update(w, g, s, 0.5, 0.5, 1.0)   # alpha / momentum = 1 -> (2 + 4) * 0.5 = 3
    assert s[0] == 3.0 and w[0] == 7.0
    # one rounding for alpha * g + smoothed: alpha = 1 + 2^-12, g = 1 + 2^-12 -> product 1 + 2^-11 + 2^-24 exactly; plus
    # smoothed = -1 the exact sum 2^-11 + 2^-24 is representable, a rounded product (1 + 2^-11) would lose the 2^-24
    a = f(1.0) + f(2.0 ** -12)
    w, g, s = np.array([0.0], f), np.array([a], f), np.array([-1.0], f)
    oracle_port.sgd_update(w, g, s, float(a), 1.0, 1.0)
    assert s[0] == f(2.0 ** -11 + 2.0 ** -24), s[0]
    # a vector: every element independently
    w = np.arange(8, dtype=f)
    g = np.ones(8, f)
    s = np.zeros(8, f)
    oracle_port.sgd_update(w, g, s, 0.5, 1.0, 1.0)
    assert np.array_equal(s, np.full(8, 0.5, f)) and np.array_equal(w, np.arange(8, dtype=f) - f(0.5))


def test_half_precision_sum_restatement_known_answers():
    """oracle.exchange.dense_sum_fp16: cast to half, add in rank order with a rounding to half after every addition, cast
    back.  2048 + 1 is a tie in half precision (spacing 2 above 2048) and goes to the even neighbour; the order of the
    additions shows; values beyond the half range become infinities."""
    from oracle import exchange as ox
    one = lambda v: [np.array([[v]], np.float32)]
    assert ox.dense_sum_fp16([one(2048.0), one(1.0)])[0][0, 0] == 2048.0
    assert ox.dense_sum_fp16([one(2048.0), one(1.0), one(1.0)])[0][0, 0] == 2048.0      # (2048 + 1) + 1: both ties go down
    assert ox.dense_sum_fp16([one(1.0), one(1.0), one(2048.0)])[0][0, 0] == 2050.0      # (1 + 1) + 2048 is exact
    assert ox.dense_sum_fp16([one(0.1), one(0.2)])[0][0, 0] == np.float32(np.float16(np.float32(np.float16(0.1)) + np.float32(np.float16(0.2))))
    with np.errstate(over="ignore"):
        assert np.isinf(ox.dense_sum_fp16([one(70000.0), one(0.0)])[0][0, 0])
    # and the fp32 sum next to it: rank order, one rounding per addition
    big = [np.array([[1e8]], np.float32)], [np.array([[1.0]], np.float32)], [np.array([[-1e8]], np.float32)]
    assert ox.dense_sum(list(big))[0][0, 0] == 0.0      # (1e8 + 1) rounds to 1e8, then - 1e8
