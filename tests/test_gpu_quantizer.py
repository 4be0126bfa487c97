"""GPU parity of the single-matrix quantizer entry points (through the C ABI) against the CPU oracle.

The bar is bit-exactness: packed words, reconstruction values, residuals and unquantized outputs must be
byte-identical to MatrixQuantizerCPU's on the same inputs, step after step with error feedback."""
import json
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def G():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    return gpu_util


@pytest.fixture(scope="module")
def digests():
    with open(os.path.join(os.path.dirname(__file__), "golden", "golden_digests.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("case", mg.UNIT_CASES, ids=lambda c: f"{c[0]}x{c[1]}")
def test_reference_unit_grid_bit_exact(G, oracle_port, digests, case):
    """Tests/UnitTests/MathTests/MatrixQuantizerTests.cpp:404-419 grid: all bit widths, both 1-bit thresholds,
    5 iterations with in-place residual and add = (iter > 0).  Checked against the oracle AND the committed digests."""
    rows, cols, low, high, seed = case
    for bits in mg.BITS:
        for zero_thr in ((False, True) if bits == 1 else (False,)):
            key = f"{rows}x{cols}_seed{seed}_b{bits}_z{int(zero_thr)}"
            res_o = np.zeros((cols, rows), np.float32)
            out_o = np.zeros((cols, rows), np.float32)
            packed_o = np.zeros(cols * oracle_port.packed_col_bytes(rows, bits), np.uint8)
            res_g = G.dev(res_o)
            out_g = G.dev(out_o)
            for it in range(mg.ITERS):
                g = mg.uniform_input(rows, cols, low, high, seed + it)
                oracle_port.quantize(g, res_o, res_o, packed_o, bits, zero_thr)
                oracle_port.unquantize(packed_o, out_o, bits, add=(it > 0))
                packed_g = G.gpu_quantize(G.dev(g), res_g, bits, zero_thr)
                G.gpu_unquantize(packed_g, out_g, bits, add=(it > 0))
                ph, rh, oh = G.host(packed_g), G.host(res_g), G.host(out_g)
                G.assert_same_bits(ph, packed_o, f"{key} it{it} packed")
                G.assert_same_bits(rh, res_o, f"{key} it{it} residual")
                G.assert_same_bits(oh, out_o, f"{key} it{it} output")
                assert mg.sha(ph, rh, oh) == digests["unit"][key][it], f"{key} it{it} digest"
                # conservation invariant of the reference test (:327-338) holds trivially when bit-exact; check anyway
            assert np.isfinite(G.host(res_g)).all()


@pytest.mark.parametrize("zero_thr", [True, False])
def test_config1_round_trip_matches_committed_digests(G, digests, zero_thr):
    """2048 x 2048, N(0, 0.01^2), seed 0 + step, 1 bit, ten quantize -> unquantize steps with error feedback."""
    res = torch.zeros((2048, 2048), dtype=torch.float32, device=G.DEV)
    out = torch.zeros((2048, 2048), dtype=torch.float32, device=G.DEV)
    for step in range(10):
        g = mg.normal_input(2048, 2048, 0.01, step)
        exp = digests["config1"][f"z{int(zero_thr)}"][step]
        assert mg.sha(g) == exp["in"]
        packed = G.gpu_quantize(G.dev(g), res, 1, zero_thr)
        G.gpu_unquantize(packed, out, 1, add=False)
        ph = G.host(packed)
        assert mg.sha(ph) == exp["packed"], f"step {step} packed words"
        assert mg.sha(ph.reshape(2048, -1)[:, :8].copy()) == exp["recon"], f"step {step} reconstruction values"
        assert mg.sha(G.host(res)) == exp["residual"], f"step {step} residual"
        assert mg.sha(G.host(out)) == exp["out"], f"step {step} output"


SHAPES_EDGE = [
    (9304, 5), (9304, 1), (2048, 33), (1000, 40), (64, 147), (512, 300), (7, 1000), (1, 1), (3, 2), (31, 31), (33, 33),
    (4097, 3), (50000, 3), (60001, 2), (130000, 1),
]


@pytest.mark.parametrize("shape", SHAPES_EDGE, ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("bits,zero_thr", [(1, True), (1, False), (2, True), (4, True), (8, True), (32, True)])
def test_edge_shapes_bit_exact(G, oracle_port, shape, bits, zero_thr):
    """Tall columns (resident and streamed), odd row counts, single rows/columns; three error-feedback steps with
    one all-zero column and one all-negative column."""
    M, N = shape
    rng = np.random.default_rng(M * 131 + N * 7 + bits)
    res_o = np.zeros((N, M), np.float32)
    res_g = G.dev(res_o)
    packed_o = np.zeros(N * oracle_port.packed_col_bytes(M, bits), np.uint8)
    out_o = np.zeros((N, M), np.float32)
    out_g = G.dev(out_o)
    for it in range(3):
        g = (rng.standard_normal((N, M)) * 1e-3).astype(np.float32)
        g[0] = 0.0
        if N > 1:
            g[-1] = -np.abs(g[-1]) - np.float32(1e-6)
        oracle_port.quantize(g, res_o, res_o, packed_o, bits, zero_thr)
        oracle_port.unquantize(packed_o, out_o, bits, add=bool(it))
        packed_g = G.gpu_quantize(G.dev(g), res_g, bits, zero_thr)
        G.gpu_unquantize(packed_g, out_g, bits, add=bool(it))
        G.assert_same_bits(G.host(packed_g), packed_o, f"{shape} b{bits} it{it} packed")
        G.assert_same_bits(G.host(res_g), res_o, f"{shape} b{bits} it{it} residual")
        G.assert_same_bits(G.host(out_g), out_o, f"{shape} b{bits} it{it} output")


def test_separate_residual_buffers_and_unaligned_base(G, oracle_port):
    """inResidual != outResidual (the V2 communicator's use, QuantizedDistributedCommunicator.h:365) and a gradient
    that starts 4 bytes off a 16-byte boundary (scalar load path)."""
    M, N, bits = 256, 9, 1
    rng = np.random.default_rng(5)
    g = (rng.standard_normal((N, M)) * 1e-2).astype(np.float32)
    r_in = (rng.standard_normal((N, M)) * 1e-3).astype(np.float32)
    r_out_o = np.zeros((N, M), np.float32)
    packed_o = np.zeros(N * oracle_port.packed_col_bytes(M, bits), np.uint8)
    oracle_port.quantize(g, r_in, r_out_o, packed_o, bits, True)
    flat = torch.zeros(N * M + 1, dtype=torch.float32, device=G.DEV)
    flat[1:] = G.dev(g).reshape(-1)
    gd = flat[1:]
    rin_d = G.dev(r_in)
    rout_d = torch.zeros((N, M), dtype=torch.float32, device=G.DEV)
    packed_d = torch.zeros(packed_o.size, dtype=torch.uint8, device=G.DEV)
    from cntk_b200 import lib
    lib.quantize(gd.data_ptr(), rin_d.data_ptr(), rout_d.data_ptr(), packed_d.data_ptr(), M, N, bits, True)
    G.assert_same_bits(G.host(packed_d), packed_o, "packed")
    G.assert_same_bits(G.host(rout_d), r_out_o, "residual out")
    G.assert_same_bits(G.host(rin_d), r_in, "residual in untouched")


def test_host_packed_entry_points(G, oracle_port):
    """qagg_quantize_to_host / qagg_unquantize_from_host: the packed matrix lives in (pinned) host memory, as the
    reference drives its GPU quantizer (MatrixQuantizerGPU.cu:243, 260-268, 300-325)."""
    from cntk_b200 import lib
    M, N, bits = 500, 20, 2
    rng = np.random.default_rng(11)
    g = (rng.standard_normal((N, M)) * 1e-2).astype(np.float32)
    res_o = np.zeros((N, M), np.float32)
    packed_o = np.zeros(N * oracle_port.packed_col_bytes(M, bits), np.uint8)
    oracle_port.quantize(g, res_o, res_o, packed_o, bits, True)
    out_o = np.zeros((N, M), np.float32)
    oracle_port.unquantize(packed_o, out_o, bits, False)
    gd, rd = G.dev(g), G.dev(np.zeros((N, M), np.float32))
    scratch = torch.zeros(packed_o.size, dtype=torch.uint8, device=G.DEV)
    hp = torch.zeros(packed_o.size, dtype=torch.uint8).pin_memory()
    lib.quantize_to_host(gd.data_ptr(), rd.data_ptr(), rd.data_ptr(), scratch.data_ptr(), hp.data_ptr(), M, N, bits, True)
    G.assert_same_bits(hp.numpy(), packed_o, "host packed")
    od = torch.zeros((N, M), dtype=torch.float32, device=G.DEV)
    lib.unquantize_from_host(hp.data_ptr(), scratch.data_ptr(), od.data_ptr(), M, N, bits, False)
    G.assert_same_bits(G.host(od), out_o, "output")


def test_argument_errors_are_reported_not_raised_in_c(G):
    from cntk_b200 import lib
    with pytest.raises(lib.QaggError):
        lib.quantize(1 << 8, 1 << 8, 1 << 8, 1 << 8, 16, 16, 3, True)  # 3 bits: not a power of two
    with pytest.raises(lib.QaggError):
        lib.unquantize(0, 0, 16, 16, 1)
    lib.quantize(0, 0, 0, 0, 0, 0, 1, True)  # empty matrix: no-op, as the reference's loops


@pytest.mark.parametrize("K", [2, 3, 4, 8])
@pytest.mark.parametrize("bits,zero_thr", [(1, True), (1, False), (2, True), (4, True)])
@pytest.mark.parametrize("self_raw", [False, True])
def test_reduce_requantize_bit_exact(G, oracle_port, K, bits, zero_thr, self_raw):
    """The owner's fused unpack + sum + requantize against the oracle's unquantize(add) chain followed by quantize
    (AllReduceDistGradAggregator.h:366-375, 405-435), two steps so the stripe residual is exercised."""
    from cntk_b200 import lib
    M, n = 777, 11
    rng = np.random.default_rng(K * 100 + bits * 10 + int(zero_thr) + 2 * int(self_raw))
    C = oracle_port.packed_col_bytes(M, bits)
    sres_o = np.zeros((n, M), np.float32)
    sres_g = G.dev(sres_o)
    for it in range(2):
        grads = [(rng.standard_normal((n, M)) * 1e-3).astype(np.float32) for _ in range(K)]
        packs = []
        for g in grads:
            p = np.zeros(n * C, np.uint8)
            r = (rng.standard_normal((n, M)) * 1e-4).astype(np.float32)
            oracle_port.quantize(g, r, r, p, bits, zero_thr)
            packs.append(p)
        agg = grads[0].copy()
        if not self_raw:
            oracle_port.unquantize(packs[0], agg, bits, add=False)
        for s in range(1, K):
            oracle_port.unquantize(packs[s], agg, bits, add=True)
        out_o = np.zeros(n * C, np.uint8)
        oracle_port.quantize(agg, sres_o, sres_o, out_o, bits, zero_thr)
        dpacks = [G.dev(p) for p in packs]
        raw = G.dev(grads[0]) if self_raw else None
        out_g = torch.zeros(n * C, dtype=torch.uint8, device=G.DEV)
        ptrs = [dp.data_ptr() for dp in dpacks]
        if self_raw:
            ptrs[0] = 0
        lib.reduce_requantize(ptrs, raw.data_ptr() if self_raw else 0, sres_g.data_ptr(), sres_g.data_ptr(), out_g.data_ptr(),
                              M, n, bits, zero_thr)
        G.assert_same_bits(G.host(out_g), out_o, f"K{K} b{bits} it{it} packed aggregate")
        G.assert_same_bits(G.host(sres_g), sres_o, f"K{K} b{bits} it{it} stripe residual")
