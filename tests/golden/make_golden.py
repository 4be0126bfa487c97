"""Generates the golden fixtures in this directory from the REFERENCE's own quantizer code.

Run where the reference checkout exists:   python tests/golden/make_golden.py
It loads oracle/_ref/libqagg_ref.so (reference headers compiled in place, see oracle/Makefile)
and writes
  golden_digests.json   sha256 digests of (packed, residual, output) after every error-feedback
                        iteration, for the reference unit-test grid
                        (Tests/UnitTests/MathTests/MatrixQuantizerTests.cpp:404-419: ten shape/range
                        cases x bits {1,2,4,8,16,32} x both 1-bit threshold modes x 5 iterations),
                        for the 2048x2048 ten-step round trip, and for small striped exchanges.
  golden_small.npz      full arrays (inputs and outputs) of the smallest cases, so a mismatch can
                        be localised without the reference.
  golden_digests_f64.json  the unit-test grid in double precision (ElemType = double, 64-bit packed words, bits up to
                        64): `python tests/golden/make_golden.py f64` writes this file alone.
Inputs come from numpy's PCG64 streams keyed by the seeds below; their digests are recorded too,
so a drift in the generator is reported as such and not as a parity failure.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import backend as ob  # noqa: E402
from oracle import exchange as ox  # noqa: E402

# (rows, cols, low, high, seed) -- the reference's own grid (MatrixQuantizerTests.cpp:410-419).
UNIT_CASES = [
    (25, 13, -1.0, 1.0, 2015),
    (25, 13, -0.005, 0.005, 2115),
    (13, 25, -0.00001, 0.00001, 2215),
    (13, 25, -10.0, 10.0, 2315),
    (25, 13, -1.0, 2.05, 2415),
    (489, 1, -0.5, 0.5, 2515),
    (1, 135, -0.5, 0.5, 2615),
    (89, 23, -0.5, 0.5, 2715),
    (15, 35, -0.5, 0.5, 2815),
    (100, 50, -0.5, 0.5, 2915),
]
BITS = [1, 2, 4, 8, 16, 32]
ITERS = 5
SMALL_FULL = {(25, 13, 2015), (489, 1, 2515), (1, 135, 2615)}

# small gradient sets for the exchange: (M, N) per tensor; includes N < K and single-column tensors.
EXCHANGE_SHAPES = [(64, 10), (33, 7), (70, 1), (128, 3), (5, 16)]
EXCHANGE_STEPS = 3


def uniform_input(rows, cols, low, high, seed):
    rng = np.random.default_rng(seed)
    return rng.uniform(low, high, size=(cols, rows)).astype(np.float32)


def normal_input(rows, cols, sigma, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(size=(cols, rows)) * sigma).astype(np.float32)


def sha(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def run_unit_case(be, rows, cols, low, high, seed, bits, zero_thr, keep=None):
    """The loop of TestRunQuantization (MatrixQuantizerTests.cpp:268-316): in-place residual, add = iter>0."""
    res = np.zeros((cols, rows), np.float32)
    out = np.zeros((cols, rows), np.float32)
    packed = np.zeros(cols * be.packed_col_bytes(rows, bits), np.uint8)
    digests, in_digests = [], []
    for it in range(ITERS):
        g = uniform_input(rows, cols, low, high, seed + it)
        in_digests.append(sha(g))
        be.quantize(g, res, res, packed, bits, zero_thr)
        be.unquantize(packed, out, bits, add=(it > 0))
        digests.append(sha(packed, res, out))
        if keep is not None:
            keep.append((g.copy(), packed.copy(), res.copy(), out.copy()))
    return digests, in_digests


def exchange_inputs(K, step):
    return [[normal_input(M, N, 1e-3, 100000 + 1000 * r + 17 * i + step) for i, (M, N) in enumerate(EXCHANGE_SHAPES)]
            for r in range(K)]


def run_exchange(be, K, bits, zero_thr, self_quant, keep=None):
    st = ox.ExchangeState(EXCHANGE_SHAPES, K)
    digests = []
    for step in range(EXCHANGE_STEPS):
        grads = exchange_inputs(K, step)
        packed = ox.aggregate_step(be, st, grads, bits, zero_thr, self_quant)
        flat = [a for r in range(K) for a in grads[r]] + [a for r in range(K) for a in st.res[r]] + \
               [a for r in range(K) for a in st.sres[r]] + list(packed[0])
        digests.append(sha(*flat))
        if keep is not None:
            keep.append((grads, packed[0]))
    return digests


# ---- ElemType = double (the reference's CPUMatrix1BitQuantizeDouble / GPUMatrix1BitQuantizeDouble grid,
# MatrixQuantizerTests.cpp:404-472: the same ten cases, bits up to 64) --------------------------------------
BITS_F64 = [1, 2, 4, 8, 16, 32, 64]


def uniform_input_f64(rows, cols, low, high, seed):
    rng = np.random.default_rng(seed)
    return rng.uniform(low, high, size=(cols, rows))


def run_unit_case_f64(be, rows, cols, low, high, seed, bits, zero_thr):
    res = np.zeros((cols, rows), np.float64)
    out = np.zeros((cols, rows), np.float64)
    packed = np.zeros(cols * be.packed_col_bytes(rows, bits), np.uint8)
    digests = []
    for it in range(ITERS):
        g = uniform_input_f64(rows, cols, low, high, seed + it)
        be.quantize(g, res, res, packed, bits, zero_thr)
        be.unquantize(packed, out, bits, add=(it > 0))
        digests.append(sha(packed, res, out))
    return digests


def unit_digests_f64(be):
    dig = {}
    for (rows, cols, low, high, seed) in UNIT_CASES:
        for bits in BITS_F64:
            for zero_thr in ((False, True) if bits == 1 else (False,)):
                dig[f"{rows}x{cols}_seed{seed}_b{bits}_z{int(zero_thr)}"] = run_unit_case_f64(be, rows, cols, low, high, seed, bits, zero_thr)
    return dig


def main_f64():
    """golden_digests_f64.json: the unit grid in double precision, from the reference's headers."""
    dig = unit_digests_f64(ob.RefBackendF64())
    with open(os.path.join(HERE, "golden_digests_f64.json"), "w") as f:
        json.dump({"unit": dig}, f, indent=1, sort_keys=True)
    print("wrote", len(dig), "double-precision unit digests")


def main():
    be = ob.RefBackend()
    dig = {"unit": {}, "config1": {}, "exchange": {}, "inputs": {}}
    small = {}
    for (rows, cols, low, high, seed) in UNIT_CASES:
        for bits in BITS:
            for zero_thr in ((False, True) if bits == 1 else (False,)):
                key = f"{rows}x{cols}_seed{seed}_b{bits}_z{int(zero_thr)}"
                keep = [] if (rows, cols, seed) in SMALL_FULL and bits in (1, 2, 4) else None
                d, ind = run_unit_case(be, rows, cols, low, high, seed, bits, zero_thr, keep)
                dig["unit"][key] = d
                dig["inputs"][f"{rows}x{cols}_seed{seed}"] = ind
                if keep is not None:
                    for it, (g, p, r, o) in enumerate(keep):
                        small[f"{key}_it{it}_in"] = g
                        small[f"{key}_it{it}_packed"] = p
                        small[f"{key}_it{it}_res"] = r
                        small[f"{key}_it{it}_out"] = o

    # 2048 x 2048, N(0, 0.01^2), seed 0 + step, 10 quantize -> unquantize steps with error feedback, 1 bit.
    for zero_thr in (True, False):
        res = np.zeros((2048, 2048), np.float32)
        out = np.zeros((2048, 2048), np.float32)
        packed = np.zeros(2048 * be.packed_col_bytes(2048, 1), np.uint8)
        steps = []
        for step in range(10):
            g = normal_input(2048, 2048, 0.01, 0 + step)
            be.quantize(g, res, res, packed, 1, zero_thr)
            be.unquantize(packed, out, 1, add=False)
            hdr = packed.reshape(2048, -1)[:, :8].copy()
            steps.append({"in": sha(g), "packed": sha(packed), "recon": sha(hdr), "residual": sha(res), "out": sha(out)})
        dig["config1"][f"z{int(zero_thr)}"] = steps

    for K in (1, 2, 3, 4, 8):
        for bits in (1, 2, 4):
            for zero_thr in ((True, False) if bits == 1 else (True,)):
                for self_quant in (True, False):
                    key = f"K{K}_b{bits}_z{int(zero_thr)}_s{int(self_quant)}"
                    keep = [] if (K in (2, 3) and bits == 1 and zero_thr and self_quant) else None
                    dig["exchange"][key] = run_exchange(be, K, bits, zero_thr, self_quant, keep)
                    if keep is not None:
                        grads, packed = keep[-1]
                        for i in range(len(EXCHANGE_SHAPES)):
                            small[f"exchange_{key}_final_agg_t{i}"] = grads[0][i]
                            small[f"exchange_{key}_final_packed_t{i}"] = packed[i]

    with open(os.path.join(HERE, "golden_digests.json"), "w") as f:
        json.dump(dig, f, indent=1, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, "golden_small.npz"), **small)
    print("wrote", len(dig["unit"]), "unit digests,", len(dig["exchange"]), "exchange digests,", len(small), "arrays")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "f64":
        main_f64()  # the float fixtures are left as they are
    else:
        main()
        main_f64()
