"""ctypes front-ends of the two CPU checkers (TEST INFRASTRUCTURE ONLY).

``OracleBackend``  -> oracle/liboracle.so        (plain-C restatement, qagg_oracle.c)
``RefBackend``     -> oracle/_ref/libqagg_ref.so (the reference's own headers, ref_driver.cpp)

Both expose the same three calls over numpy arrays in the reference's layouts: fp32
matrices are column-major M x N (stored here as C-contiguous arrays of shape (N, M), one
row of the array per matrix column), packed matrices are uint8 arrays of N * (8 + 4Q)
bytes (Source/Math/QuantizedMatrix.h:27-48).

Nothing in the product imports this module; tests, the smoke check and the benchmark's
CPU-baseline leg do.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = ctypes.POINTER(ctypes.c_float)


def reference_root():
    """Root of the CNTK checkout the reference-header checker is built from: $QAGG_REFERENCE_ROOT, else a sibling
    `reference` directory of this repository's parent; None when neither holds the quantizer headers."""
    cands = [os.environ.get("QAGG_REFERENCE_ROOT"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "Source", "Math", "ColumnQuantizer.h")):
            return c
    return None


def build(quiet=True):
    """Run oracle/Makefile (gcc only; also builds _ref when the reference checkout exists)."""
    ref = reference_root()
    out = subprocess.run(["make", "-C", _HERE] + ([f"REF={ref}"] if ref else []), capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if not quiet:
        print(out.stdout)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _check(a, name, dtype):
    if a.dtype != dtype or not a.flags["C_CONTIGUOUS"]:
        raise ValueError(f"{name} must be C-contiguous {np.dtype(dtype).name}")


class _Backend:
    prefix = None
    path = None
    kind = None
    suffix = ""          # "_f64": the double instantiation (ElemType = double, QWord = uint64)
    dtype = np.float32

    def __init__(self):
        if not os.path.exists(self.path):
            build()
        if not os.path.exists(self.path):
            raise FileNotFoundError(self.path)
        self.lib = ctypes.CDLL(self.path)
        p = self.prefix
        self._q = getattr(self.lib, p + "quantize" + self.suffix)
        self._q.restype = ctypes.c_int
        self._q.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int]
        self._u = getattr(self.lib, p + "unquantize" + self.suffix)
        self._u.restype = ctypes.c_int
        self._u.argtypes = [ctypes.c_void_p] * 2 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int]
        self._c = getattr(self.lib, p + "packed_col_bytes" + self.suffix)
        self._c.restype = ctypes.c_int64
        self._c.argtypes = [ctypes.c_int64, ctypes.c_int]

    def packed_col_bytes(self, M, bits):
        return int(self._c(M, bits))

    def quantize(self, grad, res_in, res_out, packed, bits, zero_thr=True):
        """grad/res_in/res_out: (N, M) float32 (column-major M x N); packed: uint8[N*C]. In place allowed."""
        N, M = grad.shape
        for a, n in ((grad, "grad"), (res_in, "res_in"), (res_out, "res_out")):
            _check(a, n, self.dtype)
            assert a.shape == (N, M)
        assert packed.dtype == np.uint8 and packed.size == N * self.packed_col_bytes(M, bits)
        rc = self._q(_ptr(grad), _ptr(res_in), _ptr(res_out), _ptr(packed), M, N, bits, int(bool(zero_thr)))
        if rc != 0:
            raise RuntimeError(f"{self.prefix}quantize failed rc={rc}")

    def unquantize(self, packed, out, bits, add=False):
        N, M = out.shape
        _check(out, "out", self.dtype)
        assert packed.dtype == np.uint8 and packed.size == N * self.packed_col_bytes(M, bits)
        rc = self._u(_ptr(packed), _ptr(out), M, N, bits, int(bool(add)))
        if rc != 0:
            raise RuntimeError(f"{self.prefix}unquantize failed rc={rc}")


class OracleBackend(_Backend):
    prefix = "oracle_"
    path = os.path.join(_HERE, "liboracle.so")
    kind = "port"

    def stripe(self, num_cols, rank, K):
        s, n = ctypes.c_int64(), ctypes.c_int64()
        self.lib.oracle_stripe.argtypes = [ctypes.c_int64] * 3 + [ctypes.POINTER(ctypes.c_int64)] * 2
        self.lib.oracle_stripe.restype = None
        self.lib.oracle_stripe(num_cols, rank, K, ctypes.byref(s), ctypes.byref(n))
        return int(s.value), int(n.value)


    def sgd_update(self, param, grad, smoothed, learn_rate, momentum, unit_gain):
        """Momentum-SGD step in place on float32 arrays of one size (Matrix::MomentumSGDUpdate, Source/Math/Matrix.cpp:1681-1698)."""
        for a, n in ((param, "param"), (grad, "grad"), (smoothed, "smoothed")):
            _check(a, n, np.float32)
            assert a.size == param.size
        f = self.lib.oracle_sgd_update
        f.restype = None
        f.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] + [ctypes.c_float] * 3
        f(_ptr(param), _ptr(grad), _ptr(smoothed), param.size, learn_rate, momentum, unit_gain)


class RefBackend(_Backend):
    prefix = "ref_"
    path = os.path.join(_HERE, "_ref", "libqagg_ref.so")
    kind = "reference"


class OracleBackendF64(OracleBackend):
    suffix = "_f64"
    dtype = np.float64


class RefBackendF64(RefBackend):
    suffix = "_f64"
    dtype = np.float64


def have_ref():
    return os.path.exists(RefBackend.path)


def best_backend():
    """The reference-built checker when present (it is on any box this repo was built for), else the port."""
    return RefBackend() if have_ref() else OracleBackend()
