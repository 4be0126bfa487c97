"""cntk_b200 -- B200 (sm_100a) quantized gradient aggregation, the 1-bit-SGD hot path of CNTK.

The product is ``libqagg.so`` (CUDA + NCCL behind the C ABI in ``include/qagg.h``) and the C++ headers in
``cntk_b200/csrc/cntk_compat`` that mirror the reference's MatrixQuantizerImpl / IDistGradAggregator /
QuantizedDistributedCommunicator interfaces on top of it.  This Python package is the thin ctypes driver the
tests and the benchmark use; it has no compute of its own and no CPU fallback: importing ``cntk_b200.lib``
fails if the shared library has not been built (``python -m cntk_b200.build``).
"""
__all__ = ["build", "lib"]
