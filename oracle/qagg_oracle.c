/*
 * qagg_oracle.c -- CPU restatement of CNTK's 1-bit-SGD column quantizer.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against; nothing in the shipped library calls it.  Only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark may load it.
 *
 * Parity status: PINNED.  The build recipe next to this file also compiles the
 * reference's own headers (Source/Math/ColumnQuantizer.h, ValueQuantizer.h,
 * QuantizedMatrix.h) in place into oracle/_ref/libqagg_ref.so; the committed
 * fixtures under tests/golden/ were produced by that library and this file must
 * reproduce them byte for byte (tests/test_oracle.py).
 *
 * Every function cites the reference lines it restates (paths relative to the
 * reference project root).  Arithmetic is fp32 with no FMA contraction, the
 * same as the reference CPU build (-msse4.1, Makefile:87): compile with
 * -ffp-contract=off.
 *
 * Layout (Source/Math/QuantizedMatrix.h:27-48): a packed column is
 *   float lower; float upper; uint32 bits[Q];   Q = ceil(M * nbits / 32)
 * and a packed matrix is N such columns back to back (column size 8 + 4Q bytes); for double,
 *   double lower; double upper; uint64 bits[Q]; Q = ceil(M * nbits / 64)   (column size 16 + 8Q bytes).
 * Word w of a column holds rows w, w+Q, w+2Q, ... ; the k-th of them at bit
 * k*nbits (Source/Math/ColumnQuantizer.h:50-65, 90-147).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* float: the symbols oracle_quantize, oracle_unquantize, oracle_packed_col_bytes */
#define REAL float
#define QWORD uint32_t
#define QSIGNED int32_t
#define QBITS 32
#define SQRT sqrtf
#define NAME(x) x
#include "qagg_oracle_impl.h"
#undef REAL
#undef QWORD
#undef QSIGNED
#undef QBITS
#undef SQRT
#undef NAME

/* double (QWord = uint64, 64 one-bit values per word): oracle_quantize_f64, oracle_unquantize_f64, oracle_packed_col_bytes_f64 */
#define REAL double
#define QWORD uint64_t
#define QSIGNED int64_t
#define QBITS 64
#define SQRT sqrt
#define NAME(x) x##_f64
#include "qagg_oracle_impl.h"
#undef REAL
#undef QWORD
#undef QSIGNED
#undef QBITS
#undef SQRT
#undef NAME

/* GetStripeForNode (Source/1BitSGD/AllReduceDistGradAggregator.h:56-65,
 * Source/1BitSGD/QuantizedDistributedCommunicator.h:158-165). */
ORACLE_API void oracle_stripe(int64_t numCols, int64_t nodeRank, int64_t numNodes, int64_t* start, int64_t* n)
{
    int64_t per = numCols / numNodes;
    int64_t residue = numCols % numNodes;
    *start = per * nodeRank + (residue < nodeRank ? residue : nodeRank);
    *n = per + ((nodeRank < residue) ? 1 : 0);
}

/* The learner step that consumes the aggregate: Matrix<ElemType>::MomentumSGDUpdate (Source/Math/Matrix.cpp:1681-1698) =
 *   ScaleAndAdd(unitGainFactor * learnRatePerSample, gradients, momentum, smoothedGradients);  *this -= smoothedGradients;
 * with ScaleAndAdd(alpha, a, beta, c) of Matrix.cpp:5415-5429:
 *   beta == 1: c += alpha * a;   beta == 0: c = alpha * a;   else: c += (alpha / beta) * a, then c *= beta.
 * PARITY UNPINNED for this function: the reference delegates `c += alpha * a` to a BLAS axpy (cblas_saxpy,
 * Source/Math/CPUMatrixImpl.h:5481-5507; cuBLAS on the GPU), a library that is not part of the reference checkout, and
 * whether that rounds once (fused multiply-add) or twice is the library's choice.  It is restated here as ONE fused
 * multiply-add (fmaf), which is what vectorised BLAS builds and cuBLAS do on current hardware; the scaling and the final
 * subtraction are single operations either way. */
ORACLE_API void oracle_sgd_update(float* param, const float* grad, float* smoothed, int64_t n, float learnRatePerSample, float momentum,
                                  float unitGainFactor)
{
    const float alpha = unitGainFactor * learnRatePerSample;
    for (int64_t i = 0; i < n; ++i)
    {
        float s;
        if (momentum == 1.0f)
            s = fmaf(alpha, grad[i], smoothed[i]);
        else if (momentum == 0.0f)
            s = alpha * grad[i];
        else
            s = momentum * fmaf(alpha / momentum, grad[i], smoothed[i]);
        smoothed[i] = s;
        param[i] = param[i] - s;
    }
}
