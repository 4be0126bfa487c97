// ref_driver.cpp -- thin C entry points around the REFERENCE's own quantizer headers.
//
// TEST INFRASTRUCTURE ONLY (checker / CPU baseline); never linked into the product.
//
// This file contains no quantizer arithmetic of its own: it includes the reference's
// Source/Math/ColumnQuantizer.h, ValueQuantizer.h and QuantizedMatrix.h where they lie
// (the include path is given on the compiler command line by oracle/Makefile) and calls
// ColumnQuantizer<ElemType>::ComputeRangeStatColj / Quantize / Unquantize per column (float and double), in
// the order MatrixQuantizerCPU does (Source/Math/MatrixQuantizerCPU.cpp:33-59, 90-96).
// MatrixQuantizerCPU.cpp itself cannot be linked here: it needs Matrix<T> from the
// reference's math library, which depends on Boost and a BLAS that are not installed.
// The resulting library, oracle/_ref/libqagg_ref.so, is used to generate the golden
// fixtures, to validate the plain-C restatement, and as the "reference" CPU baseline.
#include "ColumnQuantizer.h"
#include "QuantizedMatrix.h"

#include <cstddef>
#include <cstdint>

// The reference's error helpers (Common/Include/Basics.h:60) want a call-stack printer that lives in its
// Common library, which is not built here; an empty one satisfies the linker and is never reached.
namespace Microsoft { namespace MSR { namespace CNTK { namespace DebugUtil {
std::string GetCallStack(size_t, bool) { return std::string(); }
}}}}

using Microsoft::MSR::CNTK::ColumnQuantizer;
using Microsoft::MSR::CNTK::QuantizedColumn;
using Microsoft::MSR::CNTK::ValueQuantizer;

namespace {

template <class ElemType>
int quantize(const ElemType* grad, const ElemType* resIn, ElemType* resOut, void* packed, int64_t M, int64_t N, int nbits, int zeroThr)
{
    const size_t ldNbits = ValueQuantizer<ElemType>::ld((size_t) nbits);
    const size_t colBytes = QuantizedColumn<ElemType>::QuantizedColumnSize((size_t) nbits, (size_t) M);
    for (size_t j = 0; j < (size_t) N; j++)
    {
        auto& qcol = *(QuantizedColumn<ElemType>*) ((char*) packed + j * colBytes);
        if (zeroThr)
            ColumnQuantizer<ElemType>::template ComputeRangeStatColj<true>(grad, resIn, (long) M, j, (size_t) nbits, qcol.lower, qcol.upper);
        else
            ColumnQuantizer<ElemType>::template ComputeRangeStatColj<false>(grad, resIn, (long) M, j, (size_t) nbits, qcol.lower, qcol.upper);
        ColumnQuantizer<ElemType> q(ldNbits, qcol.lower, qcol.upper);
        if (zeroThr)
            q.template Quantize<true>(grad, resIn, (long) M, j, qcol.bits, resOut);
        else
            q.template Quantize<false>(grad, resIn, (long) M, j, qcol.bits, resOut);
    }
    return 0;
}

template <class ElemType>
int unquantize(const void* packed, ElemType* out, int64_t M, int64_t N, int nbits, int add)
{
    const size_t ldNbits = ValueQuantizer<ElemType>::ld((size_t) nbits);
    const size_t colBytes = QuantizedColumn<ElemType>::QuantizedColumnSize((size_t) nbits, (size_t) M);
    for (size_t j = 0; j < (size_t) N; j++)
    {
        const auto& qcol = *(const QuantizedColumn<ElemType>*) ((const char*) packed + j * colBytes);
        ColumnQuantizer<ElemType> q(ldNbits, qcol.lower, qcol.upper);
        q.Unquantize(out, (long) M, j, qcol.bits, add != 0);
    }
    return 0;
}

} // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API int64_t ref_packed_col_bytes(int64_t rows, int nbits)
{
    return (int64_t) QuantizedColumn<float>::QuantizedColumnSize((size_t) nbits, (size_t) rows);
}
REF_API int ref_quantize(const float* grad, const float* resIn, float* resOut, void* packed, int64_t M, int64_t N, int nbits, int zeroThr)
{
    return quantize<float>(grad, resIn, resOut, packed, M, N, nbits, zeroThr);
}
REF_API int ref_unquantize(const void* packed, float* out, int64_t M, int64_t N, int nbits, int add)
{
    return unquantize<float>(packed, out, M, N, nbits, add);
}
// ElemType = double: QWord = unsigned long long (Source/Math/ValueQuantizer.h:48-55), what the reference's own 1-bit end-to-end
// tests run (precision=double)
REF_API int64_t ref_packed_col_bytes_f64(int64_t rows, int nbits)
{
    return (int64_t) QuantizedColumn<double>::QuantizedColumnSize((size_t) nbits, (size_t) rows);
}
REF_API int ref_quantize_f64(const double* grad, const double* resIn, double* resOut, void* packed, int64_t M, int64_t N, int nbits, int zeroThr)
{
    return quantize<double>(grad, resIn, resOut, packed, M, N, nbits, zeroThr);
}
REF_API int ref_unquantize_f64(const void* packed, double* out, int64_t M, int64_t N, int nbits, int add)
{
    return unquantize<double>(packed, out, M, N, nbits, add);
}
