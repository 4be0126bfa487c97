// qagg_f64.cu -- the column quantizer for ElemType = double: 64-bit packed words (QuantizedWordHelper<double>::ValueType,
// Source/Math/ValueQuantizer.h:48-55), 64 one-bit values per word, bit widths 1 .. 64.  This is what the reference's own
// 1-bit end-to-end tests run (precision=double).  Single-matrix entry points only (MatrixQuantizerImpl<double>); the
// striped aggregator is built for float.
//
// Same arithmetic contract as the float kernels: every operation an explicit round-to-nearest double intrinsic, operand
// types as the reference's (size_t -> double before divides, unsigned x double, truncating double -> int64), the float
// literals 1e-36f / 0.5f / 2.0f / 4.0f promoted as the reference's template does, and every per-column sum accumulated in
// ROW ORDER.  Layout: one CTA per column at a time; the column's values v = gradient + residual pass through shared
// memory in chunks of 1024 rows, loaded by all threads; lane 0 of warp 0 walks the lower-level chain (or the single sum of
// the other modes) and lane 0 of warp 1 the upper-level chain, both carrying their accumulators from chunk to chunk;
// afterwards all threads quantize, one packed word each.  A plain kernel: the double path is a completeness row, not the
// benchmarked one.
#include "../../include/qagg.h"
#include "qagg_internal.h"

namespace qagg {

constexpr int DNT = 128;     // threads per CTA
constexpr int DCHUNK = 1024; // rows per staged chunk

struct ValQD
{
    double qmin, qmax, qmid, qfactor, ufactor;
    unsigned long long rangeend;
};

// ValueQuantizer<double> constructor (ValueQuantizer.h:68-97)
__device__ __forceinline__ ValQD make_valq_d(int bits, double lower, double upper)
{
    ValQD q;
    q.qmin = lower;
    q.qmax = upper;
    q.rangeend = (bits >= 64) ? 0ull : (1ull << bits);
    const double range = __dsub_rn(upper, lower);
    if ((range < (double) 1e-36f) || (q.rangeend == 0))
    {
        q.qfactor = q.ufactor = 0.0;
    }
    else
    {
        const double used = (double) (q.rangeend - (bits > 1 ? 1ull : 0ull)); // size_t -> double
        q.qfactor = __ddiv_rn(used, range);
        q.ufactor = __ddiv_rn(range, used);
    }
    q.qmid = __dmul_rn((double) 0.5f, __dadd_rn(upper, lower));
    return q;
}

// Quantize<ZeroThresholdFor1Bit> (ValueQuantizer.h:101-128, 144-156)
__device__ __forceinline__ unsigned long long quantize_d(const ValQD& q, int bits, bool zeroThr, double u)
{
    if (bits == 64)
        return (unsigned long long) __double_as_longlong(u);
    if (bits == 1)
        return (zeroThr ? (u >= 0.0) : (u >= q.qmid)) ? 1ull : 0ull;
    if (u <= q.qmin)
        return 0ull;
    if (u >= q.qmax)
        return q.rangeend - 1ull;
    return (unsigned long long) __double2ll_rz(__dmul_rn(__dsub_rn(u, q.qmin), q.qfactor));
}

// Unquantize (ValueQuantizer.h:131-141)
__device__ __forceinline__ double unquantize_d(const ValQD& q, int bits, unsigned long long u)
{
    if (bits == 64)
        return __longlong_as_double((long long) u);
    return __dadd_rn(__dmul_rn(__dadd_rn(__ull2double_rn(u), 0.5), q.ufactor), q.qmin);
}

// ComputeRangeStatColjSubset for one column (ColumnQuantizer.h:209-341) + Quantize (ColumnQuantizer.h:50-65, 90-147)
__global__ void __launch_bounds__(DNT) k_quantize_f64(const double* __restrict__ grad, const double* __restrict__ resIn, double* __restrict__ resOut,
                                                     unsigned char* __restrict__ packed, long long M, long long N, int bits, int zeroThr)
{
    __shared__ double sv[DCHUNK];
    __shared__ double sAcc[2];
    __shared__ unsigned sNum0;
    __shared__ double sRange[2];
    const int tid = threadIdx.x;
    const long long Q = (M * bits + 63) / 64;
    const long long colBytes = 16 + 8 * Q;
    const int vpw = 64 / bits;
    for (long long j = blockIdx.x; j < N; j += gridDim.x)
    {
        const double* __restrict__ g = grad + j * M;
        const double* __restrict__ r = resIn + j * M;
        const double rows = (double) (unsigned long long) M; // size_t -> double
        double mean = 0.0;
        // mean-threshold 1-bit mode: a first ordered pass for the column mean (:232-245)
        if (bits == 1 && !zeroThr)
        {
            double acc = 0.0;
            for (long long r0 = 0; r0 < M; r0 += DCHUNK)
            {
                const int nr = (int) min((long long) DCHUNK, M - r0);
                for (int i = tid; i < nr; i += DNT)
                    sv[i] = __dadd_rn(g[r0 + i], r[r0 + i]);
                __syncthreads();
                if (tid == 0)
                    for (int i = 0; i < nr; ++i)
                        acc = __dadd_rn(acc, sv[i]);
                __syncthreads();
            }
            if (tid == 0)
                sAcc[0] = __ddiv_rn(acc, rows);
            __syncthreads();
            mean = sAcc[0];
            __syncthreads();
        }
        // the ordered sums: two level sums and a count (1 bit), or the sum of squares (otherwise)
        double acc = 0.0;
        unsigned num0 = 0;
        for (long long r0 = 0; r0 < M; r0 += DCHUNK)
        {
            const int nr = (int) min((long long) DCHUNK, M - r0);
            for (int i = tid; i < nr; i += DNT)
                sv[i] = __dadd_rn(g[r0 + i], r[r0 + i]);
            __syncthreads();
            if (bits == 1)
            {
                if (tid == 0) // lower level: the rows with v < mean, counted; every other row adds +0 (the sum starts at +0 and stays exact)
                    for (int i = 0; i < nr; ++i)
                    {
                        const double v = sv[i];
                        const bool below = v < mean;
                        acc = __dadd_rn(acc, below ? v : 0.0);
                        num0 += below ? 1u : 0u;
                    }
                else if (tid == 32) // upper level: all other rows (a NaN lands here, as in the reference)
                    for (int i = 0; i < nr; ++i)
                    {
                        const double v = sv[i];
                        acc = __dadd_rn(acc, (v < mean) ? 0.0 : v);
                    }
            }
            else if (tid == 0)
            {
                for (int i = 0; i < nr; ++i)
                {
                    const double d = __dsub_rn(sv[i], mean);
                    acc = __dadd_rn(acc, __dmul_rn(d, d));
                }
            }
            __syncthreads();
        }
        if (tid == 0)
        {
            sAcc[0] = acc;
            sNum0 = num0;
        }
        if (tid == 32)
            sAcc[1] = acc;
        __syncthreads();
        if (tid == 0)
        {
            double lower, upper;
            if (bits == 1)
            {
                unsigned n0 = sNum0, n1 = (unsigned) M - sNum0;
                const double a0 = sAcc[0], a1 = sAcc[1];
                double radius, newmean;
                if (!zeroThr)
                {
                    const double devacc0 = __dsub_rn(__dmul_rn((double) n0, mean), a0);
                    const double devacc1 = __dsub_rn(a1, __dmul_rn((double) n1, mean));
                    const double dev = __ddiv_rn(__dadd_rn(devacc0, devacc1), rows);
                    radius = __dmul_rn((double) 2.0f, dev);
                    newmean = mean;
                }
                else
                {
                    if (n0 == 0)
                        n0 = 1;
                    if (n1 == 0)
                        n1 = 1;
                    const double mean0 = __ddiv_rn(a0, (double) n0);
                    const double mean1 = __ddiv_rn(a1, (double) n1);
                    newmean = __dmul_rn((double) 0.5f, __dadd_rn(mean0, mean1));
                    radius = __dmul_rn((double) 2.0f, __dsub_rn(mean1, newmean));
                }
                lower = __dsub_rn(newmean, radius);
                upper = __dadd_rn(newmean, radius);
            }
            else
            {
                const double stddev = __dsqrt_rn(__ddiv_rn(sAcc[0], rows));
                const double w = __dmul_rn((double) 4.0f, stddev);
                lower = __dsub_rn(mean, w);
                upper = __dadd_rn(mean, w);
            }
            sRange[0] = lower;
            sRange[1] = upper;
            double* hdr = reinterpret_cast<double*>(packed + j * colBytes);
            hdr[0] = lower;
            hdr[1] = upper;
        }
        __syncthreads();
        // QuantizeOneQWord: thread <-> packed word w, rows w, w + Q, ...
        const ValQD q = make_valq_d(bits, sRange[0], sRange[1]);
        unsigned long long* __restrict__ words = reinterpret_cast<unsigned long long*>(packed + j * colBytes + 16);
        double* __restrict__ ro = resOut + j * M;
        for (long long w = tid; w < Q; w += DNT)
        {
            unsigned long long word = 0ull;
            long long i = w;
            for (int k = 0; k < vpw && i < M; ++k, i += Q)
            {
                const double v = __dadd_rn(g[i], r[i]);
                const unsigned long long qv = quantize_d(q, bits, zeroThr != 0, v);
                ro[i] = __dsub_rn(v, unquantize_d(q, bits, qv));
                word |= qv << (k * bits);
            }
            words[w] = word;
        }
        __syncthreads();
    }
}

// UnquantizeOneQWord (ColumnQuantizer.h:150-203): thread <-> packed word
__global__ void __launch_bounds__(256) k_unquantize_f64(const unsigned char* __restrict__ packed, double* __restrict__ out, long long M, long long N, int bits,
                                                        int add)
{
    const long long Q = (M * bits + 63) / 64;
    const long long colBytes = 16 + 8 * Q;
    const int vpw = 64 / bits;
    const long long total = N * Q;
    for (long long t = (long long) blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long) gridDim.x * blockDim.x)
    {
        const long long j = t / Q, w = t - j * Q;
        const unsigned char* colp = packed + j * colBytes;
        const ValQD q = make_valq_d(bits, reinterpret_cast<const double*>(colp)[0], reinterpret_cast<const double*>(colp)[1]);
        const unsigned long long word = reinterpret_cast<const unsigned long long*>(colp + 16)[w];
        const unsigned long long mask = q.rangeend - 1ull; // all ones when rangeend == 0 (full-word pass-through)
        double* __restrict__ o = out + j * M;
        long long i = w;
        for (int k = 0; k < vpw && i < M; ++k, i += Q)
        {
            double v = unquantize_d(q, bits, (word >> (k * bits)) & mask);
            if (add)
                v = __dadd_rn(v, o[i]);
            o[i] = v;
        }
    }
}

static bool bits_ok_f64(int bits)
{
    return bits >= 1 && bits <= 64 && (bits & (bits - 1)) == 0;
}

} // namespace qagg

using namespace qagg;

extern "C" {

int64_t qagg_packed_col_bytes_f64(int64_t M, int bits)
{
    if (!bits_ok_f64(bits) || M < 0)
        return fail(QAGG_EINVAL, "qagg_packed_col_bytes_f64: bad arguments");
    return 16 + 8 * ((M * bits + 63) / 64);
}

int64_t qagg_packed_bytes_f64(int64_t M, int64_t N, int bits)
{
    if (!bits_ok_f64(bits) || M < 0 || N < 0)
        return fail(QAGG_EINVAL, "qagg_packed_bytes_f64: bad arguments");
    return N * (16 + 8 * ((M * bits + 63) / 64));
}

int qagg_quantize_f64(void* stream, const double* grad, const double* res_in, double* res_out, void* packed, int64_t M, int64_t N, int bits,
                      int zero_threshold)
{
    if (!bits_ok_f64(bits))
        return fail(QAGG_EINVAL, "bits must be a power of two in 1..64");
    if (M < 0 || N < 0 || M > 0x3fffffffLL || N > 0x7fffffffLL)
        return fail(QAGG_EINVAL, "qagg_quantize_f64: bad matrix shape");
    if (M == 0 || N == 0)
        return QAGG_OK;
    if (!grad || !res_in || !res_out || !packed)
        return fail(QAGG_EINVAL, "qagg_quantize_f64: null pointer");
    if ((reinterpret_cast<uintptr_t>(packed) & 7) || (reinterpret_cast<uintptr_t>(grad) & 7) || (reinterpret_cast<uintptr_t>(res_in) & 7) ||
        (reinterpret_cast<uintptr_t>(res_out) & 7))
        return fail(QAGG_EINVAL, "qagg_quantize_f64: buffers must be 8-byte aligned");
    const int grid = (int) (N < 148 * 16 ? N : 148 * 16);
    k_quantize_f64<<<grid, DNT, 0, (cudaStream_t) stream>>>(grad, res_in, res_out, static_cast<unsigned char*>(packed), M, N, bits, zero_threshold ? 1 : 0);
    return check_cuda(cudaGetLastError(), "double quantize kernel launch");
}

int qagg_unquantize_f64(void* stream, const void* packed, double* out, int64_t M, int64_t N, int bits, int add)
{
    if (!bits_ok_f64(bits))
        return fail(QAGG_EINVAL, "bits must be a power of two in 1..64");
    if (M < 0 || N < 0 || M > 0x3fffffffLL || N > 0x7fffffffLL)
        return fail(QAGG_EINVAL, "qagg_unquantize_f64: bad matrix shape");
    if (M == 0 || N == 0)
        return QAGG_OK;
    if (!packed || !out)
        return fail(QAGG_EINVAL, "qagg_unquantize_f64: null pointer");
    if ((reinterpret_cast<uintptr_t>(packed) & 7) || (reinterpret_cast<uintptr_t>(out) & 7))
        return fail(QAGG_EINVAL, "qagg_unquantize_f64: buffers must be 8-byte aligned");
    const long long total = N * ((M * bits + 63) / 64);
    long long grid = (total + 255) / 256;
    if (grid > 148 * 8)
        grid = 148 * 8;
    k_unquantize_f64<<<(int) grid, 256, 0, (cudaStream_t) stream>>>(static_cast<const unsigned char*>(packed), out, M, N, bits, add ? 1 : 0);
    return check_cuda(cudaGetLastError(), "double unquantize kernel launch");
}

} // extern "C"
