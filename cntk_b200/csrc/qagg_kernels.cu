// qagg_kernels.cu -- sm_100a kernels of the quantized gradient aggregation path.
//
// Arithmetic contract (what makes the results bit-identical to the reference CPU quantizer,
// Source/Math/ColumnQuantizer.h:209-341 and Source/Math/ValueQuantizer.h:68-162):
//   * every float operation is an explicit round-to-nearest intrinsic (__fadd_rn, __fmul_rn, __fdiv_rn,
//     __fsqrt_rn), so nothing is contracted into a fused multiply-add;
//   * the per-column sums (level sums for 1 bit, sum of squares otherwise, and the mean in mean-threshold
//     mode) are accumulated in ROW ORDER by one lane per column -- float addition is not associative and the
//     reference adds sequentially; counts are integers and need no order.
// A column's fp32 values (gradient + residual, or the sum of the received stripes + stripe residual) are
// staged once in shared memory; the ordered walk, the quantisation, the bit packing and the residual update
// all read them from there, so HBM sees each input and each output exactly once.
#include "qagg_internal.h"

namespace qagg {

constexpr int NT = 256; // threads per CTA

// ---- value quantizer (ValueQuantizer<float>, Source/Math/ValueQuantizer.h:68-162) ---------------------
struct ValQ
{
    float qmin, qmax, qmid, qfactor, ufactor;
    unsigned rangeend;
};

__device__ __forceinline__ ValQ make_valq(int bits, float lower, float upper)
{
    ValQ q;
    q.qmin = lower;
    q.qmax = upper;
    q.rangeend = (bits >= 32) ? 0u : (1u << bits);
    const float range = __fsub_rn(upper, lower);
    if ((range < 1e-36f) || (q.rangeend == 0))
    {
        q.qfactor = q.ufactor = 0.0f;
    }
    else
    {
        const float used = (float) (q.rangeend - (bits > 1 ? 1u : 0u));
        q.qfactor = __fdiv_rn(used, range);
        q.ufactor = __fdiv_rn(range, used);
    }
    q.qmid = __fmul_rn(0.5f, __fadd_rn(upper, lower));
    return q;
}

__device__ __forceinline__ float unquantize_val(const ValQ& q, int bits, unsigned u)
{
    if (bits == 32)
        return __uint_as_float(u);
    return __fadd_rn(__fmul_rn(__fadd_rn((float) u, 0.5f), q.ufactor), q.qmin);
}

__device__ __forceinline__ unsigned quantize_multibit(const ValQ& q, int bits, float v)
{
    if (bits == 32)
        return __float_as_uint(v);
    if (v <= q.qmin)
        return 0u;
    if (v >= q.qmax)
        return q.rangeend - 1u;
    return (unsigned) __float2int_rz(__fmul_rn(__fsub_rn(v, q.qmin), q.qfactor));
}

// ---- routing of packed column j to its owner (GetStripeForNode, AllReduceDistGradAggregator.h:56-65) ----
__device__ __forceinline__ unsigned char* packed_col(const QTensor& T, long long j)
{
    int p = 0;
    long long start = 0;
    if (T.K > 1)
    {
        const long long big = (T.per + 1) * T.rem; // columns held by the ranks that got one extra
        if (j < big)
        {
            p = (int) (j / (T.per + 1));
            start = (long long) p * (T.per + 1);
        }
        else
        {
            p = (int) (T.rem + (j - big) / T.per);
            start = big + ((long long) p - T.rem) * T.per;
        }
    }
    return T.pk[p] + (j - start) * T.colBytes;
}

// ---- element (row, column j) of the matrix being quantized; slow general form ---------------------------
template <bool STRIPES>
__device__ __forceinline__ float load_v(const QTensor& T, long long j, long long row)
{
    const long long ij = j * T.M + row;
    if (!STRIPES)
    {
        return __fadd_rn(T.grad[ij], T.res_in[ij]);
    }
    else
    {
        const int w = (int) (row % T.Q);
        const int shift = (int) (row / T.Q) * T.bits;
        const unsigned mask = (T.bits >= 32) ? 0xffffffffu : ((1u << T.bits) - 1u);
        float agg = 0.0f;
        bool first = true;
        if (T.selfRaw)
        {
            agg = T.grad[ij];
            first = false;
        }
        for (int s = T.selfRaw ? 1 : 0; s < T.nsrc; ++s)
        {
            const unsigned char* colp = T.src[s] + j * T.colBytes;
            const ValQ q = make_valq(T.bits, ((const float*) colp)[0], ((const float*) colp)[1]);
            const unsigned word = ((const unsigned*) (colp + 8))[w];
            const float val = unquantize_val(q, T.bits, (word >> shift) & mask);
            agg = first ? val : __fadd_rn(val, agg);
            first = false;
        }
        return __fadd_rn(agg, T.res_in[ij]);
    }
}

// ---- ordered accumulation over rows [0, nrows) of one staged column -------------------------------------
struct Acc
{
    float a0 = 0.0f, a1 = 0.0f; // level sums (1 bit) / sum of squares in a0 (multi-bit)
    float am = 0.0f;            // plain sum (mean-threshold mode, first pass)
    unsigned n0 = 0;            // values below the threshold
};

template <int MODE, bool MEANPASS>
__device__ __forceinline__ void walk_one(Acc& A, float v, float mean)
{
    if (MEANPASS)
    {
        A.am = __fadd_rn(A.am, v);
    }
    else if (MODE == MODE_MULTIBIT)
    {
        const float d = __fsub_rn(v, mean);
        A.a0 = __fadd_rn(A.a0, __fmul_rn(d, d));
    }
    else
    {
        if (v < mean)
        {
            A.a0 = __fadd_rn(A.a0, v);
            A.n0++;
        }
        else
        {
            A.a1 = __fadd_rn(A.a1, v);
        }
    }
}

template <int MODE, bool MEANPASS>
__device__ __forceinline__ void walk(const float* __restrict__ vcol, int nrows, Acc& A, float mean)
{
    int i = 0;
    for (; i + 4 <= nrows; i += 4)
    {
        const float4 v = *reinterpret_cast<const float4*>(vcol + i);
        walk_one<MODE, MEANPASS>(A, v.x, mean);
        walk_one<MODE, MEANPASS>(A, v.y, mean);
        walk_one<MODE, MEANPASS>(A, v.z, mean);
        walk_one<MODE, MEANPASS>(A, v.w, mean);
    }
    for (; i < nrows; ++i)
        walk_one<MODE, MEANPASS>(A, vcol[i], mean);
}

// range of one column from its ordered sums (ColumnQuantizer.h:279-316, 320-339)
template <int MODE>
__device__ __forceinline__ void finalize_range(const Acc& A, float mean, long long M, float& lower, float& upper)
{
    const float rows = (float) (unsigned long long) M;
    if (MODE == MODE_MULTIBIT)
    {
        const float stddev = __fsqrt_rn(__fdiv_rn(A.a0, rows));
        const float w = __fmul_rn(4.0f, stddev);
        lower = __fsub_rn(mean, w);
        upper = __fadd_rn(mean, w);
        return;
    }
    unsigned num0 = A.n0;
    unsigned num1 = (unsigned) M - A.n0;
    float radius, newmean;
    if (MODE == MODE_ONEBIT_MEAN)
    {
        const float devacc0 = __fsub_rn(__fmul_rn((float) num0, mean), A.a0);
        const float devacc1 = __fsub_rn(A.a1, __fmul_rn((float) num1, mean));
        const float dev = __fdiv_rn(__fadd_rn(devacc0, devacc1), rows);
        radius = __fmul_rn(2.0f, dev);
        newmean = mean;
    }
    else
    {
        if (num0 == 0)
            num0 = 1;
        if (num1 == 0)
            num1 = 1;
        const float mean0 = __fdiv_rn(A.a0, (float) num0);
        const float mean1 = __fdiv_rn(A.a1, (float) num1);
        newmean = __fmul_rn(0.5f, __fadd_rn(mean0, mean1));
        radius = __fmul_rn(2.0f, __fsub_rn(mean1, newmean));
    }
    lower = __fsub_rn(newmean, radius);
    upper = __fadd_rn(newmean, radius);
}

// ---- quantize + pack + residual for word w of column j (QuantizeOneQWord, ColumnQuantizer.h:90-147) --------
template <int MODE, bool STRIPES, bool RESIDENT>
__device__ __forceinline__ void quantize_word(const QTensor& T, long long j, int w, const float* __restrict__ vcol,
                                              float lower, float upper)
{
    const ValQ q = make_valq(T.bits, lower, upper);
    float* __restrict__ rcol = T.res_out + j * T.M;
    const long long M = T.M;
    const int Q = T.Q;
    unsigned word = 0;
    if (MODE != MODE_MULTIBIT)
    {
        const float val0 = unquantize_val(q, 1, 0u);
        const float val1 = unquantize_val(q, 1, 1u);
#pragma unroll 8
        for (int k = 0; k < 32; ++k)
        {
            const long long row = (long long) w + (long long) k * Q;
            if (row < M)
            {
                const float v = RESIDENT ? vcol[row] : load_v<STRIPES>(T, j, row);
                const bool bit = (MODE == MODE_ONEBIT_ZERO) ? (v >= 0.0f) : (v >= q.qmid);
                rcol[row] = __fsub_rn(v, bit ? val1 : val0);
                word |= (bit ? 1u : 0u) << k;
            }
        }
    }
    else
    {
        const int bits = T.bits;
        const int vpw = 32 / bits;
        for (int k = 0; k < vpw; ++k)
        {
            const long long row = (long long) w + (long long) k * Q;
            if (row < M)
            {
                const float v = RESIDENT ? vcol[row] : load_v<STRIPES>(T, j, row);
                const unsigned qv = quantize_multibit(q, bits, v);
                rcol[row] = __fsub_rn(v, unquantize_val(q, bits, qv));
                word |= qv << (k * bits);
            }
        }
    }
    unsigned char* dst = packed_col(T, j);
    reinterpret_cast<unsigned*>(dst + 8)[w] = word;
    if (w == 0)
    {
        reinterpret_cast<float*>(dst)[0] = lower;
        reinterpret_cast<float*>(dst)[1] = upper;
    }
}

// ---- stage nc whole columns into shared memory -------------------------------------------------------------
template <bool STRIPES>
__device__ __forceinline__ void fill_resident(const QTensor& T, int col0, int nc, int stride, float* __restrict__ smem)
{
    const long long M = T.M;
    if (!STRIPES)
    {
        const float* __restrict__ g = T.grad + (long long) col0 * M;
        const float* __restrict__ r = T.res_in + (long long) col0 * M;
        const bool vec = ((M & 3) == 0) && ((reinterpret_cast<uintptr_t>(g) & 15) == 0) && ((reinterpret_cast<uintptr_t>(r) & 15) == 0);
        if (vec)
        {
            const int M4 = (int) (M >> 2);
            const int total = nc * M4;
            for (int idx = threadIdx.x; idx < total; idx += NT)
            {
                const int col = idx / M4;
                const int r4 = idx - col * M4;
                const float4 a = __ldg(reinterpret_cast<const float4*>(g) + idx);
                const float4 b = __ldg(reinterpret_cast<const float4*>(r) + idx);
                float4 v;
                v.x = __fadd_rn(a.x, b.x);
                v.y = __fadd_rn(a.y, b.y);
                v.z = __fadd_rn(a.z, b.z);
                v.w = __fadd_rn(a.w, b.w);
                *reinterpret_cast<float4*>(smem + (size_t) col * stride + 4 * r4) = v;
            }
        }
        else
        {
            const long long total = (long long) nc * M;
            for (long long idx = threadIdx.x; idx < total; idx += NT)
            {
                const int col = (int) (idx / M);
                const int row = (int) (idx - (long long) col * M);
                smem[(size_t) col * stride + row] = __fadd_rn(g[idx], r[idx]);
            }
        }
    }
    else
    {
        // thread <-> (column, word): sources are added in index order; the raw own stripe (if used) comes first
        const int Q = T.Q;
        const int bits = T.bits;
        const int vpw = 32 / bits;
        const unsigned mask = (bits >= 32) ? 0xffffffffu : ((1u << bits) - 1u);
        const int total = nc * Q;
        for (int idx = threadIdx.x; idx < total; idx += NT)
        {
            const int col = idx / Q;
            const int w = idx - col * Q;
            const long long j = (long long) col0 + col;
            float* __restrict__ vcol = smem + (size_t) col * stride;
            bool first = true;
            if (T.selfRaw)
            {
                const float* __restrict__ gcol = T.grad + j * M;
                for (int k = 0; k < vpw; ++k)
                {
                    const long long row = (long long) w + (long long) k * Q;
                    if (row < M)
                        vcol[row] = gcol[row];
                }
                first = false;
            }
            for (int s = T.selfRaw ? 1 : 0; s < T.nsrc; ++s)
            {
                const unsigned char* colp = T.src[s] + j * T.colBytes;
                const ValQ q = make_valq(bits, reinterpret_cast<const float*>(colp)[0], reinterpret_cast<const float*>(colp)[1]);
                const unsigned word = reinterpret_cast<const unsigned*>(colp + 8)[w];
                if (bits == 1)
                {
                    const float val0 = unquantize_val(q, 1, 0u);
                    const float val1 = unquantize_val(q, 1, 1u);
#pragma unroll 8
                    for (int k = 0; k < 32; ++k)
                    {
                        const long long row = (long long) w + (long long) k * Q;
                        if (row < M)
                        {
                            const float val = ((word >> k) & 1u) ? val1 : val0;
                            vcol[row] = first ? val : __fadd_rn(val, vcol[row]);
                        }
                    }
                }
                else
                {
                    for (int k = 0; k < vpw; ++k)
                    {
                        const long long row = (long long) w + (long long) k * Q;
                        if (row < M)
                        {
                            const float val = unquantize_val(q, bits, (word >> (k * bits)) & mask);
                            vcol[row] = first ? val : __fadd_rn(val, vcol[row]);
                        }
                    }
                }
                first = false;
            }
            const float* __restrict__ rcol = T.res_in + j * M;
            for (int k = 0; k < vpw; ++k)
            {
                const long long row = (long long) w + (long long) k * Q;
                if (row < M)
                    vcol[row] = __fadd_rn(first ? 0.0f : vcol[row], rcol[row]);
            }
        }
    }
}

// =================================================================================================================
// Column quantizer kernel.  One work item = up to 32 adjacent columns of one matrix.
//   A. all threads stage the columns' fp32 values in shared memory (one coalesced pass over the inputs);
//   B. warp 0 walks them in row order, one lane per column, and derives each column's range;
//   C. all threads quantize, pack words, write the residual and the packed column to its owner's buffer.
// Columns too tall to stage are streamed through shared memory in chunks for B and re-read for C.
// =================================================================================================================
template <bool STRIPES, int MODE, bool TABLE>
__global__ void __launch_bounds__(NT) k_colquant(const QTensor single, const QTensor* __restrict__ tensors,
                                                 const QItem* __restrict__ items, int nItems, int colsPerItem, int smemFloats)
{
    extern __shared__ __align__(16) float smem[];
    __shared__ QTensor sT;
    __shared__ float sLower[32], sUpper[32];

    for (int it = blockIdx.x; it < nItems; it += gridDim.x)
    {
        int col0, nc;
        __syncthreads(); // previous item fully done with sT / smem / sLower
        if (TABLE)
        {
            const QItem item = items[it];
            col0 = item.col0;
            nc = item.ncols;
            const int* srcw = reinterpret_cast<const int*>(tensors + item.tensor);
            int* dstw = reinterpret_cast<int*>(&sT);
            for (int i = threadIdx.x; i < (int) (sizeof(QTensor) / sizeof(int)); i += NT)
                dstw[i] = srcw[i];
        }
        else
        {
            col0 = it * colsPerItem;
            nc = (int) min((long long) colsPerItem, single.N - col0);
            if (threadIdx.x == 0)
                sT = single;
        }
        __syncthreads();
        const QTensor& T = sT;
        const long long M = T.M;
        const int stride = smem_stride(M);
        const bool resident = ((long long) nc * stride <= (long long) smemFloats);
        const int lane = threadIdx.x & 31;
        const int warp = threadIdx.x >> 5;

        if (resident)
        {
            fill_resident<STRIPES>(T, col0, nc, stride, smem);
            __syncthreads();
            if (warp == 0 && lane < nc)
            {
                const float* vcol = smem + (size_t) lane * stride;
                Acc A;
                float mean = 0.0f;
                if (MODE == MODE_ONEBIT_MEAN)
                {
                    walk<MODE, true>(vcol, (int) M, A, 0.0f);
                    mean = __fdiv_rn(A.am, (float) (unsigned long long) M);
                }
                walk<MODE, false>(vcol, (int) M, A, mean);
                float lo, up;
                finalize_range<MODE>(A, mean, M, lo, up);
                sLower[lane] = lo;
                sUpper[lane] = up;
            }
            __syncthreads();
            const int Q = T.Q;
            const int total = nc * Q;
            for (int idx = threadIdx.x; idx < total; idx += NT)
            {
                const int col = idx / Q;
                const int w = idx - col * Q;
                quantize_word<MODE, STRIPES, true>(T, (long long) col0 + col, w, smem + (size_t) col * stride, sLower[col], sUpper[col]);
            }
        }
        else
        {
            // chunked: rows [r0, r0+cs) of the nc columns at a time
            int cs = ((smemFloats / nc - 4) / 32) * 32 + 4;
            Acc A;
            float mean = 0.0f;
            const int passes = (MODE == MODE_ONEBIT_MEAN) ? 2 : 1;
            for (int pass = 0; pass < passes; ++pass)
            {
                const bool meanPass = (MODE == MODE_ONEBIT_MEAN) && (pass == 0);
                for (long long r0 = 0; r0 < M; r0 += cs)
                {
                    const int nr = (int) min((long long) cs, M - r0);
                    const int total = nc * nr;
                    for (int idx = threadIdx.x; idx < total; idx += NT)
                    {
                        const int col = idx / nr;
                        const int rr = idx - col * nr;
                        smem[(size_t) col * cs + rr] = load_v<STRIPES>(T, (long long) col0 + col, r0 + rr);
                    }
                    __syncthreads();
                    if (warp == 0 && lane < nc)
                    {
                        if (meanPass)
                            walk<MODE, true>(smem + (size_t) lane * cs, nr, A, 0.0f);
                        else
                            walk<MODE, false>(smem + (size_t) lane * cs, nr, A, mean);
                    }
                    __syncthreads();
                }
                if (meanPass)
                    mean = __fdiv_rn(A.am, (float) (unsigned long long) M);
            }
            if (warp == 0 && lane < nc)
            {
                float lo, up;
                finalize_range<MODE>(A, mean, M, lo, up);
                sLower[lane] = lo;
                sUpper[lane] = up;
            }
            __syncthreads();
            const int Q = T.Q;
            const long long total = (long long) nc * Q;
            for (long long idx = threadIdx.x; idx < total; idx += NT)
            {
                const int col = (int) (idx / Q);
                const int w = (int) (idx - (long long) col * Q);
                quantize_word<MODE, STRIPES, false>(T, (long long) col0 + col, w, nullptr, sLower[col], sUpper[col]);
            }
        }
    }
}

// =================================================================================================================
// Unquantize kernel (UnquantizeOneQWord, ColumnQuantizer.h:150-203): thread <-> packed word, rows w + k*Q.
// =================================================================================================================
template <bool ADD, bool TABLE>
__global__ void __launch_bounds__(NT) k_unquantize(const QTensor single, const QTensor* __restrict__ tensors,
                                                   const QItem* __restrict__ items, int nItems, int colsPerItem)
{
    __shared__ QTensor sT;
    for (int it = blockIdx.x; it < nItems; it += gridDim.x)
    {
        int col0, nc;
        __syncthreads();
        if (TABLE)
        {
            const QItem item = items[it];
            col0 = item.col0;
            nc = item.ncols;
            const int* srcw = reinterpret_cast<const int*>(tensors + item.tensor);
            int* dstw = reinterpret_cast<int*>(&sT);
            for (int i = threadIdx.x; i < (int) (sizeof(QTensor) / sizeof(int)); i += NT)
                dstw[i] = srcw[i];
        }
        else
        {
            col0 = it * colsPerItem;
            nc = (int) min((long long) colsPerItem, single.N - col0);
            if (threadIdx.x == 0)
                sT = single;
        }
        __syncthreads();
        const QTensor& T = sT;
        const long long M = T.M;
        const int Q = T.Q;
        const int bits = T.bits;
        const int vpw = 32 / bits;
        const unsigned mask = (bits >= 32) ? 0xffffffffu : ((1u << bits) - 1u);
        const long long total = (long long) nc * Q;
        for (long long idx = threadIdx.x; idx < total; idx += NT)
        {
            const int col = (int) (idx / Q);
            const int w = (int) (idx - (long long) col * Q);
            const long long j = (long long) col0 + col;
            const unsigned char* colp = packed_col(T, j);
            const ValQ q = make_valq(bits, reinterpret_cast<const float*>(colp)[0], reinterpret_cast<const float*>(colp)[1]);
            const unsigned word = reinterpret_cast<const unsigned*>(colp + 8)[w];
            float* __restrict__ ocol = T.out + j * M;
            if (bits == 1)
            {
                const float val0 = unquantize_val(q, 1, 0u);
                const float val1 = unquantize_val(q, 1, 1u);
#pragma unroll 8
                for (int k = 0; k < 32; ++k)
                {
                    const long long row = (long long) w + (long long) k * Q;
                    if (row < M)
                    {
                        float val = ((word >> k) & 1u) ? val1 : val0;
                        if (ADD)
                            val = __fadd_rn(val, ocol[row]);
                        ocol[row] = val;
                    }
                }
            }
            else
            {
                for (int k = 0; k < vpw; ++k)
                {
                    const long long row = (long long) w + (long long) k * Q;
                    if (row < M)
                    {
                        float val = unquantize_val(q, bits, (word >> (k * bits)) & mask);
                        if (ADD)
                            val = __fadd_rn(val, ocol[row]);
                        ocol[row] = val;
                    }
                }
            }
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------------------

int cols_per_item(long long M, long long N, int smemFloats, bool* resident)
{
    const int stride = smem_stride(M);
    long long c = smemFloats / stride;
    bool res = true;
    if (c < 1)
    {
        res = false;
        c = 8; // streamed in row chunks of smemFloats / 8
    }
    if (c > 32)
        c = 32;
    if (c > N)
        c = N;
    if (c < 1)
        c = 1;
    if (resident)
        *resident = res;
    return (int) c;
}

int unq_cols_per_item(long long M)
{
    long long c = 65536 / (M > 0 ? M : 1);
    if (c < 1)
        c = 1;
    if (c > 4096)
        c = 4096;
    return (int) c;
}

template <bool STRIPES, int MODE, bool TABLE>
static cudaError_t launch_cq(cudaStream_t st, const QTensor* single, const QTensor* tensors, const QItem* items,
                             int nItems, int colsPerItem, const LaunchCfg& cfg)
{
    auto kern = k_colquant<STRIPES, MODE, TABLE>;
    const size_t smemBytes = (size_t) cfg.smemFloats * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smemBytes);
    if (e != cudaSuccess)
        return e;
    int grid = cfg.numSMs * cfg.ctasPerSM;
    if (grid > nItems)
        grid = nItems;
    static const QTensor zero = {};
    kern<<<grid, NT, smemBytes, st>>>(single ? *single : zero, tensors, items, nItems, colsPerItem, cfg.smemFloats);
    return cudaGetLastError();
}

cudaError_t launch_colquant(cudaStream_t st, bool stripes, int mode, const QTensor* single, const QTensor* tensors,
                            const QItem* items, int nItems, int colsPerItem, const LaunchCfg& cfg)
{
    if (nItems <= 0)
        return cudaSuccess;
    const bool table = (single == nullptr);
#define QAGG_CASE(S, MD, TB) \
    if (stripes == S && mode == MD && table == TB) \
        return launch_cq<S, MD, TB>(st, single, tensors, items, nItems, colsPerItem, cfg);
    QAGG_CASE(false, MODE_ONEBIT_ZERO, false)
    QAGG_CASE(false, MODE_ONEBIT_MEAN, false)
    QAGG_CASE(false, MODE_MULTIBIT, false)
    QAGG_CASE(true, MODE_ONEBIT_ZERO, false)
    QAGG_CASE(true, MODE_ONEBIT_MEAN, false)
    QAGG_CASE(true, MODE_MULTIBIT, false)
    QAGG_CASE(false, MODE_ONEBIT_ZERO, true)
    QAGG_CASE(false, MODE_ONEBIT_MEAN, true)
    QAGG_CASE(false, MODE_MULTIBIT, true)
    QAGG_CASE(true, MODE_ONEBIT_ZERO, true)
    QAGG_CASE(true, MODE_ONEBIT_MEAN, true)
    QAGG_CASE(true, MODE_MULTIBIT, true)
#undef QAGG_CASE
    return cudaErrorInvalidValue;
}

cudaError_t launch_unquantize(cudaStream_t st, bool add, const QTensor* single, const QTensor* tensors,
                              const QItem* items, int nItems, int colsPerItem, const LaunchCfg& cfg)
{
    if (nItems <= 0)
        return cudaSuccess;
    int grid = cfg.numSMs * 8;
    if (grid > nItems)
        grid = nItems;
    static const QTensor zero = {};
    const QTensor& s = single ? *single : zero;
    if (single)
    {
        if (add)
            k_unquantize<true, false><<<grid, NT, 0, st>>>(s, tensors, items, nItems, colsPerItem);
        else
            k_unquantize<false, false><<<grid, NT, 0, st>>>(s, tensors, items, nItems, colsPerItem);
    }
    else
    {
        if (add)
            k_unquantize<true, true><<<grid, NT, 0, st>>>(s, tensors, items, nItems, colsPerItem);
        else
            k_unquantize<false, true><<<grid, NT, 0, st>>>(s, tensors, items, nItems, colsPerItem);
    }
    return cudaGetLastError();
}

cudaError_t get_launch_cfg(int device, LaunchCfg* cfg)
{
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess)
        return e;
    cfg->numSMs = prop.multiProcessorCount;
    // two CTAs per SM: (per-SM shared memory - 1 KB reserved per CTA) / 2, rounded down to 1 KB
    size_t perSM = prop.sharedMemPerMultiprocessor;
    size_t perCta = (perSM / 2) - 1024 - 2048; // 2 KB slack for the kernel's static shared memory
    if (perCta > prop.sharedMemPerBlockOptin - 2048)
        perCta = prop.sharedMemPerBlockOptin - 2048;
    perCta &= ~(size_t) 1023;
    cfg->smemFloats = (int) (perCta / sizeof(float));
    cfg->ctasPerSM = 2;
    return cudaSuccess;
}

} // namespace qagg
