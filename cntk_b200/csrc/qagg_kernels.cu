// qagg_kernels.cu -- sm_100a kernels of the quantized gradient aggregation path.
//
// Arithmetic contract (what makes the results bit-identical to the reference CPU quantizer,
// Source/Math/ColumnQuantizer.h:209-341 and Source/Math/ValueQuantizer.h:68-162):
//   * every float operation is an explicit round-to-nearest intrinsic (__fadd_rn, __fmul_rn, __fdiv_rn,
//     __fsqrt_rn), so nothing is contracted into a fused multiply-add;
//   * the per-column sums (level sums for 1 bit, sum of squares otherwise, and the mean in mean-threshold
//     mode) are accumulated in ROW ORDER -- float addition is not associative and the reference adds
//     sequentially.  Each of the two level sums of a 1-bit column is its own chain (one lane each); counts
//     are integers, need no order, and are gathered by all threads with redux / shared-memory atomics.
// A column's fp32 values (gradient + residual, or the sum of the received stripes + stripe residual) are
// staged once in shared memory; the ordered walk, the quantisation, the bit packing and the residual update
// all read them from there, so HBM sees each input and each output exactly once.
//
// NaN inputs: a NaN in a column makes that column's range NaN, as in the reference, but the payload bits of
// the resulting NaNs are unspecified.  Zeros of either sign are handled exactly.
#include "qagg_device.cuh"

namespace qagg {

constexpr int CMAX = 128;   // most columns in one work item

// per-item scratch that lives behind the staged columns in dynamic shared memory
struct ColStats
{
    float* lower;
    float* upper;
    unsigned* n0;   // zero-threshold mode: values < 0, counted while staging
    unsigned* nan;  // zero-threshold mode: the column holds a NaN
    float* a0;      // zero-threshold mode: the two level sums, written by the two walking warps
    float* a1;
};
constexpr int COLSTAT_FLOATS = 8; // shared-memory floats reserved per column for the arrays above

// =================================================================================================================
// Phase A: stage nc whole columns (v = gradient + residual, or sum of stripes + stripe residual).
// =================================================================================================================
template <int MODE>
__device__ __forceinline__ void count4(const float4& v, unsigned& cnt, unsigned& nan)
{
    if (MODE == MODE_ONEBIT_ZERO)
    {
        cnt += (v.x < 0.0f) + (v.y < 0.0f) + (v.z < 0.0f) + (v.w < 0.0f);
        nan |= (v.x != v.x) | (v.y != v.y) | (v.z != v.z) | (v.w != v.w);
    }
}

template <int MODE>
__device__ __forceinline__ void fill_dense(const QTensor& T, int col0, int nc, int stride, float* __restrict__ smem, const ColStats& S)
{
    const int M = (int) T.M;
    const float* __restrict__ g = T.grad + (size_t) col0 * M;
    const float* __restrict__ r = T.res_in + (size_t) col0 * M;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool vec = ((M & 3) == 0) && ((reinterpret_cast<uintptr_t>(g) & 15) == 0) && ((reinterpret_cast<uintptr_t>(r) & 15) == 0);
    if (vec)
    {
        // warp task = 32 lanes x UNR float4 of ONE column.  The gradient goes global -> shared by cp.async (no registers,
        // every copy of the item in flight at once); the residual goes through registers, UNR loads in flight per lane.
        // A lane adds the residual only to the 16-byte slots it copied itself, so waiting for its own copy group is
        // all the synchronisation the two passes need.
        constexpr int UNR = 8;
        const int M4 = M >> 2;
        const int nch = (M4 + 32 * UNR - 1) / (32 * UNR);
        const int ntasks = nc * nch;
        for (int task = warp; task < ntasks; task += NWARPS)
        {
            const int col = task / nch;
            const int ch = task - col * nch;
            const float4* __restrict__ g4 = reinterpret_cast<const float4*>(g + (size_t) col * M);
            float4* __restrict__ v4 = reinterpret_cast<float4*>(smem + (size_t) col * stride);
            const int base = ch * 32 * UNR + lane;
#pragma unroll
            for (int u = 0; u < UNR; ++u)
            {
                const int idx = base + 32 * u;
                if (idx < M4)
                {
                    const unsigned dst = (unsigned) __cvta_generic_to_shared(v4 + idx);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(g4 + idx) : "memory");
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        bool waited = false;
        for (int task = warp; task < ntasks; task += NWARPS)
        {
            const int col = task / nch;
            const int ch = task - col * nch;
            const float4* __restrict__ r4 = reinterpret_cast<const float4*>(r + (size_t) col * M);
            float4* __restrict__ v4 = reinterpret_cast<float4*>(smem + (size_t) col * stride);
            const int base = ch * 32 * UNR + lane;
            float4 b[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u)
            {
                const int idx = base + 32 * u;
                if (idx < M4)
                    b[u] = __ldcs(r4 + idx);
            }
            if (!waited)
            {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                waited = true;
            }
            unsigned cnt = 0, nan = 0;
#pragma unroll
            for (int u = 0; u < UNR; ++u)
            {
                const int idx = base + 32 * u;
                if (idx < M4)
                {
                    const float4 a = v4[idx];
                    float4 v;
                    v.x = __fadd_rn(a.x, b[u].x);
                    v.y = __fadd_rn(a.y, b[u].y);
                    v.z = __fadd_rn(a.z, b[u].z);
                    v.w = __fadd_rn(a.w, b[u].w);
                    v4[idx] = v;
                    count4<MODE>(v, cnt, nan);
                }
            }
            if (MODE == MODE_ONEBIT_ZERO)
            {
                cnt = __reduce_add_sync(0xffffffffu, cnt);
                nan = __reduce_or_sync(0xffffffffu, nan);
                if (lane == 0)
                {
                    if (cnt)
                        atomicAdd(&S.n0[col], cnt);
                    if (nan)
                        S.nan[col] = 1u;
                }
            }
        }
        if (!waited)
            asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    else
    {
        const int total = nc * M;
        int cur = -1;
        unsigned cnt = 0;
        for (int idx = threadIdx.x; idx < total; idx += NT)
        {
            const int col = idx / M;
            const int row = idx - col * M;
            const float v = __fadd_rn(g[idx], r[idx]);
            smem[(size_t) col * stride + row] = v;
            if (MODE == MODE_ONEBIT_ZERO)
            {
                if (col != cur)
                {
                    if (cnt)
                        atomicAdd(&S.n0[cur], cnt);
                    cur = col;
                    cnt = 0;
                }
                cnt += (v < 0.0f);
                if (v != v)
                    S.nan[col] = 1u;
            }
        }
        if (MODE == MODE_ONEBIT_ZERO && cnt)
            atomicAdd(&S.n0[cur], cnt);
    }
}

// The K sources are added in index order, the raw own stripe (if used) first, the stripe residual LAST (the reference
// unquantizes with add = true K-1 times and only then quantizes against the residual, AllReduceDistGradAggregator.h:366-375,
// 405-435).  `pks` is shared-memory staging for the item's packed columns (nsrc x nc x (colBytes / 4) words), or null
// when that does not fit: then headers and words are read from global memory.
template <int MODE>
__device__ __forceinline__ void fill_stripes(const QTensor& T, int col0, int nc, int stride, float* __restrict__ smem, const ColStats& S,
                                             unsigned* __restrict__ pks)
{
    const int M = (int) T.M;
    const int Q = T.Q;
    const int bits = T.bits;
    const int vpw = 32 / bits;
    const unsigned mask = (bits >= 32) ? 0xffffffffu : ((1u << bits) - 1u);
    const int colWords = T.colBytes >> 2; // header (2 words) + Q packed words
    const float* __restrict__ r0 = T.res_in + (size_t) col0 * M;
    const bool async = ((M & 3) == 0) && ((reinterpret_cast<uintptr_t>(r0) & 15) == 0);
    // 1. everything this item reads goes into flight at once: the stripe residual (16-byte copies into the column slots)
    //    and the item's packed columns of all K sources (4-byte copies: packed columns are only 4-byte aligned)
    if (async)
    {
        const int M4 = M >> 2;
        const int total4 = nc * M4;
        for (int idx = threadIdx.x; idx < total4; idx += NT)
        {
            const int col = idx / M4;
            const int r4 = idx - col * M4;
            const unsigned dst = (unsigned) __cvta_generic_to_shared(smem + (size_t) col * stride + 4 * r4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(reinterpret_cast<const float4*>(r0) + idx) : "memory");
        }
    }
    if (pks)
    {
        const int perSrc = nc * colWords;
        const int totalW = T.nsrc * perSrc;
        for (int idx = threadIdx.x; idx < totalW; idx += NT)
        {
            const int s = idx / perSrc;
            const int rem = idx - s * perSrc;
            if (s == 0 && T.selfRaw)
                continue;
            const unsigned* src = reinterpret_cast<const unsigned*>(T.src[s] + (size_t) col0 * T.colBytes) + rem;
            const unsigned dst = (unsigned) __cvta_generic_to_shared(pks + idx);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    bool landed = false;
    if (pks)
    {
        // the sums below read the staged packed columns: everything must have landed first
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        landed = true;
    }

    // 2. thread <-> (column, packed word, half of the word's bit positions): sum of the K sources in registers, in
    //    index order, then the residual.  Splitting a word's positions over two threads doubles the number of tasks, which
    //    matters for tall columns (a 9304-row column has only 291 words for 256 threads).  Every thread runs the same
    //    number of trips, so the barrier inside the loop is safe.
    const int H = (bits == 1) ? 2 : 1;     // tasks per word
    const int KH = 32 / H;                 // bit positions (of the 1-bit layout) per task; multi-bit: all vpw <= 16 in one
    const int total = nc * Q * H;
    for (int idx0 = 0; idx0 < total; idx0 += NT)
    {
        const int idx = idx0 + threadIdx.x;
        const bool live = idx < total;
        const int cw = live ? idx / H : 0;
        const int kLo = live ? (idx - cw * H) * KH : 0;
        const int col = cw / Q;
        const int w = cw - col * Q;
        const int j = col0 + col;
        const int nkAll = live ? min(vpw, (M - w + Q - 1) / Q) : 0; // rows w, w+Q, ... below M
        const int nk = max(0, min(nkAll - kLo, KH));               // this task's share: positions kLo .. kLo + nk - 1
        float agg[16];
#pragma unroll
        for (int k = 0; k < 16; ++k)
            agg[k] = 0.0f;
        bool first = true;
        if (live && T.selfRaw)
        {
            const float* __restrict__ gcol = T.grad + (size_t) j * M + w + (size_t) kLo * Q;
#pragma unroll
            for (int k = 0; k < 16; ++k)
                if (k < nk)
                    agg[k] = gcol[k * Q];
            first = false;
        }
        for (int s = T.selfRaw ? 1 : 0; live && s < T.nsrc; ++s)
        {
            const unsigned* colp = pks ? pks + ((size_t) s * nc + col) * colWords
                                       : reinterpret_cast<const unsigned*>(T.src[s] + (size_t) j * T.colBytes);
            const unsigned word = colp[2 + w];
            if (bits == 1)
            {
                float val0, val1;
                levels_1bit(__uint_as_float(colp[0]), __uint_as_float(colp[1]), val0, val1);
                const unsigned part = word >> kLo;
#pragma unroll
                for (int k = 0; k < 16; ++k)
                {
                    const float val = ((part >> k) & 1u) ? val1 : val0;
                    agg[k] = first ? val : __fadd_rn(val, agg[k]);
                }
            }
            else
            {
                const ValQ q = make_valq(bits, __uint_as_float(colp[0]), __uint_as_float(colp[1]));
#pragma unroll
                for (int k = 0; k < 16; ++k)
                {
                    if (k < vpw)
                    {
                        const float val = unquantize_val(q, bits, (word >> (k * bits)) & mask);
                        agg[k] = first ? val : __fadd_rn(val, agg[k]);
                    }
                }
            }
            first = false;
        }
        if (!landed)
        {
            // the residual copies were in flight while the first sums were built from global memory
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            landed = true;
        }
        float* __restrict__ vcol = smem + (size_t) col * stride + w + (size_t) kLo * Q;
        const float* __restrict__ rcol = T.res_in + (size_t) j * M + w + (size_t) kLo * Q;
        unsigned cnt = 0;
#pragma unroll
        for (int k = 0; k < 16; ++k)
        {
            if (k < nk)
            {
                const float r = async ? vcol[k * Q] : rcol[k * Q];
                const float v = __fadd_rn(agg[k], r);
                vcol[k * Q] = v;
                if (MODE == MODE_ONEBIT_ZERO)
                {
                    cnt += (v < 0.0f);
                    if (v != v)
                        S.nan[col] = 1u;
                }
            }
        }
        if (MODE == MODE_ONEBIT_ZERO && cnt)
            atomicAdd(&S.n0[col], cnt);
    }
}

// =================================================================================================================
// Phase B: ordered sums and the column range.  1-bit modes use a lane pair per column (one chain per level).
// =================================================================================================================
template <int MODE>
__device__ __forceinline__ void walk_resident(const QTensor& T, int nc, int stride, const float* __restrict__ smem, const ColStats& S,
                                              int walkerWarp)
{
    const int M = (int) T.M;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // round r (16 column pairs, or 32 columns in multi-bit mode) is walked by warp (walkerWarp + r) % NWARPS: the first
    // round -- the only one for tall columns -- sits on a different warp in each CTA of an SM, so the walkers of the
    // co-resident CTAs do not share one scheduler
    if (MODE == MODE_MULTIBIT)
    {
        for (int r = 0; r * 32 < nc; ++r)
        {
            if (((walkerWarp + r) & (NWARPS - 1)) != warp)
                continue;
            const int col = r * 32 + lane;
            if (col < nc)
            {
                unsigned cnt = 0;
                const float a0 = walk_rows<WALK_SQUARES>(smem + (size_t) col * stride, M, 0.0f, cnt, 0.0f, false);
                float lo, up;
                finalize_range<MODE>(a0, 0.0f, 0u, 0.0f, T.M, lo, up);
                S.lower[col] = lo;
                S.upper[col] = up;
            }
        }
        return;
    }
    if (MODE == MODE_ONEBIT_ZERO)
    {
        // round r = 32 columns; its lower sums are walked by warp (walkerWarp + 2r) and its upper sums by the next warp
        for (int r = 0; r * 32 < nc; ++r)
        {
            const int col = r * 32 + lane;
            const int wl = (walkerWarp + 2 * r) & (NWARPS - 1), wu = (walkerWarp + 2 * r + 1) & (NWARPS - 1);
            if (col >= nc || (warp != wl && warp != wu))
                continue;
            unsigned cnt = 0;
            const float* vcol = smem + (size_t) col * stride;
            if (warp == wl)
            {
                S.a0[col] = walk_rows<WALK_MIN0>(vcol, M, 0.0f, cnt, 0.0f, false);
            }
            else
            {
                S.a1[col] = walk_rows<WALK_MAX0>(vcol, M, 0.0f, cnt, 0.0f, true);
            }
        }
        return;
    }
    const bool upperLane = (lane & 1) != 0;
    for (int r = 0; r * 16 < nc; ++r)
    {
        if (((walkerWarp + r) & (NWARPS - 1)) != warp)
            continue;
        const int col = r * 16 + (lane >> 1);
        const bool active = col < nc;
        const float* vcol = smem + (size_t) (active ? col : 0) * stride;
        float acc = 0.0f, mean = 0.0f;
        unsigned cnt = 0;
        if (MODE == MODE_ONEBIT_MEAN)
        {
            float sum = 0.0f;
            if (active && !upperLane)
                sum = walk_rows<WALK_SUM>(vcol, M, 0.0f, cnt, 0.0f, false);
            sum = __shfl_sync(0xffffffffu, sum, lane & ~1);
            mean = __fdiv_rn(sum, (float) (unsigned) M);
            if (active)
                acc = walk_rows<WALK_SPLIT_MEAN>(vcol, M, 0.0f, cnt, mean, upperLane);
        }
        const float other = __shfl_xor_sync(0xffffffffu, acc, 1);
        if (active && !upperLane)
        {
            float lo, up;
            finalize_range<MODE>(acc, other, cnt, mean, T.M, lo, up);
            S.lower[col] = lo;
            S.upper[col] = up;
        }
    }
}

// =================================================================================================================
// Phase C: quantize, pack, residual (QuantizeOneQWord, ColumnQuantizer.h:90-147).
// =================================================================================================================
template <int MODE>
__device__ __forceinline__ unsigned quant_one(const ValQ& q, int bits, float val0, float val1, float v, float& res)
{
    if (MODE == MODE_MULTIBIT)
    {
        const unsigned qv = quantize_multibit(q, bits, v);
        res = __fsub_rn(v, unquantize_val(q, bits, qv));
        return qv;
    }
    const bool bit = (MODE == MODE_ONEBIT_ZERO) ? (v >= 0.0f) : (v >= q.qmid);
    res = __fsub_rn(v, bit ? val1 : val0);
    return bit ? 1u : 0u;
}

template <int MODE>
__device__ __forceinline__ void quantize_resident(const QTensor& T, const Signal& sg, int col0, int nc, int stride, const float* __restrict__ smem,
                                                  const ColStats& S)
{
    const int M = (int) T.M;
    const int Q = T.Q;
    const int bits = T.bits;
    const int vpw = 32 / bits;
    const bool vec = ((Q & 3) == 0) && ((M & 3) == 0) && ((reinterpret_cast<uintptr_t>(T.res_out) & 15) == 0);
    if (vec)
    {
        // thread <-> four adjacent words: rows 4*w4 + k*Q .. +3 are one float4 in shared and in global memory
        const int Q4 = Q >> 2;
        const int total = nc * Q4;
        for (int t = threadIdx.x; t < total; t += NT)
        {
            const int col = t / Q4;
            const int w = (t - col * Q4) * 4;
            const int j = col0 + col;
            const float lower = S.lower[col], upper = S.upper[col];
            ValQ q;
            float val0 = 0.0f, val1 = 0.0f;
            if (MODE == MODE_MULTIBIT)
                q = make_valq(bits, lower, upper);
            else
            {
                q.qmid = __fmul_rn(0.5f, __fadd_rn(upper, lower));
                levels_1bit(lower, upper, val0, val1);
            }
            const float* __restrict__ vp = smem + (size_t) col * stride + w;
            float* __restrict__ rp = T.res_out + (size_t) j * M + w;
            const int nk = min(vpw, (M - w + Q - 1) / Q);
            unsigned w0 = 0, w1 = 0, w2 = 0, w3 = 0;
#pragma unroll 4
            for (int k = 0; k < nk; ++k)
            {
                const float4 v = *reinterpret_cast<const float4*>(vp + k * Q);
                float4 r;
                const int sh = k * bits;
                w0 |= quant_one<MODE>(q, bits, val0, val1, v.x, r.x) << sh;
                w1 |= quant_one<MODE>(q, bits, val0, val1, v.y, r.y) << sh;
                w2 |= quant_one<MODE>(q, bits, val0, val1, v.z, r.z) << sh;
                w3 |= quant_one<MODE>(q, bits, val0, val1, v.w, r.w) << sh;
                __stcs(reinterpret_cast<float4*>(rp + k * Q), r);
            }
            const unsigned ws[4] = {w0, w1, w2, w3};
            store_words(T, sg, j, w, ws, 4, lower, upper);
        }
    }
    else
    {
        const int total = nc * Q;
        for (int t = threadIdx.x; t < total; t += NT)
        {
            const int col = t / Q;
            const int w = t - col * Q;
            const int j = col0 + col;
            const float lower = S.lower[col], upper = S.upper[col];
            ValQ q;
            float val0 = 0.0f, val1 = 0.0f;
            if (MODE == MODE_MULTIBIT)
                q = make_valq(bits, lower, upper);
            else
            {
                q.qmid = __fmul_rn(0.5f, __fadd_rn(upper, lower));
                levels_1bit(lower, upper, val0, val1);
            }
            const float* __restrict__ vp = smem + (size_t) col * stride + w;
            float* __restrict__ rp = T.res_out + (size_t) j * M + w;
            const int nk = min(vpw, (M - w + Q - 1) / Q);
            unsigned word = 0;
#pragma unroll 8
            for (int k = 0; k < nk; ++k)
            {
                float r;
                word |= quant_one<MODE>(q, bits, val0, val1, vp[k * Q], r) << (k * bits);
                rp[k * Q] = r;
            }
            store_words(T, sg, j, w, &word, 1, lower, upper);
        }
    }
}

// same, for streamed columns: the values are recomputed from the inputs
template <int MODE, bool STRIPES>
__device__ __forceinline__ void quantize_streamed(const QTensor& T, const Signal& sg, int col0, int nc, const ColStats& S)
{
    const int M = (int) T.M;
    const int Q = T.Q;
    const int bits = T.bits;
    const int vpw = 32 / bits;
    const long long total = (long long) nc * Q;
    for (long long t = threadIdx.x; t < total; t += NT)
    {
        const int col = (int) (t / Q);
        const int w = (int) (t - (long long) col * Q);
        const int j = col0 + col;
        const float lower = S.lower[col], upper = S.upper[col];
        const ValQ q = make_valq(bits, lower, upper);
        const float val0 = unquantize_val(q, 1, 0u), val1 = unquantize_val(q, 1, 1u);
        float* __restrict__ rp = T.res_out + (size_t) j * M + w;
        const int nk = min(vpw, (M - w + Q - 1) / Q);
        unsigned word = 0;
        for (int k = 0; k < nk; ++k)
        {
            float r;
            word |= quant_one<MODE>(q, bits, val0, val1, load_v<STRIPES>(T, j, (long long) w + (long long) k * Q), r) << (k * bits);
            rp[(size_t) k * Q] = r;
        }
        store_words(T, sg, j, w, &word, 1, lower, upper);
    }
}

// =================================================================================================================
// Column quantizer kernel.  One work item = up to CMAX adjacent columns of one matrix.
//   A. all threads stage the columns' fp32 values in shared memory (one coalesced pass over the inputs);
//   B. the columns are walked in row order and each column's range is derived;
//   C. all threads quantize, pack words, write the residual and the packed column to its owner's buffer.
// Several CTAs are resident per SM, so one CTA's walk overlaps the others' memory phases.  Work items are
// handed out through a global counter (tallest columns first) when `counters` is given.
// Columns too tall to stage are streamed through shared memory in chunks for B and re-read for C.
// =================================================================================================================
template <bool STRIPES, int MODE, bool TABLE>
#ifndef QAGG_CTAS_PER_SM
#define QAGG_CTAS_PER_SM 3 // resident CTAs per SM the column kernel is compiled and configured for
#endif
__global__ void __launch_bounds__(NT, QAGG_CTAS_PER_SM) k_colquant(const QTensor single, const QTensor* __restrict__ tensors,
                                                    const QItem* __restrict__ items, int nItems, int colsPerItem, int smemFloats,
                                                    int numSMs, unsigned* __restrict__ counters, const Signal signal)
{
    extern __shared__ __align__(16) float smem[];
    __shared__ QTensor sT;
    __shared__ int sIt;
    __shared__ int sWalker;

    // which warp walks: a per-SM ticket when a counter block is given (counters[8 + smid]; it only ever grows and is
    // used modulo the warp count), else a guess from the block index (CTAs are dealt to the SMs round-robin)
    if (threadIdx.x == 0)
    {
        unsigned ticket;
        if (counters)
        {
            unsigned smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            ticket = atomicAdd(&counters[8 + (smid & 255u)], 1u);
        }
        else
        {
            ticket = blockIdx.x / (unsigned) max(numSMs, 1);
        }
        sWalker = (int) (ticket & 3u);
    }
    __syncthreads();
    const int walkerWarp = sWalker;

    for (int iter = 0;; ++iter)
    {
        __syncthreads(); // previous item fully done with sT / smem / sIt
        if (threadIdx.x == 0)
            sIt = counters ? (int) atomicAdd(&counters[0], 1u) : (int) (blockIdx.x + (unsigned) iter * gridDim.x);
        __syncthreads();
        const int it = sIt;
        if (it >= nItems)
            break;
        int col0, nc;
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
        const QTensor* gT = TABLE ? (tensors + items[it].tensor) : &single;
        const int strideGuess = smem_stride(gT->M);
        // floats of shared memory per column: staged values + per-column scratch (+ the K packed source columns)
        const int extraPerCol = STRIPES ? gT->nsrc * (gT->colBytes >> 2) : 0;
        const bool resident = ((long long) nc * (strideGuess + COLSTAT_FLOATS) <= (long long) smemFloats);
        // the K packed source columns are staged in shared memory too when that fits next to the values; else the reduce
        // kernel reads them from global memory
        const bool stagePacked = STRIPES && ((long long) nc * (strideGuess + COLSTAT_FLOATS + extraPerCol) <= (long long) smemFloats);
        // per-column scratch sits behind the staged values (resident) or behind the chunk ring (streamed)
        ColStats S;
        {
            float* tail = smem + (resident ? (size_t) nc * strideGuess : (size_t) smemFloats - COLSTAT_FLOATS * (size_t) nc);
            S.lower = tail;
            S.upper = tail + nc;
            S.n0 = reinterpret_cast<unsigned*>(tail + 2 * nc);
            S.nan = reinterpret_cast<unsigned*>(tail + 3 * nc);
            S.a0 = tail + 4 * nc;
            S.a1 = tail + 5 * nc;
        }
        for (int i = threadIdx.x; i < nc; i += NT)
        {
            S.n0[i] = 0;
            S.nan[i] = 0;
        }
        __syncthreads();
        const QTensor& T = sT;
        const int stride = strideGuess;

        if (resident)
        {
            if (STRIPES)
                fill_stripes<MODE>(T, col0, nc, stride, smem, S,
                                   stagePacked ? reinterpret_cast<unsigned*>(smem + (size_t) nc * (stride + COLSTAT_FLOATS)) : nullptr);
            else
                fill_dense<MODE>(T, col0, nc, stride, smem, S);
            __syncthreads();
            walk_resident<MODE>(T, nc, stride, smem, S, walkerWarp);
            __syncthreads();
            if (MODE == MODE_ONEBIT_ZERO)
            {
                for (int col = threadIdx.x; col < nc; col += NT)
                {
                    float lo, up;
                    finalize_range<MODE>(S.a0[col], S.nan[col] ? __int_as_float(0x7fc00000) : S.a1[col], S.n0[col], 0.0f, T.M, lo, up);
                    S.lower[col] = lo;
                    S.upper[col] = up;
                }
                __syncthreads();
            }
            quantize_resident<MODE>(T, signal, col0, nc, stride, smem, S);
        }
        else
        {
            // chunked: rows [r0, r0+cs) of the nc columns at a time, one lane per column, both sums in one lane
            const long long M = T.M;
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            const int cs = (((smemFloats - COLSTAT_FLOATS * nc) / nc - 4) / 32) * 32 + 4;
            float a0 = 0.0f, a1 = 0.0f, am = 0.0f, mean = 0.0f;
            unsigned n0 = 0, dummy = 0;
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
                        const float* vcol = smem + (size_t) lane * cs;
                        if (meanPass)
                            am = walk_rows<WALK_SUM>(vcol, nr, am, dummy, 0.0f, false);
                        else if (MODE == MODE_MULTIBIT)
                            a0 = walk_rows<WALK_SQUARES>(vcol, nr, a0, dummy, 0.0f, false);
                        else
                        {
                            a0 = walk_rows<WALK_SPLIT_MEAN>(vcol, nr, a0, n0, mean, false);
                            a1 = walk_rows<WALK_SPLIT_MEAN>(vcol, nr, a1, dummy, mean, true);
                        }
                    }
                    __syncthreads();
                }
                if (meanPass)
                    mean = __fdiv_rn(am, (float) (unsigned long long) M);
            }
            if (warp == 0 && lane < nc)
            {
                float lo, up;
                finalize_range<MODE>(a0, a1, n0, mean, M, lo, up);
                S.lower[lane] = lo;
                S.upper[lane] = up;
            }
            __syncthreads();
            quantize_streamed<MODE, STRIPES>(T, signal, col0, nc, S);
        }
    }
    // The last CTA to leave re-arms the work counter for the next launch and, if asked to, tells the peers that every
    // store of this kernel (theirs included: packed columns written straight into peer memory) has been issued:
    // each CTA's stores are ordered before its arrival by barrier + system-scope fence, the last arrival observes all
    // of them and releases the flags.
    if (counters && threadIdx.x == 0)
    {
        __threadfence_system();
        const unsigned done = atomicAdd(&counters[1], 1u);
        if (done == gridDim.x - 1)
        {
            counters[0] = 0;
            counters[1] = 0;
            release_flags(signal);
        }
    }
}

// One warp waits for the peers' flags.  Every wait is bounded: after maxPolls polls the lane gives up, records it in
// *status and the kernel ends normally.
__global__ void k_wait_flags(const unsigned* __restrict__ flags, int n, int skip, unsigned value, long long maxPolls, unsigned* __restrict__ status,
                             const HeaderPtrs hdrSrc, int hdrN, double* __restrict__ hdrOut)
{
    const int i = threadIdx.x;
    if (i < n && i != skip)
    {
        long long polls = 0;
        for (;;)
        {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
            if ((int) (v - value) >= 0)
                break;
            if (++polls >= maxPolls)
            {
                atomicOr(status, 1u);
                break;
            }
            __nanosleep(64);
        }
    }
    __threadfence_system();
    __syncwarp();
    // the header values every rank stored before it released its flag: summed in rank order (a wait that gave up sums
    // whatever is there; the status word says so)
    for (int j = i; j < hdrN; j += 32)
    {
        double s = *reinterpret_cast<const volatile double*>(hdrSrc.p[0] + j);
        for (int p = 1; p < hdrSrc.n; ++p)
            s += *reinterpret_cast<const volatile double*>(hdrSrc.p[p] + j);
        hdrOut[j] = s;
    }
}

// ---- host side ------------------------------------------------------------------------------------------------

int cols_per_item(long long M, long long N, int smemFloats, bool* resident, int extraFloatsPerCol)
{
    const int stride = smem_stride(M);
    long long c = smemFloats / (stride + COLSTAT_FLOATS + extraFloatsPerCol);
    bool res = true;
    if (c < 1)
    {
        res = false;
        c = 8; // streamed in row chunks
    }
    if (c > CMAX)
        c = CMAX;
    if (!res && c > 32)
        c = 32;
    if (c > N)
        c = N;
    if (c < 1)
        c = 1;
    if (resident)
        *resident = res;
    return (int) c;
}

template <bool STRIPES, int MODE, bool TABLE>
static cudaError_t launch_cq(cudaStream_t st, const QTensor* single, const QTensor* tensors, const QItem* items,
                             int nItems, int colsPerItem, const LaunchCfg& cfg, unsigned* counters, const Signal& signal)
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
    kern<<<grid, NT, smemBytes, st>>>(single ? *single : zero, tensors, items, nItems, colsPerItem, cfg.smemFloats, cfg.numSMs, counters, signal);
    return cudaGetLastError();
}

__global__ void k_signal_only(const Signal signal)
{
    release_flags(signal);
}

cudaError_t launch_signal_only(cudaStream_t st, const Signal& signal)
{
    k_signal_only<<<1, 1, 0, st>>>(signal);
    return cudaGetLastError();
}

// Broadcast of a finished region: every CTA copies 16-byte words from local memory into the same offset of each
// destination (peer gather slots), then the last CTA releases the flags (same hand-shake as at the end of k_colquant).
__global__ void __launch_bounds__(256) k_push(const uint4* __restrict__ src, size_t n16, const Signal signal, unsigned* __restrict__ counters)
{
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t) gridDim.x * blockDim.x)
    {
        const uint4 v = __ldg(src + i);
        for (int b = 0; b < signal.nbcast; ++b)
            reinterpret_cast<uint4*>(signal.bcastBase[b])[i] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0)
    {
        __threadfence_system();
        const unsigned done = atomicAdd(&counters[1], 1u);
        if (done == gridDim.x - 1)
        {
            counters[1] = 0;
            release_flags(signal);
        }
    }
}

cudaError_t launch_push(cudaStream_t st, const void* src, size_t bytes, const Signal& signal, unsigned* counters, int numSMs)
{
    const size_t n16 = (bytes + 15) / 16;
    int grid = (int) ((n16 + 255) / 256);
    if (grid > numSMs)
        grid = numSMs;
    if (grid < 1)
        grid = 1;
    k_push<<<grid, 256, 0, st>>>(static_cast<const uint4*>(src), n16, signal, counters);
    return cudaGetLastError();
}

// Header exchange (the DistGradHeader / loss scalars of a step): every rank stores its n doubles into slot `rank` of every
// rank's header area, then -- after the step's first flag wait -- sums the K slots in rank order, the same order everywhere.
__global__ void k_header_push(const double* __restrict__ in, int n, const HeaderPtrs dst)
{
    const int i = threadIdx.x;
    if (i < n)
    {
        const double v = in[i];
        for (int p = 0; p < dst.n; ++p)
            dst.p[p][i] = v;
    }
}

__global__ void k_header_sum(const HeaderPtrs src, int n, double* __restrict__ out)
{
    const int i = threadIdx.x;
    if (i < n)
    {
        double s = *reinterpret_cast<const volatile double*>(src.p[0] + i);
        for (int p = 1; p < src.n; ++p)
            s += *reinterpret_cast<const volatile double*>(src.p[p] + i);
        out[i] = s;
    }
}

cudaError_t launch_header_push(cudaStream_t st, const double* in, int n, const HeaderPtrs& dst)
{
    if (n <= 0 || dst.n <= 0)
        return cudaSuccess;
    k_header_push<<<1, QAGG_HEADER_MAX, 0, st>>>(in, n, dst);
    return cudaGetLastError();
}

cudaError_t launch_header_sum(cudaStream_t st, const HeaderPtrs& src, int n, double* out)
{
    if (n <= 0 || src.n <= 0)
        return cudaSuccess;
    k_header_sum<<<1, QAGG_HEADER_MAX, 0, st>>>(src, n, out);
    return cudaGetLastError();
}

cudaError_t launch_wait_flags(cudaStream_t st, const unsigned* flags, int n, int skip, unsigned value, long long maxPolls, unsigned* status,
                              const HeaderPtrs* hdrSrc, int hdrN, double* hdrOut)
{
    if (n > 32)
        return cudaErrorInvalidValue;
    static const HeaderPtrs none = {};
    const bool sum = hdrSrc && hdrN > 0 && hdrOut;
    k_wait_flags<<<1, 32, 0, st>>>(flags, n, skip, value, maxPolls, status, sum ? *hdrSrc : none, sum ? hdrN : 0, hdrOut);
    return cudaGetLastError();
}

cudaError_t launch_colquant(cudaStream_t st, bool stripes, int mode, const QTensor* single, const QTensor* tensors,
                            const QItem* items, int nItems, int colsPerItem, const LaunchCfg& cfg, unsigned* counters, const Signal* signalp)
{
    static const Signal none = {};
    const Signal& signal = signalp ? *signalp : none;
    if (nItems <= 0)
    {
        // nothing to compute, but the peers still wait for this rank's flags
        if (signal.n > 0)
        {
            k_signal_only<<<1, 1, 0, st>>>(signal);
            return cudaGetLastError();
        }
        return cudaSuccess;
    }
    const bool table = (single == nullptr);
#define QAGG_CASE(S, MD, TB) \
    if (stripes == S && mode == MD && table == TB) \
        return launch_cq<S, MD, TB>(st, single, tensors, items, nItems, colsPerItem, cfg, counters, signal);
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

cudaError_t get_launch_cfg(int device, LaunchCfg* cfg)
{
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess)
        return e;
    cfg->numSMs = prop.multiProcessorCount;
    // three CTAs per SM: a third of the SM's shared memory minus the 1 KB the system reserves per CTA and
    // 1 KB for the kernel's static shared memory
    cfg->ctasPerSM = QAGG_CTAS_PER_SM;
    size_t perCta = prop.sharedMemPerMultiprocessor / cfg->ctasPerSM - 1024 - 1024;
    if (perCta > prop.sharedMemPerBlockOptin - 1024)
        perCta = prop.sharedMemPerBlockOptin - 1024;
    perCta &= ~(size_t) 15;
    cfg->smemFloats = (int) (perCta / sizeof(float));
    return cudaSuccess;
}

} // namespace qagg
