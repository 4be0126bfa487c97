// qagg_unquantize.cu -- the unquantize kernel (UnquantizeOneQWord / Unquantize, Source/Math/ColumnQuantizer.h:69-77, 150-203).
//
// Pure expand-and-store: a packed column of Q words becomes M floats, 32/bits times as many bytes, so the kernel is bound
// by the write bandwidth of HBM and everything is arranged around the stores.
//   * Word-major mapping, as the layout suggests: word w of a column holds rows w, w + Q, w + 2Q, ...  A lane fetches FOUR
//     ADJACENT WORDS once and, per field position k, stores the four rows 4w' + kQ .. + 3 as one aligned 16-byte vector
//     (possible when M and Q are multiples of 4 and the output is 16-byte aligned).  Otherwise a lane takes four words
//     32 apart and the warp stores 32 consecutive rows per position with 4-byte stores.
//   * Work unit = 128 consecutive words of a matrix (columns laid end to end), all field positions = one warp; 16 KB of
//     output in the 1-bit case, every store independent of every other.  One unit per warp, eight warps per CTA: no shared
//     memory (in this form), no barrier, no atomics; the hardware scheduler keeps the SMs full.
//   * Units are numbered matrix after matrix, the field-position blocks of one word group next to each other:
//     neighbouring warps write neighbouring memory.
//   * Columns whose word count Q is not a multiple of 4 (a 9304-row column has Q = 291) cannot take the vector form above:
//     rows w + kQ are then not 16-byte aligned for every k.  They are expanded ROW-MAJOR instead: a warp copies the column's
//     Q packed words into its slice of shared memory (a padded layout, so that lanes reading words four apart hit distinct
//     banks), and every lane produces four CONSECUTIVE rows -- row i is field i / Q of word i % Q -- as one aligned 16-byte
//     store.  Work unit there = 2048 consecutive rows of one column.  With 4-byte stores this shape ran at 2.7 TB/s.
//   * What happens to an expanded value is the kernel's MODE: stored (UNQ_STORE), added to what the destination holds
//     (UNQ_ADD), or consumed on the spot by the momentum-SGD update that follows aggregation in the training loop
//     (UNQ_UPDATE: the smoothed gradient and the parameter are read, updated and written; the aggregated gradient itself
//     never goes to memory, which saves its write here and its read in a separate update kernel).
#include "qagg_device.cuh"

#include <algorithm>

namespace qagg {

constexpr int UNQ_WORDS = 128; // packed words per unit
constexpr int UNQ_KPU = 32;    // field positions per unit: all of them (the unit table still allows a split by position blocks)

// field-position blocks per word: 4 for 1 bit, 2 for 2 bits, else 1 (always a power of two)
__host__ __device__ __forceinline__ int unq_ksplit(int bits)
{
    const int vpw = 32 / bits;
    return (vpw + UNQ_KPU - 1) / UNQ_KPU;
}

constexpr int UNQ_RM_ROWS = 2048; // row-major form: rows per unit (32 lanes x 16 vectors x 4 rows)
constexpr int UNQ_RM_QMAX = 2048;  // row-major form: most packed words of a column (64 K rows at 1 bit)

// which shapes take the row-major form (decided by the shape alone, so that host and device agree on the unit count)
__host__ __device__ __forceinline__ bool unq_row_major(long long M, long long Q)
{
    return (M & 3) == 0 && (Q & 3) != 0 && Q <= UNQ_RM_QMAX;
}
// shared-memory words a warp needs to hold Q packed words in the padded layout
__host__ __device__ __forceinline__ int unq_rm_words(long long Q)
{
    return (int) (Q + (Q >> 5) + 1);
}

long long unq_units(long long M, long long N, int bits)
{
    if (M <= 0 || N <= 0)
        return 0;
    const long long Q = (M * bits + 31) / 32;
    if (unq_row_major(M, Q))
        return N * ((M + UNQ_RM_ROWS - 1) / UNQ_RM_ROWS);
    return ((N * Q + UNQ_WORDS - 1) / UNQ_WORDS) * unq_ksplit(bits);
}

int unq_smem_words(long long M, int bits)
{
    const long long Q = (M * bits + 31) / 32;
    return (M > 0 && unq_row_major(M, Q)) ? unq_rm_words(Q) : 0;
}

// the two constants unquantizing needs: 1 bit -> the two level values; else -> (ufactor, quantimin)
__device__ __forceinline__ void unq_consts(int bits, float lower, float upper, float& ca, float& cb)
{
    if (bits == 1)
    {
        levels_1bit(lower, upper, ca, cb);
    }
    else
    {
        const ValQ q = make_valq(bits, lower, upper);
        ca = q.ufactor;
        cb = q.qmin;
    }
}

template <bool ONEBIT>
__device__ __forceinline__ float unq_field(int bits, unsigned word, unsigned k, unsigned mask, float ca, float cb)
{
    if (ONEBIT)
        return ((word >> k) & 1u) ? cb : ca;
    if (bits == 32)
        return __uint_as_float(word);
    const unsigned field = (word >> (k * (unsigned) bits)) & mask;
    return __fadd_rn(__fmul_rn(__fadd_rn((float) field, 0.5f), ca), cb);
}

// ---- what a lane does with expanded values ----------------------------------------------------------------------------
// four consecutive rows at p (16-byte aligned); sp = the same rows of the smoothed gradient (UNQ_UPDATE only)
template <int MODE>
__device__ __forceinline__ void unq_emit4(float4* p, float4* sp, float4 v, const UpdateRule& rule)
{
    if (MODE == UNQ_STORE)
    {
        __stcs(p, v);
    }
    else if (MODE == UNQ_ADD)
    {
        const float4 o = *p;
        v.x = __fadd_rn(v.x, o.x);
        v.y = __fadd_rn(v.y, o.y);
        v.z = __fadd_rn(v.z, o.z);
        v.w = __fadd_rn(v.w, o.w);
        *p = v;
    }
    else
    {
        float4 s = __ldcs(sp);
        float4 w = __ldcs(p);
        w.x = sgd_apply(rule, v.x, s.x, w.x);
        w.y = sgd_apply(rule, v.y, s.y, w.y);
        w.z = sgd_apply(rule, v.z, s.z, w.z);
        w.w = sgd_apply(rule, v.w, s.w, w.w);
        __stcs(sp, s);
        __stcs(p, w);
    }
}
template <int MODE>
__device__ __forceinline__ void unq_emit1(float* p, float* sp, float v, const UpdateRule& rule)
{
    if (MODE == UNQ_STORE)
    {
        *p = v;
    }
    else if (MODE == UNQ_ADD)
    {
        *p = __fadd_rn(v, *p);
    }
    else
    {
        float s = *sp;
        *p = sgd_apply(rule, v, s, *p);
        *sp = s;
    }
}

template <int MODE, bool TABLE, bool ONEBIT>
__global__ void __launch_bounds__(NT, 4) k_unquantize(const QTensor single, const QTensor* __restrict__ tensors, int nTensors, long long totalUnits,
                                                   int smemWords, const UpdateRule rule)
{
    extern __shared__ unsigned sWords[]; // row-major form: smemWords words per warp
    const unsigned lane = threadIdx.x & 31;
    unsigned* const sw = sWords + (size_t) (threadIdx.x >> 5) * (size_t) smemWords;
    const long long gwarp = (long long) blockIdx.x * NWARPS + (threadIdx.x >> 5);
    const long long nwarps = (long long) gridDim.x * NWARPS;
    int cur = 0; // table entry of the previous unit: consecutive units of a warp mostly stay within one matrix
    for (long long u = gwarp; u < totalUnits; u += nwarps)
    {
        const QTensor* Tp = &single;
        if (TABLE)
        {
            // last table entry whose first unit is <= u (entries without units share their successor's first unit)
            if (!(tensors[cur].unit0 <= u && (cur + 1 >= nTensors || u < tensors[cur + 1].unit0)))
            {
                int lo = 0, hi = nTensors;
                while (hi - lo > 1)
                {
                    const int mid = (lo + hi) >> 1;
                    if (tensors[mid].unit0 <= u)
                        lo = mid;
                    else
                        hi = mid;
                }
                cur = lo;
            }
            Tp = tensors + cur;
        }
        const unsigned M = (unsigned) Tp->M;
        const unsigned Q = (unsigned) Tp->Q;
        const int bits = ONEBIT ? 1 : Tp->bits;
        const unsigned vpw = 32u / (unsigned) bits;
        const unsigned mask = (bits >= 32) ? 0xffffffffu : ((1u << bits) - 1u);
        if (unq_row_major(M, Q))
        {
            // ---- row-major form: unit = rows [r0, r0 + 1024) of one column ----
            const unsigned blocksPerCol = (M + UNQ_RM_ROWS - 1) / UNQ_RM_ROWS;
            const unsigned long long localU = (unsigned long long) (u - (TABLE ? Tp->unit0 : 0));
            const unsigned c = (unsigned) (localU / blocksPerCol);
            const unsigned r0 = (unsigned) (localU - (unsigned long long) c * blocksPerCol) * UNQ_RM_ROWS;
            const unsigned char* colp = TABLE ? packed_col(*Tp, (int) c) : single.pk[0] + (size_t) c * (size_t) single.colBytes;
            const unsigned* __restrict__ words = reinterpret_cast<const unsigned*>(colp + 8);
            __syncwarp(); // the previous unit's reads of the staging slice are done
            for (unsigned w = lane; w < Q; w += 32)
                sw[w + (w >> 5)] = __ldg(words + w);
            float ca, cb;
            unq_consts(bits, __ldg(reinterpret_cast<const float*>(colp)), __ldg(reinterpret_cast<const float*>(colp) + 1), ca, cb);
            __syncwarp();
            float* __restrict__ out = Tp->out + (size_t) c * M;
            const bool aligned = (reinterpret_cast<uintptr_t>(Tp->out) & 15) == 0 &&
                                 (MODE != UNQ_UPDATE || (reinterpret_cast<uintptr_t>(Tp->res_out) & 15) == 0);
            unsigned r = r0 + 4u * lane;
            unsigned k = r / Q, w = r - k * Q;
            const unsigned advK = 128u / Q, advW = 128u - advK * Q;
#pragma unroll 4
            for (int t = 0; t < UNQ_RM_ROWS / 128; ++t)
            {
                if (r < M)
                {
                    float v[4];
#pragma unroll
                    for (unsigned e = 0; e < 4; ++e)
                    {
                        unsigned ww = w + e, kk = k;
                        while (ww >= Q) // the four rows straddle the end of the word array (more than once when Q < 4)
                        {
                            ww -= Q;
                            ++kk;
                        }
                        v[e] = unq_field<ONEBIT>(bits, sw[ww + (ww >> 5)], kk, mask, ca, cb);
                    }
                    float* p = out + r;
                    float* sp = (MODE == UNQ_UPDATE) ? Tp->res_out + (size_t) c * M + r : nullptr;
                    if (aligned)
                    {
                        unq_emit4<MODE>(reinterpret_cast<float4*>(p), reinterpret_cast<float4*>(sp), make_float4(v[0], v[1], v[2], v[3]), rule);
                    }
                    else
                    {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            unq_emit1<MODE>(p + e, sp + e, v[e], rule);
                    }
                }
                r += 128u;
                w += advW;
                k += advK;
                if (w >= Q)
                {
                    w -= Q;
                    ++k;
                }
            }
            continue;
        }
        const int ks = unq_ksplit(bits);
        const int ksShift = (ks == 4) ? 2 : (ks == 2) ? 1 : 0;
        const unsigned long long local = (unsigned long long) (u - (TABLE ? Tp->unit0 : 0));
        const unsigned k0 = (unsigned) (local & (unsigned long long) (ks - 1)) * UNQ_KPU;
        const unsigned long long t0 = (local >> ksShift) * UNQ_WORDS; // first word of the unit, columns laid end to end
        const unsigned long long totalWords = (unsigned long long) Tp->N * Q;
        // column and word of the unit's first word: a 32-bit division when the matrix is small enough for that
        unsigned col0, w0;
        if (totalWords <= 0xffffffffull)
        {
            col0 = (unsigned) t0 / Q;
            w0 = (unsigned) t0 - col0 * Q;
        }
        else
        {
            col0 = (unsigned) (t0 / Q);
            w0 = (unsigned) (t0 - (unsigned long long) col0 * Q);
        }
        const unsigned left = (unsigned) ((totalWords - t0 < UNQ_WORDS) ? (totalWords - t0) : UNQ_WORDS); // words of this unit
        float* __restrict__ outBase = Tp->out;
        const bool vec = ((M & 3u) == 0) && ((Q & 3u) == 0) && ((reinterpret_cast<uintptr_t>(outBase) & 15) == 0) &&
                         (MODE != UNQ_UPDATE || (reinterpret_cast<uintptr_t>(Tp->res_out) & 15) == 0);
        if (vec)
        {
            // lane <-> words 4 * lane .. + 3 of the unit: the same column (Q is a multiple of 4), rows 4-aligned
            const unsigned off = 4u * lane;
            if (off < left)
            {
                const unsigned tl = w0 + off;
                const unsigned dc = tl / Q;
                const unsigned c = col0 + dc, w = tl - dc * Q;
                const unsigned char* colp = TABLE ? packed_col(*Tp, (int) c) : single.pk[0] + (size_t) c * (size_t) single.colBytes;
                const float lower = __ldg(reinterpret_cast<const float*>(colp));
                const float upper = __ldg(reinterpret_cast<const float*>(colp) + 1);
                const unsigned* __restrict__ words = reinterpret_cast<const unsigned*>(colp + 8) + w;
                const unsigned wa = __ldg(words), wb = __ldg(words + 1), wc = __ldg(words + 2), wd = __ldg(words + 3);
                float ca, cb;
                unq_consts(bits, lower, upper, ca, cb);
                float* __restrict__ op = outBase + (size_t) c * M + w;
                float* __restrict__ sp = (MODE == UNQ_UPDATE) ? Tp->res_out + (size_t) c * M + w : nullptr;
#pragma unroll
                for (unsigned kk = 0; kk < UNQ_KPU; ++kk)
                {
                    const unsigned k = k0 + kk;
                    if (k < vpw && w + k * Q < M)
                    {
                        float4 v;
                        v.x = unq_field<ONEBIT>(bits, wa, k, mask, ca, cb);
                        v.y = unq_field<ONEBIT>(bits, wb, k, mask, ca, cb);
                        v.z = unq_field<ONEBIT>(bits, wc, k, mask, ca, cb);
                        v.w = unq_field<ONEBIT>(bits, wd, k, mask, ca, cb);
                        unq_emit4<MODE>(reinterpret_cast<float4*>(op + (size_t) k * Q), reinterpret_cast<float4*>(sp + (size_t) k * Q), v, rule);
                    }
                }
            }
        }
        else
        {
            // lane <-> words lane, lane + 32, lane + 64, lane + 96 of the unit: per position the warp stores 32 consecutive rows
            unsigned wd[4], cc[4], ww[4];
            float lo[4], up[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
            {
                const unsigned off = lane + 32u * e;
                wd[e] = 0u;
                cc[e] = ww[e] = 0u;
                lo[e] = up[e] = 0.0f;
                if (off < left)
                {
                    const unsigned tl = w0 + off;
                    const unsigned dc = tl / Q;
                    cc[e] = col0 + dc;
                    ww[e] = tl - dc * Q;
                    const unsigned char* colp = TABLE ? packed_col(*Tp, (int) cc[e]) : single.pk[0] + (size_t) cc[e] * (size_t) single.colBytes;
                    lo[e] = __ldg(reinterpret_cast<const float*>(colp));
                    up[e] = __ldg(reinterpret_cast<const float*>(colp) + 1);
                    wd[e] = __ldg(reinterpret_cast<const unsigned*>(colp + 8) + ww[e]);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e)
            {
                if (lane + 32u * e < left)
                {
                    float ca, cb;
                    unq_consts(bits, lo[e], up[e], ca, cb);
                    float* __restrict__ op = outBase + (size_t) cc[e] * M + ww[e];
                    float* __restrict__ sp = (MODE == UNQ_UPDATE) ? Tp->res_out + (size_t) cc[e] * M + ww[e] : nullptr;
#pragma unroll
                    for (unsigned kk = 0; kk < UNQ_KPU; ++kk)
                    {
                        const unsigned k = k0 + kk;
                        if (k < vpw && ww[e] + k * Q < M)
                            unq_emit1<MODE>(op + (size_t) k * Q, sp + (size_t) k * Q, unq_field<ONEBIT>(bits, wd[e], k, mask, ca, cb), rule);
                    }
                }
            }
        }
    }
}

// Grid: one unit per warp, eight per CTA.  The hardware's CTA scheduler backfills the SMs as CTAs finish; a persistent grid
// whose warps loop over units measured 10 to 15 % slower here (each warp's unit starts with a chain of dependent loads --
// table entry, column header, words -- that a fresh CTA's eight warps issue all at once).
static int unq_grid(long long totalUnits, int /*numSMs*/)
{
    const long long need = (totalUnits + NWARPS - 1) / NWARPS;
    return (int) std::min<long long>(need, 0x7fffffff);
}

cudaError_t launch_unquantize(cudaStream_t st, int mode, int bits, const QTensor* single, const QTensor* tensors, int nTensors, long long totalUnits,
                              int smemWordsPerWarp, const LaunchCfg& cfg, const UpdateRule* rule)
{
    if (totalUnits <= 0)
        return cudaSuccess;
    if (mode == UNQ_UPDATE && !rule)
        return cudaErrorInvalidValue;
    const size_t smemBytes = (size_t) smemWordsPerWarp * NWARPS * sizeof(unsigned); // at most 8 x 2113 words = 66 KB
    const int grid = unq_grid(totalUnits, cfg.numSMs);
    static const QTensor zero = {};
    const QTensor& s = single ? *single : zero;
    const bool table = (single == nullptr);
    const bool onebit = (bits == 1);
    const UpdateRule r = rule ? *rule : UpdateRule{};
#define QAGG_UNQ_CASE(A, T, O)                                                                                                         \
    if (mode == A && table == T && onebit == O)                                                                                        \
    {                                                                                                                                  \
        if (smemBytes > 48 * 1024)                                                                                                     \
        {                                                                                                                              \
            const cudaError_t e = cudaFuncSetAttribute(k_unquantize<A, T, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smemBytes); \
            if (e != cudaSuccess)                                                                                                      \
                return e;                                                                                                              \
        }                                                                                                                              \
        k_unquantize<A, T, O><<<grid, NT, smemBytes, st>>>(s, tensors, nTensors, totalUnits, smemWordsPerWarp, r);                      \
    }
    QAGG_UNQ_CASE(UNQ_STORE, false, false)
    QAGG_UNQ_CASE(UNQ_STORE, false, true)
    QAGG_UNQ_CASE(UNQ_STORE, true, false)
    QAGG_UNQ_CASE(UNQ_STORE, true, true)
    QAGG_UNQ_CASE(UNQ_ADD, false, false)
    QAGG_UNQ_CASE(UNQ_ADD, false, true)
    QAGG_UNQ_CASE(UNQ_ADD, true, false)
    QAGG_UNQ_CASE(UNQ_ADD, true, true)
    QAGG_UNQ_CASE(UNQ_UPDATE, false, false)
    QAGG_UNQ_CASE(UNQ_UPDATE, false, true)
    QAGG_UNQ_CASE(UNQ_UPDATE, true, false)
    QAGG_UNQ_CASE(UNQ_UPDATE, true, true)
#undef QAGG_UNQ_CASE
    return cudaGetLastError();
}

} // namespace qagg
