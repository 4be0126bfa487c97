// qagg_unquantize.cu -- the unquantize kernel (UnquantizeOneQWord / Unquantize, Source/Math/ColumnQuantizer.h:69-77, 150-203).
//
// Pure expand-and-store: a packed column of Q words becomes M floats, 32/bits times as many bytes, so the kernel is bound
// by the write bandwidth of HBM and everything is arranged around the stores.
//   * Output-major mapping.  Row i of a column is field i / Q of word i % Q.  A lane produces FOUR CONSECUTIVE ROWS and
//     stores them as one aligned 16-byte vector, whatever Q is (the word-major mapping of the reference kernel, thread <->
//     word, yields vector stores only when Q is a multiple of 4; a 9304-row column has Q = 291).  The four fields come
//     from (usually) four adjacent words, re-read from the L1 cache for every field position.
//   * Work unit = 512 consecutive rows of one column = one warp, four vectors per lane, all of a unit's words fetched before
//     the first store.  Warps take units u, u + (warps in the grid), ...: no shared memory, no barrier, no atomics.  A launch
//     has thousands of units per SM-resident warp set, so the grid (4 CTAs per SM) ends evenly; a launch with one CTA per
//     group of columns did not (its last partial wave of CTAs ran on a mostly idle GPU).
//   * Units are numbered matrix after matrix, column after column: consecutive warps write consecutive memory.
// Matrices whose rows are not a multiple of 4 (or whose output is not 16-byte aligned) take a scalar form of the same loop.
#include "qagg_device.cuh"

namespace qagg {

constexpr int UNQ_ROWS = 512; // rows per unit: 32 lanes x 4 vectors x 4 rows
constexpr int UNQ_VEC = 4;    // vectors per lane and unit

long long unq_units(long long M, long long N)
{
    if (M <= 0 || N <= 0)
        return 0;
    return N * ((M + UNQ_ROWS - 1) / UNQ_ROWS);
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

__device__ __forceinline__ float unq_field(int bits, unsigned word, unsigned k, unsigned mask, float ca, float cb)
{
    if (bits == 1)
        return ((word >> k) & 1u) ? cb : ca;
    if (bits == 32)
        return __uint_as_float(word);
    const unsigned field = (word >> (k * (unsigned) bits)) & mask;
    return __fadd_rn(__fmul_rn(__fadd_rn((float) field, 0.5f), ca), cb);
}

template <bool ADD, bool TABLE>
__global__ void __launch_bounds__(NT, 4) k_unquantize(const QTensor single, const QTensor* __restrict__ tensors, int nTensors, long long totalUnits)
{
    const int lane = threadIdx.x & 31;
    const long long gwarp = (long long) blockIdx.x * NWARPS + (threadIdx.x >> 5);
    const long long nwarps = (long long) gridDim.x * NWARPS;
    int cur = 0; // table entry of the previous unit: units of one warp mostly stay within one matrix
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
        const int bits = Tp->bits;
        const unsigned mask = (bits >= 32) ? 0xffffffffu : ((1u << bits) - 1u);
        const unsigned blocksPerCol = (M + UNQ_ROWS - 1) / UNQ_ROWS;
        const unsigned long long local = (unsigned long long) (u - (TABLE ? Tp->unit0 : 0));
        const unsigned col = (unsigned) (local / blocksPerCol);
        const unsigned row0 = (unsigned) (local - (unsigned long long) col * blocksPerCol) * UNQ_ROWS;
        const unsigned char* colp = TABLE ? packed_col(*Tp, (int) col) : single.pk[0] + (size_t) col * (size_t) single.colBytes;
        const float lower = __ldg(reinterpret_cast<const float*>(colp));
        const float upper = __ldg(reinterpret_cast<const float*>(colp) + 1);
        const unsigned* __restrict__ words = reinterpret_cast<const unsigned*>(colp + 8);
        float ca, cb;
        unq_consts(bits, lower, upper, ca, cb);
        float* __restrict__ out = Tp->out + (size_t) col * M;
        const bool vec = ((M & 3u) == 0) && ((reinterpret_cast<uintptr_t>(Tp->out) & 15) == 0);
        if (vec)
        {
            // lane <-> rows row0 + 4 * lane + 128 * i .. + 3
            const unsigned r0 = row0 + 4u * lane;
            unsigned k = r0 / Q, w = r0 - k * Q;
            const unsigned advK = 128u / Q, advW = 128u - advK * Q;
            unsigned wd[UNQ_VEC][4], kk[UNQ_VEC][4];
#pragma unroll
            for (int i = 0; i < UNQ_VEC; ++i)
            {
                const bool live = r0 + 128u * i < M;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                {
                    unsigned ww = w + e, ke = k;
                    while (ww >= Q) // the four rows straddle the end of the word array (several times over when Q < 4)
                    {
                        ww -= Q;
                        ++ke;
                    }
                    kk[i][e] = ke;
                    wd[i][e] = live ? __ldg(words + ww) : 0u;
                }
                w += advW;
                k += advK;
                if (w >= Q)
                {
                    w -= Q;
                    ++k;
                }
            }
#pragma unroll
            for (int i = 0; i < UNQ_VEC; ++i)
            {
                const unsigned r = r0 + 128u * i;
                if (r < M)
                {
                    float4 v;
                    v.x = unq_field(bits, wd[i][0], kk[i][0], mask, ca, cb);
                    v.y = unq_field(bits, wd[i][1], kk[i][1], mask, ca, cb);
                    v.z = unq_field(bits, wd[i][2], kk[i][2], mask, ca, cb);
                    v.w = unq_field(bits, wd[i][3], kk[i][3], mask, ca, cb);
                    float4* p = reinterpret_cast<float4*>(out + r);
                    if (ADD)
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
                        __stcs(p, v);
                    }
                }
            }
        }
        else
        {
            // lane <-> rows row0 + lane + 32 * i
            const unsigned r0 = row0 + lane;
            unsigned k = r0 / Q, w = r0 - k * Q;
            const unsigned advK = 32u / Q, advW = 32u - advK * Q;
            constexpr int NS = UNQ_ROWS / 32;
#pragma unroll 4
            for (int i = 0; i < NS; ++i)
            {
                const unsigned r = r0 + 32u * i;
                if (r < M)
                {
                    float val = unq_field(bits, __ldg(words + w), k, mask, ca, cb);
                    if (ADD)
                        val = __fadd_rn(val, out[r]);
                    out[r] = val;
                }
                w += advW;
                k += advK;
                if (w >= Q)
                {
                    w -= Q;
                    ++k;
                }
            }
        }
    }
}

cudaError_t launch_unquantize(cudaStream_t st, bool add, const QTensor* single, const QTensor* tensors, int nTensors, long long totalUnits,
                              const LaunchCfg& cfg)
{
    if (totalUnits <= 0)
        return cudaSuccess;
    long long grid = (long long) cfg.numSMs * 4;
    const long long need = (totalUnits + NWARPS - 1) / NWARPS;
    if (grid > need)
        grid = need;
    static const QTensor zero = {};
    const QTensor& s = single ? *single : zero;
    if (single)
    {
        if (add)
            k_unquantize<true, false><<<(int) grid, NT, 0, st>>>(s, nullptr, 1, totalUnits);
        else
            k_unquantize<false, false><<<(int) grid, NT, 0, st>>>(s, nullptr, 1, totalUnits);
    }
    else
    {
        if (add)
            k_unquantize<true, true><<<(int) grid, NT, 0, st>>>(s, tensors, nTensors, totalUnits);
        else
            k_unquantize<false, true><<<(int) grid, NT, 0, st>>>(s, tensors, nTensors, totalUnits);
    }
    return cudaGetLastError();
}

} // namespace qagg
