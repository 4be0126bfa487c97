// qagg_unquantize.cu -- the unquantize kernel (UnquantizeOneQWord / Unquantize, Source/Math/ColumnQuantizer.h:69-77, 150-203).
//
// Pure expand-and-store: a packed column of Q words becomes M floats, 32/bits times as many bytes, so the kernel is bound
// by the write bandwidth of HBM and everything is arranged around the stores.
//   * Word-major mapping, as the layout suggests: word w of a column holds rows w, w + Q, w + 2Q, ...  A lane fetches FOUR
//     ADJACENT WORDS once and, per field position k, stores the four rows 4w' + kQ .. + 3 as one aligned 16-byte vector
//     (possible when M and Q are multiples of 4 and the output is 16-byte aligned).  Otherwise a lane takes four words
//     32 apart and the warp stores 32 consecutive rows per position with 4-byte stores.
//   * Work unit = 128 consecutive words of a matrix (columns laid end to end) x 8 field positions = one warp; 4 KB of
//     output in the 1-bit case.  Warps take units u, u + (warps in the grid), ...: no shared memory, no barrier, no
//     atomics.  A launch has ten or so units per resident warp and the grid is sized so that they divide evenly, so all
//     CTAs end together; a launch with one CTA per group of columns did not (its last partial wave of CTAs ran on a mostly
//     idle GPU).
//   * Units are numbered matrix after matrix, the field-position blocks of one word group next to each other:
//     neighbouring warps write neighbouring memory.
#include "qagg_device.cuh"

namespace qagg {

constexpr int UNQ_WORDS = 128; // packed words per unit
constexpr int UNQ_KPU = 8;     // field positions per unit

// field-position blocks per word: 4 for 1 bit, 2 for 2 bits, else 1 (always a power of two)
__host__ __device__ __forceinline__ int unq_ksplit(int bits)
{
    const int vpw = 32 / bits;
    return (vpw + UNQ_KPU - 1) / UNQ_KPU;
}

long long unq_units(long long M, long long N, int bits)
{
    if (M <= 0 || N <= 0)
        return 0;
    const long long Q = (M * bits + 31) / 32;
    return ((N * Q + UNQ_WORDS - 1) / UNQ_WORDS) * unq_ksplit(bits);
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

// One unit as a lane sees it: where it writes, and the packed words and column headers it needs (fetched one unit ahead).
struct UnqUnit
{
    float* op[4];     // destination of position 0 of each of the lane's (up to four) words; vector form: op[0] only
    unsigned wd[4];   // the words
    float lo[4], up[4];
    unsigned w[4];    // word index within its column (for the end-of-column check)
    unsigned M, Q, k0;
    int bits;
    unsigned live;    // bit e set: word e exists
    bool vec;
};

template <bool TABLE>
__device__ __forceinline__ void unq_fetch(UnqUnit& x, const QTensor& single, const QTensor* __restrict__ tensors, int nTensors, long long u, int& cur,
                                          unsigned lane, bool onebit)
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
    x.M = M;
    x.Q = Q;
    x.bits = onebit ? 1 : Tp->bits;
    const int ks = unq_ksplit(x.bits);
    const int ksShift = (ks == 4) ? 2 : (ks == 2) ? 1 : 0;
    const unsigned long long local = (unsigned long long) (u - (TABLE ? Tp->unit0 : 0));
    x.k0 = (unsigned) (local & (unsigned long long) (ks - 1)) * UNQ_KPU;
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
    x.vec = ((M & 3u) == 0) && ((Q & 3u) == 0) && ((reinterpret_cast<uintptr_t>(outBase) & 15) == 0);
    x.live = 0u;
    if (x.vec)
    {
        // lane <-> words 4 * lane .. + 3 of the unit: the same column (Q is a multiple of 4), rows 4-aligned
        const unsigned off = 4u * lane;
        if (off < left)
        {
            const unsigned tl = w0 + off;
            const unsigned dc = tl / Q;
            const unsigned c = col0 + dc, w = tl - dc * Q;
            const unsigned char* colp = TABLE ? packed_col(*Tp, (int) c) : single.pk[0] + (size_t) c * (size_t) single.colBytes;
            x.lo[0] = __ldg(reinterpret_cast<const float*>(colp));
            x.up[0] = __ldg(reinterpret_cast<const float*>(colp) + 1);
            const unsigned* __restrict__ words = reinterpret_cast<const unsigned*>(colp + 8) + w;
#pragma unroll
            for (int e = 0; e < 4; ++e)
                x.wd[e] = __ldg(words + e);
            x.w[0] = w;
            x.op[0] = outBase + (size_t) c * M + w + (size_t) x.k0 * Q;
            x.live = 1u;
        }
    }
    else
    {
        // lane <-> words lane, lane + 32, lane + 64, lane + 96 of the unit: per position the warp stores 32 consecutive rows
#pragma unroll
        for (int e = 0; e < 4; ++e)
        {
            const unsigned off = lane + 32u * e;
            if (off < left)
            {
                const unsigned tl = w0 + off;
                const unsigned dc = tl / Q;
                const unsigned c = col0 + dc, w = tl - dc * Q;
                const unsigned char* colp = TABLE ? packed_col(*Tp, (int) c) : single.pk[0] + (size_t) c * (size_t) single.colBytes;
                x.lo[e] = __ldg(reinterpret_cast<const float*>(colp));
                x.up[e] = __ldg(reinterpret_cast<const float*>(colp) + 1);
                x.wd[e] = __ldg(reinterpret_cast<const unsigned*>(colp + 8) + w);
                x.w[e] = w;
                x.op[e] = outBase + (size_t) c * M + w + (size_t) x.k0 * Q;
                x.live |= 1u << e;
            }
        }
    }
}

template <bool ADD, bool ONEBIT>
__device__ __forceinline__ void unq_emit(const UnqUnit& x)
{
    const int bits = ONEBIT ? 1 : x.bits;
    const unsigned vpw = 32u / (unsigned) bits;
    const unsigned mask = (bits >= 32) ? 0xffffffffu : ((1u << bits) - 1u);
    const unsigned Q = x.Q, k0 = x.k0;
    // positions of this unit that exist at all; a word's rows may end earlier (last words of a column whose height is not
    // a multiple of Q): `full` says that they do not
    const unsigned nk = (vpw - k0 < UNQ_KPU) ? vpw - k0 : UNQ_KPU;
    if (x.vec)
    {
        if (!x.live)
            return;
        float ca, cb;
        unq_consts(bits, x.lo[0], x.up[0], ca, cb);
        const bool full = (nk == UNQ_KPU) && (x.w[0] + (k0 + UNQ_KPU - 1) * Q < x.M);
        float* __restrict__ op = x.op[0];
#pragma unroll
        for (unsigned kk = 0; kk < UNQ_KPU; ++kk)
        {
            const unsigned k = k0 + kk;
            if (full || (kk < nk && x.w[0] + k * Q < x.M))
            {
                float4 v;
                v.x = unq_field<ONEBIT>(bits, x.wd[0], k, mask, ca, cb);
                v.y = unq_field<ONEBIT>(bits, x.wd[1], k, mask, ca, cb);
                v.z = unq_field<ONEBIT>(bits, x.wd[2], k, mask, ca, cb);
                v.w = unq_field<ONEBIT>(bits, x.wd[3], k, mask, ca, cb);
                float4* p = reinterpret_cast<float4*>(op + (size_t) kk * Q);
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
#pragma unroll
        for (int e = 0; e < 4; ++e)
        {
            if (x.live & (1u << e))
            {
                float ca, cb;
                unq_consts(bits, x.lo[e], x.up[e], ca, cb);
                const bool full = (nk == UNQ_KPU) && (x.w[e] + (k0 + UNQ_KPU - 1) * Q < x.M);
                float* __restrict__ op = x.op[e];
                const unsigned word = x.wd[e];
#pragma unroll
                for (unsigned kk = 0; kk < UNQ_KPU; ++kk)
                {
                    const unsigned k = k0 + kk;
                    if (full || (kk < nk && x.w[e] + k * Q < x.M))
                    {
                        float val = unq_field<ONEBIT>(bits, word, k, mask, ca, cb);
                        if (ADD)
                            val = __fadd_rn(val, op[(size_t) kk * Q]);
                        op[(size_t) kk * Q] = val;
                    }
                }
            }
        }
    }
}

// Warps take units u, u + warps, ...; the words and headers of a warp's next unit are fetched before it expands the
// current one, so the (dependent) loads of one unit overlap the stores of the other.
template <bool ADD, bool TABLE, bool ONEBIT>
__global__ void __launch_bounds__(NT, 3) k_unquantize(const QTensor single, const QTensor* __restrict__ tensors, int nTensors, long long totalUnits)
{
    const unsigned lane = threadIdx.x & 31;
    const long long gwarp = (long long) blockIdx.x * NWARPS + (threadIdx.x >> 5);
    const long long nwarps = (long long) gridDim.x * NWARPS;
    long long u = gwarp;
    if (u >= totalUnits)
        return;
    int cur = 0; // table entry of the previous unit: consecutive units of a warp mostly stay within one matrix
    UnqUnit xa, xb;
    unq_fetch<TABLE>(xa, single, tensors, nTensors, u, cur, lane, ONEBIT);
    for (;;)
    {
        const bool moreB = u + nwarps < totalUnits;
        if (moreB)
            unq_fetch<TABLE>(xb, single, tensors, nTensors, u + nwarps, cur, lane, ONEBIT);
        unq_emit<ADD, ONEBIT>(xa);
        if (!moreB)
            break;
        u += nwarps;
        const bool moreA = u + nwarps < totalUnits;
        if (moreA)
            unq_fetch<TABLE>(xa, single, tensors, nTensors, u + nwarps, cur, lane, ONEBIT);
        unq_emit<ADD, ONEBIT>(xb);
        if (!moreA)
            break;
        u += nwarps;
    }
}

// Grid: at most three CTAs per SM; among the sizes from two to three per SM, the one whose warps share the units most evenly.
static int unq_grid(long long totalUnits, int numSMs)
{
    const long long need = (totalUnits + NWARPS - 1) / NWARPS;
    const long long most = (long long) numSMs * 3;
    if (need <= most)
        return (int) need;
    long long best = most;
    double bestWaste = 2.0;
    for (long long g = most; g >= (long long) numSMs * 2; --g)
    {
        const long long warps = g * NWARPS;
        const long long rounds = (totalUnits + warps - 1) / warps;
        const double waste = 1.0 - (double) totalUnits / (double) (rounds * warps);
        if (waste < bestWaste - 1e-9)
        {
            bestWaste = waste;
            best = g;
        }
    }
    return (int) best;
}

cudaError_t launch_unquantize(cudaStream_t st, bool add, int bits, const QTensor* single, const QTensor* tensors, int nTensors, long long totalUnits,
                              const LaunchCfg& cfg)
{
    if (totalUnits <= 0)
        return cudaSuccess;
    const int grid = unq_grid(totalUnits, cfg.numSMs);
    static const QTensor zero = {};
    const QTensor& s = single ? *single : zero;
    const bool table = (single == nullptr);
    const bool onebit = (bits == 1);
#define QAGG_UNQ_CASE(A, T, O)                  \
    if (add == A && table == T && onebit == O) \
        k_unquantize<A, T, O><<<grid, NT, 0, st>>>(s, tensors, nTensors, totalUnits);
    QAGG_UNQ_CASE(false, false, false)
    QAGG_UNQ_CASE(false, false, true)
    QAGG_UNQ_CASE(false, true, false)
    QAGG_UNQ_CASE(false, true, true)
    QAGG_UNQ_CASE(true, false, false)
    QAGG_UNQ_CASE(true, false, true)
    QAGG_UNQ_CASE(true, true, false)
    QAGG_UNQ_CASE(true, true, true)
#undef QAGG_UNQ_CASE
    return cudaGetLastError();
}

} // namespace qagg
