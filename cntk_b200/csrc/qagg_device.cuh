// qagg_device.cuh -- device code shared by the column kernels (qagg_kernels.cu, qagg_stream.cu): the value quantizer,
// the routing of packed columns, the range of a column from its ordered sums, and the ordered walks.
//
// Arithmetic contract (what makes the results bit-identical to the reference CPU quantizer,
// Source/Math/ColumnQuantizer.h:209-341 and Source/Math/ValueQuantizer.h:68-162):
//   * every float operation is an explicit round-to-nearest intrinsic (__fadd_rn, __fmul_rn, __fdiv_rn,
//     __fsqrt_rn), so nothing is contracted into a fused multiply-add;
//   * the per-column sums (level sums for 1 bit, sum of squares otherwise, and the mean in mean-threshold
//     mode) are accumulated in ROW ORDER -- float addition is not associative and the reference adds
//     sequentially.  Each of the two level sums of a 1-bit column is its own chain; counts are integers and
//     need no order.
#pragma once

#include "qagg_internal.h"

namespace qagg {

constexpr int NT = 256;     // threads per CTA
constexpr int NWARPS = NT / 32;

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

// The two reconstruction values of a 1-bit column, Unquantize(0) and Unquantize(1) (ValueQuantizer.h:131-141 with
// Nbits = 1): there rangeend = usedrangeend = 2, so ufactor = (upper - lower) / 2.  Halving a normal float is exact
// (the range is at least 1e-36 here), so the divide is replaced by a multiplication by 0.5 with the same result.
__device__ __forceinline__ void levels_1bit(float lower, float upper, float& val0, float& val1)
{
    const float range = __fsub_rn(upper, lower);
    const float ufactor = (range < 1e-36f) ? 0.0f : __fmul_rn(0.5f, range);
    val0 = __fadd_rn(__fmul_rn(0.5f, ufactor), lower);
    val1 = __fadd_rn(__fmul_rn(1.5f, ufactor), lower);
}

// one element of the momentum-SGD update (see UpdateRule): returns the new parameter, rewrites the smoothed gradient
__device__ __forceinline__ float sgd_apply(const UpdateRule& r, float g, float& smoothed, float param)
{
    float s;
    if (r.kind == 0)
        s = __fmaf_rn(r.a, g, smoothed);
    else if (r.kind == 1)
        s = __fmul_rn(r.a, g);
    else
        s = __fmul_rn(r.beta, __fmaf_rn(r.a, g, smoothed));
    smoothed = s;
    return __fsub_rn(param, s);
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
__device__ __forceinline__ unsigned char* packed_col(const QTensor& T, int j)
{
    int p = 0;
    long long first = 0; // first column of owner p's stripe that lies inside this descriptor, in whole-matrix numbering
    const long long jj = (long long) j + T.col0;
    if (T.K > 1)
    {
        const long long per = T.per, rem = T.rem;
        const long long big = (per + 1) * rem; // columns held by the ranks that got one extra
        if (jj < big)
        {
            p = (int) (jj / (per + 1));
            first = (long long) p * (per + 1);
        }
        else
        {
            p = (int) (rem + (jj - big) / per);
            first = big + (p - rem) * per;
        }
        if (first < T.col0)
            first = T.col0;
    }
    else
    {
        first = T.col0;
    }
    return T.pk[p] + (size_t) (jj - first) * (size_t) T.colBytes;
}

// ---- element (row, column j) of the matrix being quantized; slow general form (streamed columns only) ----
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

// ---- range of one column from its ordered sums (ColumnQuantizer.h:279-316, 320-339) ---------------------
template <int MODE>
__device__ __forceinline__ void finalize_range(float a0, float a1, unsigned n0, float mean, long long M, float& lower, float& upper)
{
    const float rows = (float) (unsigned long long) M;
    if (MODE == MODE_MULTIBIT)
    {
        const float stddev = __fsqrt_rn(__fdiv_rn(a0, rows));
        const float w = __fmul_rn(4.0f, stddev);
        lower = __fsub_rn(mean, w);
        upper = __fadd_rn(mean, w);
        return;
    }
    unsigned num0 = n0;
    unsigned num1 = (unsigned) M - n0;
    float radius, newmean;
    if (MODE == MODE_ONEBIT_MEAN)
    {
        const float devacc0 = __fsub_rn(__fmul_rn((float) num0, mean), a0);
        const float devacc1 = __fsub_rn(a1, __fmul_rn((float) num1, mean));
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
        const float mean0 = __fdiv_rn(a0, (float) num0);
        const float mean1 = __fdiv_rn(a1, (float) num1);
        newmean = __fmul_rn(0.5f, __fadd_rn(mean0, mean1));
        radius = __fmul_rn(2.0f, __fsub_rn(mean1, newmean));
    }
    lower = __fsub_rn(newmean, radius);
    upper = __fadd_rn(newmean, radius);
}

// =================================================================================================================
// Ordered walks over one staged column.  Rows are consumed sixteen at a time with the next sixteen already loaded,
// so the only serial dependence is the 4-cycle fp32 add chain of the accumulator.
// =================================================================================================================
enum WalkKind
{
    WALK_SUM = 0,    // acc += v                               (mean of mean-threshold mode)
    WALK_SQUARES,    // acc += v * v                           (multi-bit: mean is the constant 0)
    WALK_MIN0,       // acc += min(v, 0): the rows with v < 0, everything else adds a zero     (zero threshold, lower level)
    WALK_MAX0,       // acc += max(v, 0): the rows with v > 0, everything else adds a zero     (zero threshold, upper level)
    WALK_SPLIT_MEAN  // lower lane: rows with v < mean (counted); upper lane: all other rows   (mean threshold)
};
// One warp issues at most one instruction every other cycle, so a walk keeps up with its 4-cycle add chain only if it
// spends no more than two instructions per row.  WALK_MIN0 / WALK_MAX0 do (FMNMX + FADD); they run in two different
// warps, because inside one warp both levels would have to share one instruction stream.  Adding a zero of either
// sign leaves these sums unchanged (they start at +0 and a round-to-nearest sum is -0 only if both operands are).
// min/max drop a NaN (the reference adds it to the upper sum): the staging pass flags such columns and the upper sum
// is replaced by NaN afterwards.
// The lane's role (lower / upper level) is DATA, not a template argument: both lanes of a pair must run the same
// instruction stream, or the warp would execute the two walks one after the other.

// In the split kinds a lane adds a row only if the row belongs to its level; for the other rows it adds +0, which
// leaves the accumulator unchanged (these sums start at +0 and a round-to-nearest sum with a +0 operand is never -0).
// The selection is done with integer masks, not predicates or branches: a predicate computed per row would sit on
// the critical path of every add, and a branch would make the two lanes of a pair diverge on every row.  With masks
// the selected operands of the next rows are ready long before the add chain needs them, so the walk runs at the
// latency of one fp32 add per row.
//   below  = (v - threshold) has its sign bit set   (exactly v < threshold; also true for -0 - +0 = -0, which adds
//            a harmless -0 to the lower sum where the reference adds it to the upper sum: neither sum changes)
//   lower lane takes v & below, upper lane takes v & ~below.
// A NaN row poisons whichever lane its sign bit selects; the reference poisons the upper sum.  Either way the
// column's range comes out NaN.
__device__ __forceinline__ float pick_mine(float v, float threshold, int laneMask, bool zeroThreshold, unsigned& cnt, bool count)
{
    const int below = __float_as_int(zeroThreshold ? v : __fsub_rn(v, threshold)) >> 31; // all ones when below
    if (count)
        cnt += ((v < threshold) && (laneMask == 0)) ? 1u : 0u;                           // lower lane counts its rows (exact compare)
    return __int_as_float(__float_as_int(v) & (below ^ laneMask));
}

template <int KIND>
__device__ __forceinline__ void walk_step(float& acc, unsigned& cnt, float v, float mean, bool upperLane)
{
    if (KIND == WALK_SUM)
        acc = __fadd_rn(acc, v);
    else if (KIND == WALK_SQUARES)
        acc = __fadd_rn(acc, __fmul_rn(v, v));
    else if (KIND == WALK_MIN0)
        acc = __fadd_rn(acc, fminf(v, 0.0f));
    else if (KIND == WALK_MAX0)
        acc = __fadd_rn(acc, fmaxf(v, 0.0f));
    else
        acc = __fadd_rn(acc, pick_mine(v, mean, upperLane ? -1 : 0, false, cnt, true));
}

template <int KIND>
__device__ __forceinline__ void walk_step4(float& acc, unsigned& cnt, const float4& v, float mean, bool upperLane)
{
    walk_step<KIND>(acc, cnt, v.x, mean, upperLane);
    walk_step<KIND>(acc, cnt, v.y, mean, upperLane);
    walk_step<KIND>(acc, cnt, v.z, mean, upperLane);
    walk_step<KIND>(acc, cnt, v.w, mean, upperLane);
}

// Sixteen rows per trip, the next sixteen already in flight.  The loop is counted in trips and the prefetch index of
// the last trip is clamped (it re-reads its own rows) instead of peeling an epilogue: measured 4.6 cycles per row in
// this shape against 5.3-5.9 for the peeled shapes and 6.9 for eight rows per trip.
template <int KIND>
__device__ __forceinline__ float walk_rows(const float* __restrict__ vcol, int nrows, float acc, unsigned& cnt, float mean, bool upperLane)
{
    const int trips = nrows >> 4;
    if (trips > 0)
    {
        const float4* __restrict__ p = reinterpret_cast<const float4*>(vcol);
        float4 a = p[0], b = p[1], c = p[2], d = p[3];
        for (int t = 0; t < trips; ++t)
        {
            const int nx = (t + 1 < trips) ? (t + 1) * 4 : t * 4;
            const float4 na = p[nx], nb = p[nx + 1], nc = p[nx + 2], nd = p[nx + 3];
            walk_step4<KIND>(acc, cnt, a, mean, upperLane);
            walk_step4<KIND>(acc, cnt, b, mean, upperLane);
            walk_step4<KIND>(acc, cnt, c, mean, upperLane);
            walk_step4<KIND>(acc, cnt, d, mean, upperLane);
            a = na;
            b = nb;
            c = nc;
            d = nd;
        }
    }
    for (int i = trips << 4; i < nrows; ++i)
        walk_step<KIND>(acc, cnt, vcol[i], mean, upperLane);
    return acc;
}

// Releases the peers' flags: ONE system-scope fence orders every earlier store of this thread (and, cumulatively, the
// stores of the CTAs whose arrival it observed) before the flag stores that follow, which can then be relaxed.  A release
// store per flag would repeat the fence once per peer (measured: 2 us each).
__device__ __forceinline__ void release_flags(const Signal& sg)
{
    __threadfence_system();
    for (int i = 0; i < sg.n; ++i)
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(sg.flag[i]), "r"(sg.value) : "memory");
}

__device__ __forceinline__ void store_header(unsigned char* dst, float lower, float upper)
{
    reinterpret_cast<float*>(dst)[0] = lower;
    reinterpret_cast<float*>(dst)[1] = upper;
}

// a packed column's words (and, from the thread that owns word 0, its header) go to the owner's buffer and to every
// broadcast copy: with peer pointers in pk[] / bcast[] these stores ARE the scatter / all-gather traffic over NVLink
__device__ __forceinline__ void store_words(const QTensor& T, const Signal& sg, int j, int w, const unsigned* words, int nw, float lower, float upper)
{
    unsigned char* dst = packed_col(T, j);
    const size_t off = (size_t) (dst - T.pk[0]) + (size_t) T.bcastOff; // used only when T.bcast is set (K == 1 routing)
    const int nb = T.bcast ? sg.nbcast : 0;
    for (int b = -1; b < nb; ++b)
    {
        unsigned char* d = (b < 0) ? dst : sg.bcastBase[b] + off;
        unsigned* pw = reinterpret_cast<unsigned*>(d + 8) + w;
        for (int i = 0; i < nw; ++i)
            pw[i] = words[i];
        if (w == 0)
            store_header(d, lower, upper);
    }
}

} // namespace qagg
