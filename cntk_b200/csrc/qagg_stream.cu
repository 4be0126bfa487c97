// qagg_stream.cu -- streaming column kernel for 1-bit quantization with threshold 0 and a deferred residual.
//
// Why a second column kernel.  The per-column level sums must be added in row order (qagg_device.cuh), one 4-cycle
// fp32 add per row and level.  A kernel that keeps whole columns in shared memory until their range is known (needed
// to write the residual v - Unquantize(bit)) can hold only a handful of tall columns per SM, so few add chains run at
// once and the memory system idles while they do.  For 1 bit with threshold 0 the bit of a value does not depend on
// the range at all, only the residual does -- and the residual is read again only by the next step.  So this kernel
// stores v itself plus the column's two reconstruction values and lets the NEXT read form v - level(v): the same
// single round-to-nearest subtraction the reference performs (ColumnQuantizer.h:100-125), merely later.  Nothing has
// to stay resident: columns stream through shared memory in row chunks, every input and output crosses HBM once, and
// the number of add chains in flight is no longer tied to the column height.
//
// One work item = nc <= 32 adjacent columns of one matrix, processed in chunks of R rows (nc * R <= 1536 values):
//   * six "element" warps copy the chunk's inputs global -> shared with cp.async (two chunks ahead), then form
//       v = gradient + (prev - level(prev))                                   (quantize), or
//       v = sum over the K packed stripes in source order + (prev - level(prev))   (owner's reduce-requantize),
//     store v to global memory and to the chunk tile, and OR the bit (v >= 0) into the item's packed words, which
//     live in shared memory until the item ends;
//   * two "walker" warps (one per level, lane = column) add min(v, 0) resp. max(v, 0) of the previous chunk to their
//     running sums, in row order;
//   * at the end the ranges and the new reconstruction values are derived and the packed columns go to their owners.
#include "qagg_device.cuh"

#include <algorithm>

namespace qagg {

constexpr int ST_WALK_WARPS = 2;
constexpr int ST_ETHREADS = NT - 32 * ST_WALK_WARPS; // 192 element threads
#ifndef QAGG_ST_U
#define QAGG_ST_U 2
#endif
#ifndef QAGG_ST_STAGES
#define QAGG_ST_STAGES 4
#endif
#ifndef QAGG_ST_CTAS
#define QAGG_ST_CTAS 3
#endif
constexpr int ST_U = QAGG_ST_U;                      // 16-byte positions per element thread and chunk
constexpr int ST_TILE_VALUES = 4 * ST_U * ST_ETHREADS; // 1536 values per chunk
constexpr int ST_STAGES = QAGG_ST_STAGES;                         // chunk tiles in the ring: 1 walked, 1 formed, 2 in flight
constexpr int ST_DIST = ST_STAGES - 2;               // how many chunks ahead the copies run
constexpr int ST_TILE_FLOATS = ST_TILE_VALUES + 4 * QAGG_STREAM_CMAX; // room for the 4-float pad of every column
constexpr int ST_CTAS_PER_SM = QAGG_ST_CTAS;
constexpr size_t ST_SMEM_BYTES = (size_t) (2 * ST_STAGES * ST_TILE_FLOATS + QAGG_STREAM_PKWORDS) * 4;

// rows per chunk for an item of nc columns: a multiple of 32, so that the tile's column stride R + 4 is 4 mod 32 and
// the walkers' 128-bit reads of neighbouring columns fall into distinct banks
__device__ __forceinline__ int stream_rows(int nc)
{
    return ((ST_TILE_VALUES / nc) >> 5) << 5;
}

__device__ __forceinline__ void cp_async16(float* dstShared, const float* src)
{
    const unsigned dst = (unsigned) __cvta_generic_to_shared(dstShared);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(float* dstShared, const float* src)
{
    const unsigned dst = (unsigned) __cvta_generic_to_shared(dstShared);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ float deferred_residual(float prev, float lv0, float lv1)
{
    return __fsub_rn(prev, (prev >= 0.0f) ? lv1 : lv0);
}

// optional phase timers for development builds (-DQAGG_PROBE; the array is defined in qagg_kernels.cu)
#ifdef QAGG_PROBE
#define ST_MARK(var) const long long var = clock64()
#define ST_ADD(i, a, b)  \
    if (et == 0 && !isWalker) \
    atomicAdd(&g_probe[i], (unsigned long long) ((b) - (a)))
#else
#define ST_MARK(var)
#define ST_ADD(i, a, b)
#endif

static_assert(sizeof(QTensor) % 16 == 0 && sizeof(QTensor) <= 32 * 16, "a warp copies one descriptor with 16-byte cp.async");

template <bool STRIPES>
__global__ void __launch_bounds__(NT, ST_CTAS_PER_SM) k_stream1(const QTensor* __restrict__ tensors, const QItem* __restrict__ items, int nItems,
                                                                unsigned* __restrict__ counters, const Signal signal)
{
    extern __shared__ __align__(16) float dsm[];
    float* const tileG = dsm;                               // gradient (or raw own stripe), replaced in place by v
    float* const tileP = dsm + ST_STAGES * ST_TILE_FLOATS;   // previous state
    // the item's packed words (nc x Q), then -- owner kernel -- its packed source columns, headers included
    // ([source][column][2 + Q] words)
    unsigned* const pkw = reinterpret_cast<unsigned*>(dsm + 2 * ST_STAGES * ST_TILE_FLOATS);
    // descriptor, work item and previous reconstruction values are double-buffered: while one item streams, the next
    // one's are fetched
    __shared__ __align__(16) QTensor sT[2];
    __shared__ QItem sItem[2];
    __shared__ int sIt[2];
    __shared__ int sWalker;
    __shared__ float sLv0[QAGG_STREAM_CMAX], sLv1[QAGG_STREAM_CMAX], sA0[QAGG_STREAM_CMAX], sA1[QAGG_STREAM_CMAX];
    __shared__ float sLower[QAGG_STREAM_CMAX], sUpper[QAGG_STREAM_CMAX];
    __shared__ unsigned sN0[QAGG_STREAM_CMAX], sNan[QAGG_STREAM_CMAX];
    __shared__ unsigned char* sDst[QAGG_STREAM_CMAX];
    __shared__ float sSrc0[STRIPES ? QAGG_MAXK : 1][QAGG_STREAM_CMAX], sSrc1[STRIPES ? QAGG_MAXK : 1][QAGG_STREAM_CMAX];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#ifdef QAGG_PROBE
    const long long tKernel0 = clock64();
    unsigned long long gt0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt0));
#endif
    if (tid == 0)
    {
        // the walkers of the CTAs that share an SM sit on different warp pairs (a per-SM ticket that only ever grows)
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        sWalker = (int) ((atomicAdd(&counters[8 + (smid & 255u)], 1u) & 3u) * 2u);
        const int first = (int) atomicAdd(&counters[0], 1u);
        sIt[0] = first;
        if (first < nItems)
            sItem[0] = items[first];
    }
    __syncthreads();
    const int ww = sWalker;
    const bool isWalker = (warp == ww) || (warp == ww + 1);
    const int et = ((warp > ww) ? warp - ST_WALK_WARPS : warp) * 32 + lane; // index among the element threads
    bool more = sIt[0] < nItems;
    if (more)
    {
        const int* srcw = reinterpret_cast<const int*>(tensors + sItem[0].tensor);
        int* dstw = reinterpret_cast<int*>(&sT[0]);
        for (int i = tid; i < (int) (sizeof(QTensor) / sizeof(int)); i += NT)
            dstw[i] = srcw[i];
    }
    __syncthreads();

    // ---- the item being streamed: geometry (uniform) and this thread's positions ----------------------------------------
    const QTensor* Tp = &sT[0];
    int M = 1, Q = 1, nc = 1, col0 = 0, R = 32, stride = 36, nchunks = 0;
    bool hasG = true, vec = false;
    const float* gbase = nullptr;
    const float* pbase = nullptr;
    float* obase = nullptr;
    unsigned advK = 0, advW = 0;
    unsigned ring = 0;                  // ring slot of the item's chunk 0
    float lvReg0 = 0.0f, lvReg1 = 0.0f; // thread c < nc: the previous reconstruction values of column c, loaded ahead
    // An element thread owns the same ST_U 16-byte positions (column, four rows) of every chunk.  Row i of a column is
    // bit i / Q of packed word i % Q; the position's (word, bit) pair moves by a fixed step from chunk to chunk.
    bool pv[ST_U];
    int sofs[ST_U], pcol[ST_U], prow[ST_U];
    size_t gofs[ST_U];
    unsigned pw[ST_U], pk[ST_U], nanf[ST_U];

    // element threads: the inputs of chunk q, 16 bytes per position (4 bytes per value for unaligned matrices)
    auto issue = [&](int q) {
        if (q < nchunks)
        {
            const int slotOff = (int) ((ring + (unsigned) q) % ST_STAGES) * ST_TILE_FLOATS;
            const int row0 = q * R;
#pragma unroll
            for (int u = 0; u < ST_U; ++u)
            {
                const int row = row0 + prow[u];
                if (!pv[u] || row >= M)
                    continue;
                const int so = slotOff + sofs[u];
                const size_t go = gofs[u] + (size_t) row0;
                if (vec)
                {
                    if (hasG)
                        cp_async16(tileG + so, gbase + go);
                    cp_async16(tileP + so, pbase + go);
                }
                else
                {
                    for (int i = 0; i < 4 && row + i < M; ++i)
                    {
                        if (hasG)
                            cp_async4(tileG + so + i, gbase + go + i);
                        cp_async4(tileP + so + i, pbase + go + i);
                    }
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // take over the item described by sT[b] / sItem[b] and put its first chunks into flight (every tile must be free of
    // readers and writers of the generic proxy: call after a barrier that follows the last walk)
    auto adopt = [&](int b, unsigned chunksBefore) {
        Tp = &sT[b];
        const QTensor& T = *Tp;
        ring = (ring + chunksBefore) % ST_STAGES;
        M = (int) T.M;
        Q = T.Q;
        nc = sItem[b].ncols;
        col0 = sItem[b].col0;
        R = stream_rows(nc);
        stride = R + 4;
        nchunks = (M + R - 1) / R;
        hasG = !STRIPES || T.selfRaw;
        gbase = T.grad;
        pbase = T.res_in;
        obase = T.res_out;
        vec = ((M & 3) == 0) && ((reinterpret_cast<uintptr_t>(pbase) & 15) == 0) && ((reinterpret_cast<uintptr_t>(obase) & 15) == 0) &&
              (!hasG || (reinterpret_cast<uintptr_t>(gbase) & 15) == 0);
        advK = (unsigned) R / (unsigned) Q;
        advW = (unsigned) R - advK * (unsigned) Q;
        const int R4 = R >> 2;
#pragma unroll
        for (int u = 0; u < ST_U; ++u)
        {
            const int f = et + ST_ETHREADS * u;
            pv[u] = !isWalker && f < nc * R4;
            const int c = pv[u] ? f / R4 : 0;
            const int r = pv[u] ? 4 * (f - c * R4) : 0;
            pcol[u] = c;
            prow[u] = r;
            sofs[u] = c * stride + r;
            gofs[u] = (size_t) (col0 + c) * (size_t) M + (size_t) r;
            pk[u] = (unsigned) r / (unsigned) Q;
            pw[u] = (unsigned) r - pk[u] * (unsigned) Q;
            nanf[u] = 0u;
        }
        if (!isWalker)
            for (int q = 0; q < ST_DIST; ++q)
                issue(q);
        if (tid < nc)
        {
            lvReg0 = T.lv[2 * (size_t) (col0 + tid)];
            lvReg1 = T.lv[2 * (size_t) (col0 + tid) + 1];
        }
    };

    int par = 0;
    if (more)
        adopt(0, 0u);

    while (more)
    {
        ST_MARK(tItem0);
        const QTensor& T = *Tp;
        const int nsrc = STRIPES ? T.nsrc : 0;
        const int firstPacked = hasG ? 1 : 0;      // owner kernel: sources firstPacked .. nsrc - 1 are packed
        const int colWords = Q + 2;
        unsigned* const srcw = pkw + nc * Q;       // staged packed sources

        // ---- per-item state --------------------------------------------------------------------------------------------
        for (int i = tid; i < nc * Q; i += NT)
            pkw[i] = 0u;
        if (tid < nc)
        {
            sLv0[tid] = lvReg0;
            sLv1[tid] = lvReg1;
            sNan[tid] = 0u;
            sDst[tid] = packed_col(T, col0 + tid);
        }
        // owner kernel: the item's columns of every packed source are staged in shared memory when they fit next to the
        // item's own packed words (one contiguous block of nc * (2 + Q) words per source); else they are read in place
        const bool staged = STRIPES && (nc * Q + (nsrc - firstPacked) * nc * colWords <= QAGG_STREAM_PKWORDS);
        if (STRIPES)
        {
            if (staged)
            {
                const int blockWords = nc * colWords;
                for (int s = firstPacked; s < nsrc; ++s)
                {
                    const unsigned* src = reinterpret_cast<const unsigned*>(T.src[s] + (size_t) col0 * T.colBytes);
                    unsigned* dst = srcw + (s - firstPacked) * blockWords;
                    for (int i = tid; i < blockWords; i += NT)
                        dst[i] = __ldg(src + i);
                }
                __syncthreads();
            }
            for (int i = tid; i < (nsrc - firstPacked) * nc; i += NT)
            {
                const int sp = i / nc, c = i - sp * nc;
                const unsigned* hdr = staged ? srcw + (sp * nc + c) * colWords
                                             : reinterpret_cast<const unsigned*>(T.src[sp + firstPacked] + (size_t) (col0 + c) * T.colBytes);
                float v0, v1;
                levels_1bit(__uint_as_float(hdr[0]), __uint_as_float(hdr[1]), v0, v1);
                sSrc0[STRIPES ? sp : 0][c] = v0;
                sSrc1[STRIPES ? sp : 0][c] = v1;
            }
        }
        __syncthreads();

        auto form = [&](int q) {
            const int slotOff = (int) ((ring + (unsigned) q) % ST_STAGES) * ST_TILE_FLOATS;
            const int row0 = q * R;
#pragma unroll
            for (int u = 0; u < ST_U; ++u)
            {
                const int row = row0 + prow[u];
                if (pv[u] && row < M)
                {
                    const int c = pcol[u];
                    const int so = slotOff + sofs[u];
                    const int nv = vec ? 4 : min(4, M - row);
                    float prev[4];
                    float agg[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    {
                        const float4 p4 = *reinterpret_cast<const float4*>(tileP + so);
                        prev[0] = p4.x;
                        prev[1] = p4.y;
                        prev[2] = p4.z;
                        prev[3] = p4.w;
                        if (hasG)
                        {
                            const float4 g4 = *reinterpret_cast<const float4*>(tileG + so);
                            agg[0] = g4.x;
                            agg[1] = g4.y;
                            agg[2] = g4.z;
                            agg[3] = g4.w;
                        }
                    }
                    const float lv0 = sLv0[c], lv1 = sLv1[c];
                    // the usual case: the four rows are the same bit of four adjacent words
                    const bool flat = (nv == 4) && (pw[u] + 3u < (unsigned) Q);
                    if (STRIPES)
                    {
                        // (word, bit) of the four rows
                        unsigned wi[4], ki[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                        {
                            const unsigned w = pw[u] + i;
                            const unsigned over = flat ? 0u : w / (unsigned) Q;
                            ki[i] = pk[u] + over;
                            wi[i] = w - over * (unsigned) Q;
                        }
                        // the K sources in index order (the own stripe first), the residual last
                        // (AllReduceDistGradAggregator.h:366-375, 405-435)
                        bool first = !hasG;
                        for (int sp = 0; sp < nsrc - firstPacked; ++sp)
                        {
                            const float s0 = sSrc0[STRIPES ? sp : 0][c], s1 = sSrc1[STRIPES ? sp : 0][c];
                            const unsigned* words = staged ? srcw + (sp * nc + c) * colWords + 2
                                                           : reinterpret_cast<const unsigned*>(T.src[sp + firstPacked] + (size_t) (col0 + c) * T.colBytes) + 2;
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                            {
                                if (i < nv)
                                {
                                    const unsigned word = staged ? words[wi[i]] : __ldg(words + wi[i]);
                                    const float val = ((word >> ki[i]) & 1u) ? s1 : s0;
                                    agg[i] = first ? val : __fadd_rn(val, agg[i]);
                                }
                            }
                            first = false;
                        }
                    }
                    float v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        v[i] = __fadd_rn(agg[i], deferred_residual(prev[i], lv0, lv1));
                    unsigned* const myWords = pkw + c * Q;
                    if (flat)
                    {
                        unsigned* const wp = myWords + pw[u];
                        const unsigned m = 1u << pk[u];
                        nanf[u] |= ((v[0] != v[0]) | (v[1] != v[1]) | (v[2] != v[2]) | (v[3] != v[3])) ? 1u : 0u;
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#ifndef QAGG_ST_NO_ATOM
                            if (v[i] >= 0.0f)
#else
                            if (v[i] == 123.0f)
#endif
                                atomicOr(wp + i, m);
                    }
                    else
                    {
                        for (int i = 0; i < nv; ++i)
                        {
                            const unsigned w = pw[u] + i;
                            const unsigned over = w / (unsigned) Q;
                            nanf[u] |= (v[i] != v[i]) ? 1u : 0u;
                            if (v[i] >= 0.0f)
                                atomicOr(myWords + (w - over * (unsigned) Q), 1u << (pk[u] + over));
                        }
                    }
                    const float4 v4 = make_float4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<float4*>(tileG + so) = v4;
                    float* gout = obase + gofs[u] + (size_t) row0;
                    if (vec)
                        *reinterpret_cast<float4*>(gout) = v4;
                    else
                        for (int i = 0; i < nv; ++i)
                            gout[i] = v[i];
                }
                // on to the next chunk's rows
                pw[u] += advW;
                pk[u] += advK;
                if (pw[u] >= (unsigned) Q)
                {
                    pw[u] -= (unsigned) Q;
                    ++pk[u];
                }
            }
        };

        // ---- the chunk loop ----------------------------------------------------------------------------------------------
        // iteration q: chunk q's values are formed, chunk q - 1 is walked and on its way to global memory, the inputs of
        // chunks q + 1 .. q + ST_DIST are in flight
        float acc = 0.0f; // a walker lane's running sum of its column
        ST_MARK(tLoop0);
        ST_ADD(0, tItem0, tLoop0);
        for (int q = 0; q <= nchunks; ++q)
        {
            ST_MARK(tq0);
            if (!isWalker)
            {
                issue(q + ST_DIST); // into the tile of chunk q - 2, which was walked before the last barrier
                ST_MARK(tq1);
                ST_ADD(1, tq0, tq1);
                // all but the ST_DIST newest copy groups have landed: chunk q is complete, and this thread forms exactly
                // the positions it copied itself
                asm volatile("cp.async.wait_group %0;" ::"n"(ST_DIST) : "memory");
                ST_MARK(tq2);
                ST_ADD(2, tq1, tq2);
                if (q < nchunks)
                    form(q);
                ST_MARK(tq3);
                ST_ADD(3, tq2, tq3);
            }
            else
            {
                if (q == 0 && warp == ww)
                {
                    // nothing to walk yet: fetch the index of this CTA's next item, the item and (asynchronously) its
                    // descriptor; they are read after the loop's last barrier
                    int nx = 0;
                    if (lane == 0)
                        nx = (int) atomicAdd(&counters[0], 1u);
                    nx = __shfl_sync(0xffffffffu, nx, 0);
                    if (lane == 0)
                        sIt[par ^ 1] = nx;
                    if (nx < nItems)
                    {
                        const int word = (lane < 3) ? reinterpret_cast<const int*>(items + nx)[lane] : 0;
                        if (lane < 3)
                            reinterpret_cast<int*>(&sItem[par ^ 1])[lane] = word;
                        const int tIdx = __shfl_sync(0xffffffffu, word, 0);
                        if (lane < (int) (sizeof(QTensor) / 16))
                            cp_async16(reinterpret_cast<float*>(&sT[par ^ 1]) + 4 * lane, reinterpret_cast<const float*>(tensors + tIdx) + 4 * lane);
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                }
#ifdef QAGG_ST_NO_WALK
                if (q == 1 && lane < nc)
#else
                if (q >= 1 && lane < nc)
#endif
                {
                    const int qq = q - 1;
                    const int nrows = min(R, M - qq * R);
                    const float* vcol = tileG + (int) ((ring + (unsigned) qq) % ST_STAGES) * ST_TILE_FLOATS + lane * stride;
                    unsigned dummy = 0;
                    if (warp == ww)
                        acc = walk_rows<WALK_MIN0>(vcol, nrows, acc, dummy, 0.0f, false);
                    else
                        acc = walk_rows<WALK_MAX0>(vcol, nrows, acc, dummy, 0.0f, true);
                }
                if (q == nchunks && warp == ww)
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            ST_MARK(tq4);
            __syncthreads(); // chunk q is formed (next: walked and stored), chunk q - 1 is walked
            ST_MARK(tq5);
            ST_ADD(4, tq4, tq5);
            ST_ADD(6, 0, 1);
        }
        ST_MARK(tLoop1);

        // ---- finish: the next item's first chunks go into flight first (every tile is free now) ------------------------------
        if (isWalker)
        {
            if (lane < nc)
                (warp == ww ? sA0 : sA1)[lane] = acc;
        }
        else
        {
#pragma unroll
            for (int u = 0; u < ST_U; ++u)
                if (pv[u] && nanf[u])
                    sNan[pcol[u]] = 1u;
        }
        const int fnc = nc, fQ = Q, fcol0 = col0; // the finishing item's geometry
        const unsigned used = (unsigned) nchunks; // ring slots this item went through
        more = sIt[par ^ 1] < nItems;
        if (more)
            adopt(par ^ 1, used);
        __syncthreads();
        // rows below the threshold = rows whose bit is 0 (a NaN row has bit 0 too, but then the range is NaN whatever the count)
        for (int c = warp; c < fnc; c += NWARPS)
        {
            unsigned ones = 0;
            for (int w = lane; w < fQ; w += 32)
                ones += __popc(pkw[c * fQ + w]);
            ones = __reduce_add_sync(0xffffffffu, ones);
            if (lane == 0)
                sN0[c] = (unsigned) T.M - ones;
        }
        __syncthreads();
        if (tid < fnc)
        {
            // min/max drop a NaN where the reference adds it to the upper sum: put it back
            float lo, up, v0, v1;
            finalize_range<MODE_ONEBIT_ZERO>(sA0[tid], sNan[tid] ? __int_as_float(0x7fc00000) : sA1[tid], sN0[tid], 0.0f, T.M, lo, up);
            sLower[tid] = lo;
            sUpper[tid] = up;
            levels_1bit(lo, up, v0, v1);
            T.lv[2 * (size_t) (fcol0 + tid)] = v0;
            T.lv[2 * (size_t) (fcol0 + tid) + 1] = v1;
        }
        __syncthreads();
        // packed columns to their owners (and to the broadcast copies): warp <-> column, lane <-> word
        {
            const int nb = T.bcast ? signal.nbcast : 0;
            for (int c = warp; c < fnc; c += NWARPS)
            {
                unsigned char* const dst = sDst[c];
                const size_t off = (size_t) (dst - T.pk[0]) + (size_t) T.bcastOff;
                for (int b = -1; b < nb; ++b)
                {
                    unsigned char* d = (b < 0) ? dst : signal.bcastBase[b] + off;
                    unsigned* out = reinterpret_cast<unsigned*>(d + 8);
                    for (int w = lane; w < fQ; w += 32)
                        out[w] = pkw[c * fQ + w];
                    if (lane == 0)
                        store_header(d, sLower[c], sUpper[c]);
                }
            }
        }
        __syncthreads(); // the item is done with its shared-memory state
        ST_MARK(tItem1);
        ST_ADD(5, tLoop1, tItem1);
        ST_ADD(7, 0, 1);
        par ^= 1;
    }

#ifdef QAGG_PROBE
    if (tid == 0)
    {
        unsigned long long gt1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt1));
        atomicAdd(&g_probe[8], (unsigned long long) (clock64() - tKernel0)); // cycles this CTA lived
        atomicAdd(&g_probe[9], gt1 - gt0);                                    // nanoseconds this CTA lived
        atomicAdd(&g_probe[10], 1ull);
        atomicMin(&g_probe[11], gt0);
        atomicMax(&g_probe[12], gt1);
        atomicMax(&g_probe[13], gt1 - gt0);
    }
#endif
    // The last CTA to leave re-arms the work counter for the next launch and releases the peers' flags: each CTA's
    // stores (into peer memory too) are ordered before its arrival by barrier + system-scope fence.
    if (tid == 0)
    {
        __threadfence_system();
        const unsigned done = atomicAdd(&counters[1], 1u);
        if (done == gridDim.x - 1)
        {
            counters[0] = 0;
            counters[1] = 0;
            __threadfence_system();
            for (int i = 0; i < signal.n; ++i)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(signal.flag[i]), "r"(signal.value) : "memory");
        }
    }
}

// the residual proper of a deferred state, element by element (export, checkpoint, tests)
__global__ void __launch_bounds__(256) k_materialize(const float* __restrict__ buf, const float* __restrict__ lv, float* __restrict__ dst,
                                                     long long M, long long N)
{
    const long long total = M * N;
    for (long long idx = (long long) blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long) gridDim.x * blockDim.x)
    {
        const long long col = idx / M;
        dst[idx] = deferred_residual(buf[idx], lv[2 * col], lv[2 * col + 1]);
    }
}

// Column counts whose chunk (1536 / nc rows, a multiple of 32) fills the chunk tile completely; the one nearest in ratio
// to `want`, at most `most`
static int nice_cols(double want, int most)
{
    static const int nice[] = {1, 2, 3, 4, 6, 8, 12, 16, 24};
    if (want < 1.0)
        want = 1.0;
    int best = 1;
    double bestRatio = want;
    for (int n : nice)
    {
        if (n > most)
            break;
        const double ratio = n > want ? n / want : want / n;
        if (ratio < bestRatio)
        {
            bestRatio = ratio;
            best = n;
        }
    }
    return best;
}

void stream_make_items(const std::vector<std::pair<long long, long long>>& shapes, int numSMs, int bits, int packedSources,
                       std::vector<QItem>& out)
{
    long long total = 0;
    for (auto& sh : shapes)
        total += sh.first * sh.second;
    const long long slots = (long long) numSMs * ST_CTAS_PER_SM;
    long long target = total / (3 * slots > 0 ? 3 * slots : 1);
    target = target < 4096 ? 4096 : (target > 49152 ? 49152 : target);
    struct Cand
    {
        long long cost;
        QItem item;
        int fit; // most columns an item of this matrix may have
    };
    std::vector<Cand> cand;
    for (size_t t = 0; t < shapes.size(); ++t)
    {
        const long long M = shapes[t].first, N = shapes[t].second;
        if (M <= 0 || N <= 0)
            continue;
        const long long Q = (M * bits + 31) / 32;
        // the owner kernel stages its packed sources in shared memory if an item is narrow enough for that
        int fit = stream_max_cols(Q, packedSources);
        if (fit < 1)
            fit = stream_max_cols(Q);
        const long long c = nice_cols((double) target / (double) M, (int) std::min<long long>(fit, N));
        for (long long c0 = 0; c0 < N; c0 += c)
        {
            const int n = (int) (c < N - c0 ? c : N - c0);
            cand.push_back(Cand{M * n, QItem{(int) t, (int) c0, n}, fit});
        }
    }
    std::stable_sort(cand.begin(), cand.end(), [](const Cand& x, const Cand& y) { return x.cost > y.cost; });
    out.clear();
    long long done = 0;
    for (const Cand& cd : cand)
    {
        const bool split = done * 4 >= total * 3 && cd.item.ncols >= 2;
        done += cd.cost;
        if (!split)
        {
            out.push_back(cd.item);
            continue;
        }
        const int piece = nice_cols(cd.item.ncols / 4.0, cd.item.ncols);
        for (int c0 = 0; c0 < cd.item.ncols; c0 += piece)
            out.push_back(QItem{cd.item.tensor, cd.item.col0 + c0, piece < cd.item.ncols - c0 ? piece : cd.item.ncols - c0});
    }
}

cudaError_t launch_stream1(cudaStream_t st, bool stripes, const QTensor* tensors, const QItem* items, int nItems,
                           const LaunchCfg& cfg, unsigned* counters, const Signal* signalp)
{
    static const Signal none = {};
    const Signal& signal = signalp ? *signalp : none;
    if (!counters)
        return cudaErrorInvalidValue;
    if (nItems <= 0)
        return signal.n > 0 ? launch_signal_only(st, signal) : cudaSuccess;
    int grid = cfg.numSMs * ST_CTAS_PER_SM;
    if (grid > nItems)
        grid = nItems;
    cudaError_t e;
    if (stripes)
    {
        e = cudaFuncSetAttribute(k_stream1<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) ST_SMEM_BYTES);
        if (e != cudaSuccess)
            return e;
        k_stream1<true><<<grid, NT, ST_SMEM_BYTES, st>>>(tensors, items, nItems, counters, signal);
    }
    else
    {
        e = cudaFuncSetAttribute(k_stream1<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) ST_SMEM_BYTES);
        if (e != cudaSuccess)
            return e;
        k_stream1<false><<<grid, NT, ST_SMEM_BYTES, st>>>(tensors, items, nItems, counters, signal);
    }
    return cudaGetLastError();
}

cudaError_t launch_materialize(cudaStream_t st, const float* buf, const float* lv, float* dst, long long M, long long N, int numSMs)
{
    if (M <= 0 || N <= 0)
        return cudaSuccess;
    long long blocks = (M * N + 255) / 256;
    if (blocks > (long long) numSMs * 8)
        blocks = (long long) numSMs * 8;
    k_materialize<<<(int) blocks, 256, 0, st>>>(buf, lv, dst, M, N);
    return cudaGetLastError();
}

} // namespace qagg
