// qagg_owner.cu -- the stripe owner's reduce-requantize (AllReduceDistGradAggregator.h:366-375, 405-435) for 1 bit with
// threshold 0, in two phases.
//
// For every column the owner has to (a) add the K unpacked stripes in source order, (b) add the stripe residual,
// (c) take the two level sums IN ROW ORDER to get the column's range, (d) emit bits and the new residual.  With the
// residual kept in deferred form (qagg_internal.h) neither the bits nor the stored state depend on the range, so only
// the column's 8-byte header does -- and only step (c) is serial.  The two are therefore separate kernels:
//
//   k_owner_form   everything that is parallel.  Thread <-> (column, packed word, half of the word's 32 rows): it reads the
//                  K source words once, the 16 previous-state values of its rows (rows w + kQ: for a fixed k the warp reads
//                  128 consecutive bytes), forms v = sum of sources + (prev - level(prev)), stores v, and stores its 16
//                  result bits as one 16-bit half of the packed word -- straight into this rank's gather slot and into
//                  every peer's.  No shared memory, no barrier; warps take 32-word units u, u + warps, ...
//                  It also counts each column's rows with v >= 0 and flags NaNs (integers: no order needed).
//   k_owner_walk   the serial part, nothing else.  One CTA = a producer warp and two walking warps (one per level); a work
//                  item is 32 adjacent columns, lane <-> column.  The producer brings tiles of 252 rows x 32 columns of
//                  the just-written state (mostly still in L2) into a 6-slot ring with one tensor copy each; both walkers
//                  add min(v, 0) resp. max(v, 0) down their lane's tile column.  All columns of all owned stripes walk
//                  concurrently, every walking warp has up to 32 active lanes, and the launch lasts as long as the tallest
//                  column's add chain (about 4.4 cycles per row).  At the end: range, header (to all gather slots), the
//                  new reconstruction values, and the release of the peers' flags by the last CTA.
//
// The kernel this replaces kept whole columns resident in shared memory and walked them with two one-lane warps per CTA
// while the other 254 threads waited at a barrier; at 8 ranks it ran at 0.09 of the HBM roofline.
// Other modes (mean threshold, 2..32 bits) cannot defer anything and keep the resident-column kernel.
#include "qagg_async.cuh"

#include <algorithm>

namespace qagg {

constexpr int OW_HALF = 16;   // rows (field positions) per thread
constexpr int OW_SRC = 4;     // packed sources fetched per batch
constexpr int OW_R = 252;     // tile rows: 4 x an odd number, so that the 128-bit reads of neighbouring tile columns fall
                              // into distinct banks (the tile is dense: column stride = OW_R floats); at most 256 (copy box)
constexpr int OW_C = 32;      // tile columns = lanes of a walking warp
constexpr int OW_STAGES = 6;  // ring slots: a walking warp drains a tile in about 0.6 us, a tensor copy takes a few times that
constexpr int OW_TILE_FLOATS = OW_R * OW_C;
constexpr int OW_THREADS = 96;
constexpr size_t OW_SMEM_BYTES = (size_t) OW_STAGES * OW_TILE_FLOATS * 4;

long long owner_form_units(long long M, long long n)
{
    if (M <= 0 || n <= 0)
        return 0;
    const long long Q = (M + 31) / 32;
    return 2 * ((n * Q + 31) / 32);
}

// where a unit's lane works: table entry, column, word, first field position
struct FormCtx
{
    const QTensor* T;
    unsigned c, w, kb, col0;
    bool live, full; // full: all OW_HALF rows of this lane exist (no per-row checks needed)
};

__device__ __forceinline__ FormCtx form_locate(const QTensor* __restrict__ tensors, int nTensors, long long u, int& cur, unsigned lane)
{
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
    FormCtx x;
    x.T = tensors + cur;
    const unsigned M = (unsigned) x.T->M;
    const unsigned Q = (unsigned) x.T->Q;
    const unsigned long long local = (unsigned long long) (u - x.T->unit0);
    x.kb = (unsigned) (local & 1ull) * OW_HALF;          // this unit's rows are field positions kb .. kb + 15
    const unsigned long long t0 = (local >> 1) * 32ull;  // first word of the unit, columns laid end to end
    const unsigned long long totalWords = (unsigned long long) x.T->N * Q;
    unsigned w0;
    if (totalWords <= 0xffffffffull)
    {
        x.col0 = (unsigned) t0 / Q;
        w0 = (unsigned) t0 - x.col0 * Q;
    }
    else
    {
        x.col0 = (unsigned) (t0 / Q);
        w0 = (unsigned) (t0 - (unsigned long long) x.col0 * Q);
    }
    x.live = t0 + lane < totalWords;
    const unsigned tl = w0 + lane;
    const unsigned dc = tl / Q;
    x.c = x.live ? x.col0 + dc : x.col0;
    x.w = x.live ? tl - dc * Q : 0u;
    x.full = x.live && (x.w + (x.kb + OW_HALF - 1) * Q < M);
    return x;
}

// The unit's previous-state values go into flight: 4-byte asynchronous copies into the warp's staging buffer, slot
// [k][lane] for row k of this lane.  A lane reads back only what it copied itself, so waiting for its own copy groups is
// all the synchronisation needed.
__device__ __forceinline__ void form_stage_prev(const FormCtx& x, float* __restrict__ buf, unsigned lane)
{
    if (x.live)
    {
        const unsigned M = (unsigned) x.T->M, Q = (unsigned) x.T->Q;
        const float* __restrict__ p = x.T->res_in + (size_t) x.c * M + x.w + (size_t) x.kb * Q;
        const unsigned dst = smem_addr(buf + lane);
#pragma unroll
        for (int k = 0; k < OW_HALF; ++k)
            if (x.full || x.w + (x.kb + k) * Q < M)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + (unsigned) k * 128u), "l"(p + (size_t) k * Q) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory"); // every lane commits, with or without copies: the group counts stay in step
}

__device__ __forceinline__ void form_unit(const FormCtx& x, const float* __restrict__ buf, const Signal& signal, unsigned lane)
{
    const QTensor* __restrict__ Tp = x.T;
    const unsigned M = (unsigned) Tp->M, Q = (unsigned) Tp->Q;
    const unsigned c = x.c, w = x.w, kb = x.kb;
    unsigned bitsOut = 0u;
    float nanSum = 0.0f;
    if (x.live)
    {
        const size_t colOff = (size_t) c * M + w + (size_t) kb * Q;
        float* __restrict__ outp = Tp->res_out + colOff;
        const bool selfRaw = Tp->selfRaw != 0;
        const int nsrc = Tp->nsrc;
        const size_t colBytes = (size_t) Tp->colBytes;
        const float lv0 = Tp->lv[2 * (size_t) c], lv1 = Tp->lv[2 * (size_t) c + 1];
        float agg[OW_HALF];
        // the K sources in index order (the own stripe first), the residual last (AllReduceDistGradAggregator.h:366-375, 405-435)
        if (selfRaw)
        {
            const float* __restrict__ rawp = Tp->grad + colOff;
#pragma unroll
            for (int k = 0; k < OW_HALF; ++k)
                agg[k] = (x.full || w + (kb + k) * Q < M) ? __ldcs(rawp + (size_t) k * Q) : 0.0f;
        }
        else
        {
            // the first packed source starts the sum (the reference unquantizes it with add = false)
            const unsigned char* colp = Tp->src[0] + (size_t) c * colBytes;
            float v0, v1;
            levels_1bit(__ldg(reinterpret_cast<const float*>(colp)), __ldg(reinterpret_cast<const float*>(colp) + 1), v0, v1);
            const unsigned word = __ldg(reinterpret_cast<const unsigned*>(colp + 8) + w) >> kb;
#pragma unroll
            for (int k = 0; k < OW_HALF; ++k)
                agg[k] = (word & (1u << k)) ? v1 : v0;
        }
        for (int s = 1; s < nsrc; s += OW_SRC)
        {
            unsigned sw[OW_SRC];
            float sv0[OW_SRC], sv1[OW_SRC];
#pragma unroll
            for (int j = 0; j < OW_SRC; ++j)
            {
                // a source index past the end re-reads the last source; its result is discarded below
                const unsigned char* colp = Tp->src[min(s + j, nsrc - 1)] + (size_t) c * colBytes;
                sv0[j] = __ldg(reinterpret_cast<const float*>(colp));
                sv1[j] = __ldg(reinterpret_cast<const float*>(colp) + 1);
                sw[j] = __ldg(reinterpret_cast<const unsigned*>(colp + 8) + w) >> kb;
            }
#pragma unroll
            for (int j = 0; j < OW_SRC; ++j)
            {
                if (s + j < nsrc) // uniform over the warp's live lanes of one table entry
                {
                    float v0, v1;
                    levels_1bit(sv0[j], sv1[j], v0, v1);
#pragma unroll
                    for (int k = 0; k < OW_HALF; ++k)
                        agg[k] = __fadd_rn((sw[j] & (1u << k)) ? v1 : v0, agg[k]);
                }
            }
        }
        if (x.full)
        {
#pragma unroll
            for (int k = 0; k < OW_HALF; ++k)
            {
                const float v = __fadd_rn(agg[k], deferred_residual(buf[k * 32 + lane], lv0, lv1));
                outp[(size_t) k * Q] = v; // read again by the walk kernel: a plain store, so that it stays in L2
                bitsOut |= (v >= 0.0f) ? (1u << k) : 0u;
                nanSum = __fadd_rn(nanSum, v);
            }
        }
        else
        {
#pragma unroll
            for (int k = 0; k < OW_HALF; ++k)
            {
                if (w + (kb + k) * Q < M)
                {
                    const float v = __fadd_rn(agg[k], deferred_residual(buf[k * 32 + lane], lv0, lv1));
                    outp[(size_t) k * Q] = v;
                    bitsOut |= (v >= 0.0f) ? (1u << k) : 0u;
                    nanSum = __fadd_rn(nanSum, v);
                }
            }
        }
        // this half of the packed word, to this rank's gather slot and to every peer's
        unsigned char* const dst = Tp->pk[0] + (size_t) c * colBytes;
        const size_t wordOff = 8 + 4 * (size_t) w + (kb ? 2 : 0);
        *reinterpret_cast<unsigned short*>(dst + wordOff) = (unsigned short) bitsOut;
        if (Tp->bcast)
        {
            const size_t off = (size_t) (dst - Tp->pk[0]) + (size_t) Tp->bcastOff + wordOff;
            for (int b = 0; b < signal.nbcast; ++b)
                *reinterpret_cast<unsigned short*>(signal.bcastBase[b] + off) = (unsigned short) bitsOut;
        }
    }
    // per-column count of rows with v >= 0: one atomic per warp when the warp lies inside one column
    const unsigned ones = __popc(bitsOut);
    unsigned* __restrict__ stats = Tp->stats;
    const bool oneColumn = __all_sync(0xffffffffu, !x.live || c == x.col0);
    if (oneColumn)
    {
        const unsigned tot = __reduce_add_sync(0xffffffffu, ones);
        if (lane == 0 && tot)
            atomicAdd(&stats[2 * (size_t) x.col0], tot);
    }
    else if (x.live && ones)
    {
        atomicAdd(&stats[2 * (size_t) c], ones);
    }
    // a NaN among the values shows in their running sum (so does a pair of opposite infinities, whose column range is NaN
    // in the reference as well: its level means are then infinities of opposite sign)
    if (x.live && nanSum != nanSum)
        atomicOr(&stats[2 * (size_t) c + 1], 1u);
}

// Warps take units u, u + warps, ...  The previous-state values of a warp's next two units are already on their way into
// its three staging buffers while it works on the current one, so the memory latency overlaps the arithmetic without
// holding registers (the loop is unrolled by three so that every buffer and context has a fixed name).
constexpr int FORM_BUF_FLOATS = OW_HALF * 32;
__global__ void __launch_bounds__(NT, 3) k_owner_form(const QTensor* __restrict__ tensors, int nTensors, long long unitBegin, long long totalUnits,
                                                     const Signal signal)
{
    // this launch covers units [unitBegin, totalUnits) of the table
    __shared__ __align__(16) float sStage[NWARPS][3][FORM_BUF_FLOATS];
    const unsigned lane = threadIdx.x & 31;
    const unsigned warp = threadIdx.x >> 5;
    const long long gwarp = unitBegin + (long long) blockIdx.x * NWARPS + warp;
    const long long nwarps = (long long) gridDim.x * NWARPS;
    if (gwarp >= totalUnits)
        return;
    int cur = 0;
    float* const b0 = sStage[warp][0];
    float* const b1 = sStage[warp][1];
    float* const b2 = sStage[warp][2];
    FormCtx x0, x1, x2;
    // units of this warp: u0 = gwarp, then + nwarps each; `have` says whether the unit exists
    long long u = gwarp;
    x0 = form_locate(tensors, nTensors, u, cur, lane);
    form_stage_prev(x0, b0, lane);
    bool have1 = u + nwarps < totalUnits;
    if (have1)
        x1 = form_locate(tensors, nTensors, u + nwarps, cur, lane);
    else
        x1 = x0, x1.live = false;
    form_stage_prev(x1, b1, lane);
    for (;;)
    {
        // ---- current x0, next x1, staging x2 ----
        bool have2 = u + 2 * nwarps < totalUnits;
        if (have2)
            x2 = form_locate(tensors, nTensors, u + 2 * nwarps, cur, lane);
        else
            x2 = x0, x2.live = false;
        form_stage_prev(x2, b2, lane);
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        form_unit(x0, b0, signal, lane);
        if (!have1)
            break;
        u += nwarps;
        // ---- current x1, next x2, staging x0 ----
        bool have0 = u + 2 * nwarps < totalUnits;
        if (have0)
            x0 = form_locate(tensors, nTensors, u + 2 * nwarps, cur, lane);
        else
            x0 = x1, x0.live = false;
        form_stage_prev(x0, b0, lane);
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        form_unit(x1, b1, signal, lane);
        if (!have2)
            break;
        u += nwarps;
        // ---- current x2, next x0, staging x1 ----
        have1 = u + 2 * nwarps < totalUnits;
        if (have1)
            x1 = form_locate(tensors, nTensors, u + 2 * nwarps, cur, lane);
        else
            x1 = x2, x1.live = false;
        form_stage_prev(x1, b1, lane);
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        form_unit(x2, b2, signal, lane);
        if (!have0)
            break;
        u += nwarps;
        // the roles are back where they started: x0 current, x1 next
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// one walking warp's pass over the tiles of an item: full tiles with the unrolled walk, the last (partial) one generally
template <int KIND>
__device__ __forceinline__ float walk_item(const float* tiles, unsigned long long* sFull, unsigned long long* sEmpty, unsigned* sBroken, unsigned* status,
                                           unsigned pos, int ntiles, int M, bool active, int lane)
{
    float acc = 0.0f;
    for (int q = 0; q < ntiles; ++q)
    {
        const unsigned p = pos + (unsigned) q;
        const unsigned slot = p % OW_STAGES;
        mbar_wait(&sFull[slot], (p / OW_STAGES) & 1u, sBroken, status, ST_WAIT_TRIES, 20);
        if (active && !*reinterpret_cast<volatile unsigned*>(sBroken))
        {
            // rows past the end of the matrix are zero-filled, but a partial tile is walked only as far as the matrix goes
            const float* vcol = tiles + slot * OW_TILE_FLOATS + lane * OW_R;
            const int nrows = M - q * OW_R;
            acc = (nrows >= OW_R) ? walk_tile<KIND, OW_R>(vcol, acc) : walk_chunk<KIND>(vcol, nrows, acc);
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive(&sEmpty[slot]);
    }
    return acc;
}

__global__ void __launch_bounds__(OW_THREADS, 1) k_owner_walk(const QTensor* __restrict__ tensors, const QItem* __restrict__ items, int nItems,
                                                           const Signal signal, unsigned* __restrict__ counters, unsigned* __restrict__ status,
                                                           int doneSlot, unsigned nLaunches)
{
    extern __shared__ __align__(128) float tiles[];
    __shared__ __align__(8) unsigned long long sFull[OW_STAGES], sEmpty[OW_STAGES];
    __shared__ unsigned sBroken;
    __shared__ float sA[2][2][OW_C]; // [item parity][level][column]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0)
    {
        for (int i = 0; i < OW_STAGES; ++i)
        {
            mbar_init(&sFull[i], 1u);
            mbar_init(&sEmpty[i], 2u); // both walking warps hand a slot back
        }
        sBroken = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    unsigned pos = 0; // ring position of the current item's tile 0 (all warps keep the same count)
    unsigned itemNo = 0;
    // Items are sorted tallest first and dealt out in rounds, every other round in reverse CTA order: the CTAs that drew
    // the tallest items of one round get the shortest of the next (or none).
    for (;; ++itemNo)
    {
        const int it = (int) (itemNo * gridDim.x + ((itemNo & 1u) ? gridDim.x - 1u - blockIdx.x : blockIdx.x));
        if (it >= nItems)
            break;
        const QItem item = items[it];
        const QTensor* __restrict__ Tp = tensors + item.tensor;
        const int M = (int) Tp->M;
        const int col0 = item.col0, nc = item.ncols;
        const void* const tmap = Tp->tm[0][1];
        const int ntiles = tmap ? (M + OW_R - 1) / OW_R : 0;
        if (warp == 0)
        {
            // ================================ producer ================================
            for (int q = 0; q < ntiles; ++q)
            {
                const unsigned p = pos + (unsigned) q;
                const unsigned slot = p % OW_STAGES;
                if (p >= (unsigned) OW_STAGES)
                    mbar_wait(&sEmpty[slot], ((p / OW_STAGES) - 1u) & 1u, &sBroken, status);
                if (*reinterpret_cast<volatile unsigned*>(&sBroken))
                    break;
                if (lane == 0)
                {
                    // the whole box counts, whether or not part of it lies outside the matrix (that part is zero-filled)
                    mbar_arrive_expect_tx(&sFull[slot], (unsigned) (OW_TILE_FLOATS * 4));
                    tensor_load_2d(tiles + slot * OW_TILE_FLOATS, tmap, q * OW_R, col0, &sFull[slot]);
                }
            }
        }
        else
        {
            // ================================ walkers: warp 1 = lower level, warp 2 = upper level ================================
            float acc = 0.0f;
            if (tmap)
            {
                // the two levels are two copies of the loop, so that each warp runs straight-line code for its own level
                if (warp == 1)
                    acc = walk_item<WALK_MIN0>(tiles, sFull, sEmpty, &sBroken, status, pos, ntiles, M, lane < nc, lane);
                else
                    acc = walk_item<WALK_MAX0>(tiles, sFull, sEmpty, &sBroken, status, pos, ntiles, M, lane < nc, lane);
            }
            else if (lane < nc)
            {
                // no tensor map (rows not a multiple of 4): the lane walks its column in global memory
                const float* __restrict__ vcol = Tp->res_out + (size_t) (col0 + lane) * (size_t) M;
                for (int i = 0; i < M; ++i)
                {
                    const float v = __ldcg(vcol + i);
                    acc = __fadd_rn(acc, (warp == 1) ? fminf(v, 0.0f) : fmaxf(v, 0.0f));
                }
            }
            if (lane < nc)
                sA[itemNo & 1][warp - 1][lane] = acc;
            asm volatile("bar.sync 1, 64;" ::: "memory"); // the two walking warps
            if (warp == 1 && lane < nc)
            {
                const size_t j = (size_t) (col0 + lane);
                unsigned* __restrict__ stats = Tp->stats;
                const unsigned ones = stats[2 * j], nanFlag = stats[2 * j + 1];
                stats[2 * j] = 0u; // re-armed for the next step
                stats[2 * j + 1] = 0u;
                // rows below the threshold = rows whose bit is 0 (a NaN row has bit 0 too, but then the range is NaN whatever
                // the count); min/max drop a NaN where the reference adds it to the upper sum: put it back
                float lo, up, v0, v1;
                finalize_range<MODE_ONEBIT_ZERO>(sA[itemNo & 1][0][lane], nanFlag ? __int_as_float(0x7fc00000) : sA[itemNo & 1][1][lane],
                                                 (unsigned) M - ones, 0.0f, Tp->M, lo, up);
                levels_1bit(lo, up, v0, v1);
                Tp->lv[2 * j] = v0;
                Tp->lv[2 * j + 1] = v1;
                unsigned char* const dst = Tp->pk[0] + j * (size_t) Tp->colBytes;
                store_header(dst, lo, up);
                if (Tp->bcast)
                {
                    const size_t off = (size_t) (dst - Tp->pk[0]) + (size_t) Tp->bcastOff;
                    for (int b = 0; b < signal.nbcast; ++b)
                        store_header(signal.bcastBase[b] + off, lo, up);
                }
            }
        }
        pos += (unsigned) ntiles;
    }
    __syncthreads();
    // The last CTA to leave releases the peers' flags: each CTA's stores (into peer memory too) are ordered before its
    // arrival by barrier + system-scope fence; the form kernel's stores were complete before this kernel began.  When the
    // owner's work is split over nLaunches concurrent walk launches, the last CTA of each arrives at a second counter and
    // the last of those releases.
    if (tid == 0)
    {
        __threadfence_system();
        const unsigned done = atomicAdd(&counters[doneSlot], 1u);
        if (done == gridDim.x - 1)
        {
            counters[doneSlot] = 0;
            bool last = true;
            if (nLaunches > 1u)
            {
                __threadfence();
                last = (atomicAdd(&counters[3], 1u) == nLaunches - 1u);
                if (last)
                    counters[3] = 0;
            }
            if (last)
                release_flags(signal);
        }
    }
}

// ---- host side -------------------------------------------------------------------------------------------------------

void owner_make_items(const std::vector<std::pair<long long, long long>>& shapes, std::vector<QItem>& out)
{
    struct Cand
    {
        long long rows;
        QItem item;
    };
    std::vector<Cand> cand;
    for (size_t e = 0; e < shapes.size(); ++e)
    {
        const long long M = shapes[e].first, n = shapes[e].second;
        if (M <= 0 || n <= 0)
            continue;
        for (long long c0 = 0; c0 < n; c0 += OW_C)
            cand.push_back(Cand{M, QItem{(int) e, (int) c0, (int) std::min<long long>(OW_C, n - c0)}});
    }
    // tallest columns first: a launch lasts as long as its longest walk
    std::stable_sort(cand.begin(), cand.end(), [](const Cand& x, const Cand& y) { return x.rows > y.rows; });
    out.clear();
    for (const Cand& cd : cand)
        out.push_back(cd.item);
}

bool owner_set_map(QTensor* t, unsigned char* hostMap, unsigned char* devMap)
{
    const bool ok = (reinterpret_cast<uintptr_t>(devMap) & 127) == 0 && encode_map_2d(hostMap, t->res_out, t->M, t->N, OW_R, OW_C);
    t->tm[0][0] = nullptr;
    t->tm[0][1] = ok ? devMap : nullptr;
    t->tm[1][0] = t->tm[1][1] = nullptr;
    return ok;
}

// grid of the form kernel: at most three CTAs per SM; among the sizes from two to three per SM, the one whose warps share
// the units most evenly
static int form_grid(long long totalUnits, int numSMs)
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

cudaError_t launch_owner(cudaStream_t st, const QTensor* tensors, int nTensors, long long formUnits, const QItem* items, int nItems,
                         const LaunchCfg& cfg, unsigned* counters, const Signal* signalp, unsigned* status, const OwnerSplit* split, cudaEvent_t afterForm)
{
    static const Signal none = {};
    const Signal& signal = signalp ? *signalp : none;
    if (!counters)
        return cudaErrorInvalidValue;
    if (nItems <= 0 || formUnits <= 0)
        return signal.n > 0 ? launch_signal_only(st, signal) : cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(k_owner_walk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) OW_SMEM_BYTES);
    if (e != cudaSuccess)
        return e;
    const int tallGrid = split ? std::min(split->tallItems, cfg.numSMs) : 0;
    if (split && split->tallItems > 0 && split->tallItems < nItems && split->tallUnits > 0 && split->tallUnits < formUnits && 8 * tallGrid <= cfg.numSMs)
    {
        // (Taken only when the tall walk needs few SMs: with many tall items -- 2 ranks on the speech set -- the form work
        // dominates and one launch of each kind measured faster.)
        // Tall matrices first: their walk is the longest dependent chain of the step, so it starts as early as possible, and
        // the other matrices are formed and walked beside it, on a second stream, on the SMs it leaves free (one walk CTA
        // fills an SM's shared memory, so the launches that run beside it are sized for the remaining SMs).  The tall walk
        // stays on `st`, right behind the form launch it depends on: a same-stream successor starts before work that waits
        // for an event, and the launches beside it must not take its SMs first.
        const int restSMs = cfg.numSMs - tallGrid;
        k_owner_form<<<form_grid(split->tallUnits, cfg.numSMs), NT, 0, st>>>(tensors, nTensors, 0, split->tallUnits, signal);
        if ((e = cudaGetLastError()) != cudaSuccess || (e = cudaEventRecord(split->fork, st)) != cudaSuccess)
            return e;
        k_owner_walk<<<tallGrid, OW_THREADS, OW_SMEM_BYTES, st>>>(tensors, items, split->tallItems, signal, counters, status, 1, 2u);
        if ((e = cudaGetLastError()) != cudaSuccess || (e = cudaStreamWaitEvent(split->side, split->fork, 0)) != cudaSuccess)
            return e;
        k_owner_form<<<form_grid(formUnits - split->tallUnits, restSMs), NT, 0, split->side>>>(tensors, nTensors, split->tallUnits, formUnits, signal);
        if ((e = cudaGetLastError()) != cudaSuccess)
            return e;
        const int restItems = nItems - split->tallItems;
        k_owner_walk<<<std::min(restItems, restSMs), OW_THREADS, OW_SMEM_BYTES, split->side>>>(tensors, items + split->tallItems, restItems, signal, counters,
                                                                                               status, 2, 2u);
        if ((e = cudaGetLastError()) != cudaSuccess || (e = cudaEventRecord(split->join, split->side)) != cudaSuccess)
            return e;
        return cudaStreamWaitEvent(st, split->join, 0);
    }
    k_owner_form<<<form_grid(formUnits, cfg.numSMs), NT, 0, st>>>(tensors, nTensors, 0, formUnits, signal);
    if ((e = cudaGetLastError()) != cudaSuccess)
        return e;
    if (afterForm && (e = cudaEventRecord(afterForm, st)) != cudaSuccess)
        return e;
    int grid = cfg.numSMs; // one CTA per SM: the ring takes most of an SM's shared memory
    if (grid > nItems)
        grid = nItems;
    k_owner_walk<<<grid, OW_THREADS, OW_SMEM_BYTES, st>>>(tensors, items, nItems, signal, counters, status, 1, 1u);
    return cudaGetLastError();
}

} // namespace qagg
