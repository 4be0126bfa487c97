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
// One work item = nc <= 32 adjacent columns of one matrix, processed in chunks of R rows (nc * R <= 1536 values).
// The CTA's nine warps have three roles:
//   * one "producer" warp fetches work items from the queue and brings every chunk's inputs global -> shared with ONE
//     tensor copy per input (cp.async.bulk.tensor through a tensor map of the matrix: box = R rows x nc columns; an
//     mbarrier per ring slot counts the bytes), as far ahead as the input ring has free slots -- across item
//     boundaries too, so the consumers never wait for a pipeline to refill;
//   * six "element" warps form v = gradient + (prev - level(prev)), store v to global memory and to a padded tile for the walkers, and OR the bit (v >= 0) into the item's packed
//     words, which live in shared memory until the item ends;
//   * two "walker" warps (one per level, lane = column) add min(v, 0) resp. max(v, 0) of the previous chunk to their
//     running sums, in row order;
//   * at the end the ranges and the new reconstruction values are derived and the packed columns go to their owners.
// Every wait on an mbarrier is bounded: if one runs out, the CTA stops waiting altogether, bit 1 of the status word
// is set and the kernel ends normally (the results of that launch are then invalid).
// Matrices whose columns are not 16-byte aligned have no tensor maps; their chunks are fetched with plain loads.
#include "qagg_async.cuh"

#include <cuda.h>

#include <algorithm>
#include <cstring>

namespace qagg {

constexpr int ST_WALK_WARPS = 2;
constexpr int ST_ETHREADS = NT - 32 * ST_WALK_WARPS;   // 192 element threads
constexpr int ST_U = 2;                                // 16-byte positions per element thread and chunk
constexpr int ST_TILE_VALUES = 4 * ST_U * ST_ETHREADS; // 1536 values per chunk
constexpr int ST_IN_FLOATS = ST_TILE_VALUES;           // input tile: dense box, column stride R
constexpr int ST_V_FLOATS = ST_TILE_VALUES + 4 * QAGG_STREAM_CMAX; // walkers' tile: column stride R + 4
constexpr int ST_CTAS_PER_SM = 3;
constexpr int ST_IN_STAGES = 4; // input ring slots: one being formed, the others in flight
constexpr size_t ST_SMEM_BYTES = (size_t) (2 * ST_IN_STAGES * ST_IN_FLOATS + 2 * ST_V_FLOATS + QAGG_STREAM_PKWORDS) * 4;

// rows per chunk for a tile geometry of `boxCols` columns: a multiple of 32 (so that the walkers' tile, whose column
// stride is R + 4, spreads the 128-bit reads of neighbouring columns over distinct banks), at most 256 (tensor copy box)
__host__ __device__ __forceinline__ int stream_rows(int boxCols)
{
    const int r = ((ST_TILE_VALUES / boxCols) >> 5) << 5;
    return r > 256 ? 256 : r;
}

constexpr int ST_DESC = 4; // work items whose descriptors may be fetched ahead of the consumers

// barrier of the eight consumer warps (the producer warp does not take part)
__device__ __forceinline__ void consumer_sync()
{
    asm volatile("bar.sync 1, 256;" ::: "memory");
}

// which of a descriptor's two tile geometries an item of `ncols` columns uses (the same answer on both sides of the ring)
__device__ __forceinline__ int stream_geometry(const QTensor& T, int ncols)
{
    return (T.boxCols[1] > 0 && ncols <= T.boxCols[1]) ? 1 : 0;
}

__global__ void __launch_bounds__(NT + 32, ST_CTAS_PER_SM) k_stream1(const QTensor* __restrict__ tensors, const QItem* __restrict__ items, int nItems,
                                                                     unsigned* __restrict__ counters, const Signal signal, unsigned* __restrict__ status)
{
    constexpr int SIN = ST_IN_STAGES;
    extern __shared__ __align__(128) float dsm[];
    float* const inG = dsm;                                  // input ring: gradient boxes
    float* const inP = dsm + SIN * ST_IN_FLOATS;             // input ring: previous-state boxes
    float* const vt = dsm + 2 * SIN * ST_IN_FLOATS;          // the formed values of two chunks: one being walked, one being written
    // the item's packed words (nc x Q)
    unsigned* const pkw = reinterpret_cast<unsigned*>(dsm + 2 * SIN * ST_IN_FLOATS + 2 * ST_V_FLOATS);
    // work items in flight: buffer (n % ST_DESC) holds the CTA's n-th item: its queue index (>= nItems: the queue is
    // empty), the item and its matrix descriptor
    __shared__ QTensor sT[ST_DESC];
    __shared__ QItem sItem[ST_DESC];
    __shared__ int sIt[ST_DESC];
    // sFull[slot]: the chunk's inputs have landed (producer's arrival + byte count).  sEmpty[slot]: the element warps have
    // formed the chunk.  sMetaFull[b]: buffer b describes the next item.  sMetaEmpty[b]: the consumers are done with it.
    __shared__ __align__(8) unsigned long long sFull[SIN], sEmpty[SIN], sMetaFull[ST_DESC], sMetaEmpty[ST_DESC];
    __shared__ unsigned sBroken;
    __shared__ int sWalker;
    __shared__ float sLv0[QAGG_STREAM_CMAX], sLv1[QAGG_STREAM_CMAX], sA0[QAGG_STREAM_CMAX], sA1[QAGG_STREAM_CMAX];
    __shared__ float sLower[QAGG_STREAM_CMAX], sUpper[QAGG_STREAM_CMAX];
    __shared__ unsigned sN0[QAGG_STREAM_CMAX], sNan[QAGG_STREAM_CMAX];
    __shared__ unsigned char* sDst[QAGG_STREAM_CMAX];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (blockIdx.x == 0 && tid < signal.hdrN)
    {
        // the step's header values ride along: into this rank's slot of every rank's window (ordered before the flag release
        // like every other store of this CTA)
        const double v = signal.hdrIn[tid];
        for (int p = 0; p < signal.hdrDstN; ++p)
            signal.hdrDst[p][tid] = v;
    }
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
        for (int i = 0; i < SIN; ++i)
        {
            mbar_init(&sFull[i], 1u);
            mbar_init(&sEmpty[i], 1u);
        }
        for (int i = 0; i < ST_DESC; ++i)
        {
            mbar_init(&sMetaFull[i], 1u);
            mbar_init(&sMetaEmpty[i], 1u);
        }
        sBroken = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (sIt[0] < nItems)
    {
        const int* srcw = reinterpret_cast<const int*>(tensors + sItem[0].tensor);
        int* dstw = reinterpret_cast<int*>(&sT[0]);
        for (int i = tid; i < (int) (sizeof(QTensor) / sizeof(int)); i += NT + 32)
            dstw[i] = srcw[i];
    }
    __syncthreads();
    if (tid == 0)
        mbar_arrive(&sMetaFull[0]); // the first item is published like every later one

    if (warp == NWARPS)
    {
        // =============================================== producer warp ===============================================
        unsigned pos = 0; // ring position of the current item's chunk 0
        for (unsigned itemNo = 0;; ++itemNo)
        {
            const int b = (int) (itemNo % ST_DESC);
            if (sIt[b] >= nItems || *reinterpret_cast<volatile unsigned*>(&sBroken))
                break;
            const QTensor& T = sT[b];
            const int M = (int) T.M, col0 = sItem[b].col0;
            const int geo = stream_geometry(T, sItem[b].ncols);
            const int boxCols = T.boxCols[geo];
            const void* const tmG = T.tm[geo][0];
            const void* const tmP = T.tm[geo][1];
            const bool vec = tmP != nullptr && tmG != nullptr;
            const int R = vec ? stream_rows(boxCols) : 1;
            const int nchunks = vec ? (M + R - 1) / R : 0;
            int issued = 0;
            // bring chunks [issued, upto) on their way, each as soon as its ring slot is free
            auto pump = [&](int upto) {
                for (; issued < upto; ++issued)
                {
                    const unsigned p = pos + (unsigned) issued;
                    const unsigned slot = p % SIN;
                    if (p >= (unsigned) SIN)
                        mbar_wait(&sEmpty[slot], ((p / SIN) - 1u) & 1u, &sBroken, status);
                    if (*reinterpret_cast<volatile unsigned*>(&sBroken))
                        return; // a wait ran out: nothing more is put in flight
                    if (lane == 0)
                    {
                        // the whole box counts, whether or not part of it lies outside the matrix (that part is zero-filled)
                        mbar_arrive_expect_tx(&sFull[slot], (unsigned) (2 * boxCols * R * 4));
                        tensor_load_2d(inG + slot * ST_IN_FLOATS, tmG, issued * R, col0, &sFull[slot]);
                        tensor_load_2d(inP + slot * ST_IN_FLOATS, tmP, issued * R, col0, &sFull[slot]);
                    }
                }
            };
            pump(min(nchunks, 2));
            // the item after this one: its queue index, the item and its descriptor (this warp may block on global
            // memory here -- the chunks above keep the consumers busy meanwhile)
            {
                const unsigned n1 = itemNo + 1u;
                const int b1 = (int) (n1 % ST_DESC);
                if (n1 >= ST_DESC)
                    mbar_wait(&sMetaEmpty[b1], ((n1 / ST_DESC) - 1u) & 1u, &sBroken, status);
                int nx = 0;
                if (lane == 0)
                    nx = (int) atomicAdd(&counters[0], 1u);
                nx = __shfl_sync(0xffffffffu, nx, 0);
                if (lane == 0)
                    sIt[b1] = nx;
                if (nx < nItems)
                {
                    const int word = (lane < 3) ? reinterpret_cast<const int*>(items + nx)[lane] : 0;
                    if (lane < 3)
                        reinterpret_cast<int*>(&sItem[b1])[lane] = word;
                    const int tIdx = __shfl_sync(0xffffffffu, word, 0);
                    const int* srcw = reinterpret_cast<const int*>(tensors + tIdx);
                    int* dstw = reinterpret_cast<int*>(&sT[b1]);
                    for (int i = lane; i < (int) (sizeof(QTensor) / sizeof(int)); i += 32)
                        dstw[i] = srcw[i];
                }
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&sMetaFull[b1]);
            }
            pump(nchunks);
            pos += (unsigned) nchunks;
        }
    }
    else
    {
        // ========================================= consumer warps (element + walker) =========================================
        const int ww = sWalker;
        const bool isWalker = (warp == ww) || (warp == ww + 1);
        const int firstElementWarp = (ww == 0) ? ST_WALK_WARPS : 0;
        const int et = ((warp > ww) ? warp - ST_WALK_WARPS : warp) * 32 + lane; // index among the element threads

        // ---- the item being streamed: geometry (uniform) and this thread's positions ----------------------------------------
        const QTensor* Tp = &sT[0];
        int M = 1, Q = 1, nc = 1, col0 = 0, R = 32, nchunks = 0;
        bool vec = false;
        const float* gbase = nullptr;
        const float* pbase = nullptr;
        float* obase = nullptr;
        unsigned advK = 0, advW = 0;
        unsigned pos = 0;                   // ring position of the item's chunk 0
        float lvReg0 = 0.0f, lvReg1 = 0.0f; // thread c < nc: the previous reconstruction values of column c, loaded ahead
        // An element thread owns the same ST_U 16-byte positions (column, four rows) of every chunk.  Row i of a column is
        // bit i / Q of packed word i % Q; the position's (word, bit) pair moves by a fixed step from chunk to chunk.
        bool pv[ST_U];
        int iofs[ST_U], vofs[ST_U], pcol[ST_U], prow[ST_U];
        size_t gofs[ST_U];
        unsigned pw[ST_U], pk[ST_U], nanf[ST_U];

        // wait for the CTA's n-th item to be described, and take it over unless the queue was empty
        auto adopt = [&](unsigned n) -> bool {
            const int b = (int) (n % ST_DESC);
            mbar_wait(&sMetaFull[b], (n / ST_DESC) & 1u, &sBroken, status);
            if (sIt[b] >= nItems || *reinterpret_cast<volatile unsigned*>(&sBroken))
                return false;
            Tp = &sT[b];
            const QTensor& T = *Tp;
            M = (int) T.M;
            Q = T.Q;
            nc = sItem[b].ncols;
            col0 = sItem[b].col0;
            const int geo = stream_geometry(T, nc);
            vec = T.tm[geo][1] != nullptr && T.tm[geo][0] != nullptr;
            R = stream_rows(vec ? T.boxCols[geo] : nc);
            nchunks = (M + R - 1) / R;
            gbase = T.grad;
            pbase = T.res_in;
            obase = T.res_out;
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
                iofs[u] = c * R + r;       // in the dense input box
                vofs[u] = c * (R + 4) + r; // in the walkers' tile
                gofs[u] = (size_t) (col0 + c) * (size_t) M + (size_t) r;
                pk[u] = (unsigned) r / (unsigned) Q;
                pw[u] = (unsigned) r - pk[u] * (unsigned) Q;
                nanf[u] = 0u;
            }
            if (tid < nc)
            {
                lvReg0 = T.lv[2 * (size_t) (col0 + tid)];
                lvReg1 = T.lv[2 * (size_t) (col0 + tid) + 1];
            }
            return true;
        };

        unsigned itemNo = 0;
        bool more = adopt(0u);
        while (more)
        {
            const QTensor& T = *Tp;
            const int vstride = R + 4;

            // ---- per-item state ----------------------------------------------------------------------------------------
            for (int i = tid; i < nc * Q; i += NT)
                pkw[i] = 0u;
            if (tid < nc)
            {
                sLv0[tid] = lvReg0;
                sLv1[tid] = lvReg1;
                sNan[tid] = 0u;
                sDst[tid] = packed_col(T, col0 + tid);
            }
            consumer_sync();

            auto form = [&](int q) {
                const int inOff = (int) ((pos + (unsigned) q) % SIN) * ST_IN_FLOATS;
                float* const vtile = vt + (q & 1) * ST_V_FLOATS;
                const int row0 = q * R;
#pragma unroll
                for (int u = 0; u < ST_U; ++u)
                {
                    const int row = row0 + prow[u];
                    if (pv[u] && row < M)
                    {
                        const int c = pcol[u];
                        const int nv = vec ? 4 : min(4, M - row);
                        float prev[4];
                        float agg[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (vec)
                        {
                            const float4 p4 = *reinterpret_cast<const float4*>(inP + inOff + iofs[u]);
                            prev[0] = p4.x;
                            prev[1] = p4.y;
                            prev[2] = p4.z;
                            prev[3] = p4.w;
                            const float4 g4 = *reinterpret_cast<const float4*>(inG + inOff + iofs[u]);
                            agg[0] = g4.x;
                            agg[1] = g4.y;
                            agg[2] = g4.z;
                            agg[3] = g4.w;
                        }
                        else
                        {
                            // matrices without tensor maps: plain loads
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                            {
                                prev[i] = (i < nv) ? pbase[gofs[u] + (size_t) row0 + i] : 0.0f;
                                agg[i] = (i < nv) ? gbase[gofs[u] + (size_t) row0 + i] : 0.0f;
                            }
                        }
                        const float lv0 = sLv0[c], lv1 = sLv1[c];
                        // the usual case: the four rows are the same bit of four adjacent words
                        const bool flat = (nv == 4) && (pw[u] + 3u < (unsigned) Q);
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
                                if (v[i] >= 0.0f)
                                    atomicOr(wp + i, m);
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                            {
                                const unsigned w = pw[u] + i;
                                const unsigned over = w / (unsigned) Q;
                                if (i < nv)
                                {
                                    nanf[u] |= (v[i] != v[i]) ? 1u : 0u;
                                    if (v[i] >= 0.0f)
                                        atomicOr(myWords + (w - over * (unsigned) Q), 1u << (pk[u] + over));
                                }
                            }
                        }
                        const float4 v4 = make_float4(v[0], v[1], v[2], v[3]);
                        *reinterpret_cast<float4*>(vtile + vofs[u]) = v4;
                        float* gout = obase + gofs[u] + (size_t) row0;
                        if (vec)
                        {
                            *reinterpret_cast<float4*>(gout) = v4;
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                if (i < nv)
                                    gout[i] = v[i];
                        }
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

            // ---- the chunk loop: in iteration q, chunk q's values are formed and chunk q - 1 is walked -----------------------
            float acc = 0.0f; // a walker lane's running sum of its column
            for (int q = 0; q <= nchunks; ++q)
            {
                if (!isWalker)
                {
                    if (vec && q >= 1 && warp == firstElementWarp && lane == 0)
                    {
                        // every element warp passed the last barrier: the input slot of chunk q - 1 may be refilled
                        mbar_arrive(&sEmpty[(pos + (unsigned) (q - 1)) % SIN]);
                    }
                    if (q < nchunks)
                    {
                        if (vec)
                        {
                            // one warp watches the mbarrier, the other element warps sleep at a hardware barrier meanwhile
                            const unsigned p = pos + (unsigned) q;
                            if (warp == firstElementWarp)
                                mbar_wait(&sFull[p % SIN], (p / SIN) & 1u, &sBroken, status);
                            asm volatile("bar.sync 2, %0;" ::"n"(ST_ETHREADS) : "memory");
                        }
                        form(q);
                    }
                }
                else if (q >= 1)
                {
                    if (lane < nc)
                    {
                        const int qq = q - 1;
                        const int nrows = min(R, M - qq * R);
                        const float* vcol = vt + (qq & 1) * ST_V_FLOATS + lane * vstride;
                        if (warp == ww)
                            acc = walk_chunk<WALK_MIN0>(vcol, nrows, acc);
                        else
                            acc = walk_chunk<WALK_MAX0>(vcol, nrows, acc);
                    }
                }
                consumer_sync(); // chunk q is formed (next: walked), chunk q - 1 is walked (its tile may be overwritten)
            }

            // ---- finish ------------------------------------------------------------------------------------------------------
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
            if (vec)
                pos += (unsigned) nchunks;
            // the next item's geometry and previous reconstruction values are fetched before this item's last steps
            more = adopt(itemNo + 1u);
            consumer_sync();
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
            consumer_sync();
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
            consumer_sync();
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
            consumer_sync(); // the item is done with its shared-memory state and with its descriptor buffer
            if (tid == 0)
                mbar_arrive(&sMetaEmpty[itemNo % ST_DESC]);
            ++itemNo;
        }
    }
    __syncthreads();

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
            release_flags(signal);
        }
    }
}

// One warp waits, with the streaming kernel's own bounded wait, for an mbarrier phase that nothing completes: the wait
// runs out after `maxTries` polls, sets bit 1 of *status, and the kernel ends normally.  A second wait then returns at
// once (the CTA-wide "broken" flag).  polls[0] / polls[1] receive the clock cycles the two waits took.
__global__ void k_stream_wait_selftest(int maxTries, unsigned* __restrict__ status, long long* __restrict__ cycles)
{
    __shared__ __align__(8) unsigned long long bar;
    __shared__ unsigned broken;
    if (threadIdx.x == 0)
    {
        mbar_init(&bar, 1u);
        broken = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const long long t0 = clock64();
    mbar_wait(&bar, 0u, &broken, status, maxTries);
    const long long t1 = clock64();
    mbar_wait(&bar, 0u, &broken, status, maxTries);
    const long long t2 = clock64();
    if (threadIdx.x == 0 && cycles)
    {
        cycles[0] = t1 - t0;
        cycles[1] = t2 - t1;
    }
}

cudaError_t launch_stream_wait_selftest(cudaStream_t st, int maxTries, unsigned* status, long long* cycles)
{
    k_stream_wait_selftest<<<1, 32, 0, st>>>(maxTries, status, cycles);
    return cudaGetLastError();
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

void stream_make_items(const std::vector<std::pair<long long, long long>>& shapes, int numSMs, int bits, std::vector<QItem>& out,
                       std::vector<std::pair<int, int>>& boxCols)
{
    boxCols.assign(shapes.size(), std::pair<int, int>(0, 0));
    long long total = 0;
    for (auto& sh : shapes)
        total += sh.first * sh.second;
    const long long slots = (long long) numSMs * ST_CTAS_PER_SM;
    long long target = total / (2 * slots > 0 ? 2 * slots : 1);
    // at most 24 K values per item: on the speech set 12-column items (128-row chunks) of the 2048-row matrices measured 5 %
    // faster than 24-column ones (64-row chunks), 16 columns the same as 24, 8 columns slower
    target = target < 4096 ? 4096 : (target > 24576 ? 24576 : target);
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
        const int fit = stream_max_cols(Q);
        // at least eight columns where the matrix has them: with fewer, a chunk has so many rows that the walkers' add
        // chains, not the memory system, set the pace
        const int most = (int) std::min<long long>(fit, N);
        const long long c = std::max(nice_cols((double) target / (double) M, most), std::min(8, most));
        boxCols[t].first = (int) c;
        // an item takes about as long as it has chunks, whatever its width: a single tall column is a long item
        const long long chunks = (M + stream_rows((int) c) - 1) / stream_rows((int) c);
        for (long long c0 = 0; c0 < N; c0 += c)
        {
            const int n = (int) (c < N - c0 ? c : N - c0);
            cand.push_back(Cand{chunks, QItem{(int) t, (int) c0, n}, fit});
        }
    }
    std::stable_sort(cand.begin(), cand.end(), [](const Cand& x, const Cand& y) { return x.cost > y.cost; });
    out.clear();
    total = 0;
    for (const Cand& cd : cand)
        total += cd.cost;
    long long done = 0;
    for (const Cand& cd : cand)
    {
        const bool split = done * 4 >= total * 3 && cd.item.ncols >= 16;
        done += cd.cost;
        if (!split)
        {
            out.push_back(cd.item);
            continue;
        }
        // one piece size per matrix (its items were all cut from full ones of the same width, but for the last)
        int piece = boxCols[cd.item.tensor].second;
        if (piece == 0)
        {
            piece = std::max(8, nice_cols(boxCols[cd.item.tensor].first / 3.0, boxCols[cd.item.tensor].first));
            if (piece >= boxCols[cd.item.tensor].first)
            {
                out.push_back(cd.item);
                continue;
            }
            boxCols[cd.item.tensor].second = piece;
        }
        for (int c0 = 0; c0 < cd.item.ncols; c0 += piece)
            out.push_back(QItem{cd.item.tensor, cd.item.col0 + c0, piece < cd.item.ncols - c0 ? piece : cd.item.ncols - c0});
    }
}

// ---- tensor maps ---------------------------------------------------------------------------------------------------------
// cuTensorMapEncodeTiled is a driver entry point; it is looked up at run time so that the library needs no link-time
// dependency on the driver library.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn tensor_map_encoder()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// map of a column-major M x N fp32 matrix with a box of boxRows rows x boxCols columns; false if it cannot be encoded
bool encode_map_2d(void* out128, const float* base, long long M, long long N, int boxRows, int boxCols)
{
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc || !base || M <= 0 || N <= 0 || (M & 3) || (reinterpret_cast<uintptr_t>(base) & 15) || boxRows < 1 || boxRows > 256 || boxCols < 1 ||
        boxCols > 256)
        return false;
    const cuuint64_t dims[2] = {(cuuint64_t) M, (cuuint64_t) N};
    const cuuint64_t strides[1] = {(cuuint64_t) M * 4};
    const cuuint32_t box[2] = {(cuuint32_t) boxRows, (cuuint32_t) boxCols};
    const cuuint32_t estr[2] = {1, 1};
    alignas(64) CUtensorMap m;
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return false;
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    std::memcpy(out128, &m, 128);
    return true;
}

void stream_set_maps(QTensor* t, unsigned char* hostMaps, unsigned char* devMaps)
{
    bool ok = (reinterpret_cast<uintptr_t>(t->res_out) & 15) == 0 && (reinterpret_cast<uintptr_t>(devMaps) & 127) == 0;
    for (int g = 0; g < 2 && ok; ++g)
    {
        if (t->boxCols[g] <= 0)
            continue;
        const int R = stream_rows(t->boxCols[g]);
        ok = ok && encode_map_2d(hostMaps + (2 * g) * 128, t->grad, t->M, t->N, R, t->boxCols[g]);
        ok = ok && encode_map_2d(hostMaps + (2 * g + 1) * 128, t->res_in, t->M, t->N, R, t->boxCols[g]);
    }
    for (int g = 0; g < 2; ++g)
    {
        const bool have = ok && t->boxCols[g] > 0;
        t->tm[g][0] = have ? devMaps + (2 * g) * 128 : nullptr;
        t->tm[g][1] = have ? devMaps + (2 * g + 1) * 128 : nullptr;
    }
}

cudaError_t launch_stream1(cudaStream_t st, const QTensor* tensors, const QItem* items, int nItems, const LaunchCfg& cfg, unsigned* counters,
                           const Signal* signalp, unsigned* status)
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
    cudaError_t e = cudaFuncSetAttribute(k_stream1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) ST_SMEM_BYTES);
    if (e != cudaSuccess)
        return e;
    k_stream1<<<grid, NT + 32, ST_SMEM_BYTES, st>>>(tensors, items, nItems, counters, signal, status);
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
