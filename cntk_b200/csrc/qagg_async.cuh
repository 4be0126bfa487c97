// qagg_async.cuh -- device helpers shared by the kernels that stream tiles through shared memory (qagg_stream.cu,
// qagg_owner.cu): mbarriers with BOUNDED waits, tensor copies (cp.async.bulk.tensor, never multicast, local memory only),
// the ordered walk over one tile column, and the deferred residual.
#pragma once

#include "qagg_device.cuh"

namespace qagg {

// ---- mbarriers and bulk asynchronous copies (addresses and sizes are multiples of 16 bytes) -----------------------------
__device__ __forceinline__ unsigned smem_addr(const void* p)
{
    return (unsigned) __cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// one non-blocking test: has the phase with this parity completed?
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity)
{
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_addr(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Bounded wait for the phase of `bar` with the given parity to complete.  After ST_WAIT_TRIES tries it gives up: the
// CTA-wide flag *broken makes every later wait return at once, and bit 1 of *status tells the host.
constexpr int ST_WAIT_TRIES = 1 << 22;
__device__ __forceinline__ void mbar_wait(unsigned long long* bar, unsigned parity, unsigned* broken, unsigned* status, int maxTries = ST_WAIT_TRIES,
                                          unsigned sleepNs = 128)
{
    if (mbar_try_wait(bar, parity))
        return;
    if (*reinterpret_cast<volatile unsigned*>(broken))
        return;
    // not there yet: poll with the warp asleep in between, so that the waiting costs the other warps no issue slots
    for (int tries = 0; tries < maxTries; ++tries)
    {
        __nanosleep(sleepNs);
        if (mbar_try_wait(bar, parity))
            return;
    }
    *reinterpret_cast<volatile unsigned*>(broken) = 1u;
    if (status)
        atomicOr(status, 2u);
}
// box (rows x0 .., columns x1 ..) of the matrix behind `tmap` -> dense tile [column][row]
__device__ __forceinline__ void tensor_load_2d(float* dstShared, const void* tmap, int x0, int x1, unsigned long long* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_addr(dstShared)),
                 "l"(tmap), "r"(smem_addr(bar)), "r"(x0), "r"(x1)
                 : "memory");
}

// Ordered walk over the rows of one tile column (a multiple of 4 rows): thirty-two rows per loop trip in two register
// sets of sixteen, each set reloaded while the other is being added, so the loop carries no register moves.
template <int KIND>
__device__ __forceinline__ float walk_chunk(const float* __restrict__ vcol, int nrows, float acc)
{
    const float4* __restrict__ p = reinterpret_cast<const float4*>(vcol);
    const int n16 = nrows >> 4;
    unsigned dummy = 0;
    if (n16 > 0)
    {
        float4 a0 = p[0], a1 = p[1], a2 = p[2], a3 = p[3];
        int t = 0;
        for (; t + 2 <= n16; t += 2)
        {
            const float4 b0 = p[4 * t + 4], b1 = p[4 * t + 5], b2 = p[4 * t + 6], b3 = p[4 * t + 7];
            walk_step4<KIND>(acc, dummy, a0, 0.0f, false);
            walk_step4<KIND>(acc, dummy, a1, 0.0f, false);
            walk_step4<KIND>(acc, dummy, a2, 0.0f, false);
            walk_step4<KIND>(acc, dummy, a3, 0.0f, false);
            const int nx = 4 * min(t + 2, n16 - 1); // the last trip reloads rows it will not use
            a0 = p[nx];
            a1 = p[nx + 1];
            a2 = p[nx + 2];
            a3 = p[nx + 3];
            walk_step4<KIND>(acc, dummy, b0, 0.0f, false);
            walk_step4<KIND>(acc, dummy, b1, 0.0f, false);
            walk_step4<KIND>(acc, dummy, b2, 0.0f, false);
            walk_step4<KIND>(acc, dummy, b3, 0.0f, false);
        }
        if (t < n16)
        {
            walk_step4<KIND>(acc, dummy, a0, 0.0f, false);
            walk_step4<KIND>(acc, dummy, a1, 0.0f, false);
            walk_step4<KIND>(acc, dummy, a2, 0.0f, false);
            walk_step4<KIND>(acc, dummy, a3, 0.0f, false);
        }
    }
    int i = n16 << 4;
    for (; i + 4 <= nrows; i += 4)
        walk_step4<KIND>(acc, dummy, p[i >> 2], 0.0f, false);
    for (; i < nrows; ++i)
        walk_step<KIND>(acc, dummy, vcol[i], 0.0f, false);
    return acc;
}

// The same walk over a tile column whose height is known at compile time, fully unrolled: the compiler hoists the
// shared-memory loads far ahead of the add chain, and the walk runs at the latency of one fp32 add per row (4.6 cycles
// per row measured, against 6 to 8 for walk_chunk, whose trip count is a run-time value).  Worth its code size only where
// the walk is all a kernel does: in the streaming quantize kernel, unrolled walks for every chunk height slowed the element
// warps down more than they sped the walkers up.
template <int KIND, int R>
__device__ __forceinline__ float walk_tile(const float* __restrict__ vcol, float acc)
{
    static_assert(R % 4 == 0, "tile height must be a multiple of 4");
    const float4* __restrict__ p = reinterpret_cast<const float4*>(vcol);
    unsigned dummy = 0;
#pragma unroll
    for (int i = 0; i < R / 4; ++i)
        walk_step4<KIND>(acc, dummy, p[i], 0.0f, false);
    return acc;
}
// the residual proper of a value kept in deferred form: prev - level(prev), the single subtraction of
// ColumnQuantizer.h:100-125 performed when the state is next read
__device__ __forceinline__ float deferred_residual(float prev, float lv0, float lv1)
{
    return __fsub_rn(prev, (prev >= 0.0f) ? lv1 : lv0);
}

} // namespace qagg
