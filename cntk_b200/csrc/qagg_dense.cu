// qagg_dense.cu -- the unquantized fp32 aggregation arm (gradientBits = 32): SimpleDistGradAggregator
// (Source/SGDLib/SimpleDistGradAggregator.h:262-485) and MPICommunicatorImpl::AggregateImpl
// (Source/CNTKv2LibraryDll/DistributedCommunicator.cpp:311-492) rebuilt for device buffers.
//
// The reference copies every tensor below its pack threshold (32 MB by default) into one contiguous buffer and all-reduces
// that buffer (and each larger tensor by itself) with MPI or NCCL.  Here ALL tensors are laid end to end in one flat
// sequence of floats (16-byte aligned tensor starts), which is cut into K equal slices; rank p owns slice p.  A step is
// three kernels over peer-mapped windows -- the same two flag hand-shakes as the quantized path, no collective call:
//   k_dense_scatter  every float of this rank's gradients is stored into slot [rank] of its owner's receive window
//                    (own slice: local store; other slices: NVLink stores) -- the reduce-scatter's transfer;
//   k_dense_reduce   the owner adds the K slots of its slice IN RANK ORDER (fp32, round to nearest: the result is the same
//                    on every run and every rank) and stores the sum into slice [rank] of every rank's gather window --
//                    the all-gather's transfer;
//   k_dense_unpack   gather window -> the gradient tensors, in place.
// Without peer mapping the flat buffer is all-reduced with ncclAllReduce (the baseline path; its summation order is
// NCCL's).  One rank: nothing to do.  Device-side waits are the bounded flag waits of the quantized path.
#include "../../include/qagg.h"
#include "qagg_comm.h"
#include "qagg_device.cuh"

#include <cuda_fp16.h>

#include <algorithm>
#include <cstring>
#include <memory>
#include <vector>

using namespace qagg;

namespace {

struct DenseTensor
{
    float* ptr;          // the gradient tensor (device)
    long long flat4;     // its first 16-byte unit in the flat sequence
    long long count;     // floats
};

constexpr int DT = 256;

// flat unit u (16 bytes = 4 floats) -> tensor index: last entry whose flat4 <= u
__device__ __forceinline__ int dense_find(const DenseTensor* __restrict__ t, int n, long long u, int cur)
{
    if (t[cur].flat4 <= u && (cur + 1 >= n || u < t[cur + 1].flat4))
        return cur;
    int lo = 0, hi = n;
    while (hi - lo > 1)
    {
        const int mid = (lo + hi) >> 1;
        if (t[mid].flat4 <= u)
            lo = mid;
        else
            hi = mid;
    }
    return lo;
}

struct DensePeers
{
    float* base[QAGG_MAXK]; // per owner p: where this rank's floats of slice p go (scatter), or per rank: its gather window (reduce)
    int K;
};

// the four floats of flat unit u of tensor tt (zero past the tensor's end: the tail of its last unit)
__device__ __forceinline__ float4 dense_load_unit(const DenseTensor& tt, long long u)
{
    const long long off = (u - tt.flat4) * 4;
    const float* p = tt.ptr + off;
    if (off + 4 <= tt.count && (reinterpret_cast<uintptr_t>(p) & 15) == 0)
        return *reinterpret_cast<const float4*>(p);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (off + 0 < tt.count) v.x = p[0];
    if (off + 1 < tt.count) v.y = p[1];
    if (off + 2 < tt.count) v.z = p[2];
    if (off + 3 < tt.count) v.w = p[3];
    return v;
}

__device__ __forceinline__ void dense_store_unit(const DenseTensor& tt, long long u, const float4& v)
{
    const long long off = (u - tt.flat4) * 4;
    float* p = tt.ptr + off;
    if (off + 4 <= tt.count && (reinterpret_cast<uintptr_t>(p) & 15) == 0)
    {
        *reinterpret_cast<float4*>(p) = v;
        return;
    }
    if (off + 0 < tt.count) p[0] = v.x;
    if (off + 1 < tt.count) p[1] = v.y;
    if (off + 2 < tt.count) p[2] = v.z;
    if (off + 3 < tt.count) p[3] = v.w;
}

// ---- fp16 transport (useFP16AllReduce, Source/CNTKv2LibraryDll/DistributedCommunicator.cpp:411-429): the gradients are cast
// to half (round to nearest), summed as halves, cast back.  A unit is then four halves (8 bytes); the windows keep their
// fp32 geometry and the half units use the first half of every slot.  The sum of two halves is taken in fp32 and rounded to
// half (what a half addition without a native instruction does), rank after rank.
__device__ __forceinline__ uint2 dense_to_half4(const float4& v)
{
    const __half2 a = __halves2half2(__float2half_rn(v.x), __float2half_rn(v.y));
    const __half2 b = __halves2half2(__float2half_rn(v.z), __float2half_rn(v.w));
    uint2 r;
    r.x = *reinterpret_cast<const unsigned*>(&a);
    r.y = *reinterpret_cast<const unsigned*>(&b);
    return r;
}
__device__ __forceinline__ float4 dense_from_half4(const uint2& h)
{
    const __half2 a = *reinterpret_cast<const __half2*>(&h.x);
    const __half2 b = *reinterpret_cast<const __half2*>(&h.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ float dense_half_round(float x)
{
    return __half2float(__float2half_rn(x));
}

// last CTA of a kernel: re-arm the counter and release the peers' flags (every CTA's stores were fenced before its arrival)
__device__ __forceinline__ void dense_finish(unsigned* counters, const Signal& signal)
{
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

template <bool HALF>
__global__ void __launch_bounds__(DT) k_dense_scatter(const DenseTensor* __restrict__ tensors, int nT, long long total4, long long slice4,
                                                      const DensePeers dst, unsigned* __restrict__ counters, const Signal signal)
{
    int cur = 0;
    for (long long u = (long long) blockIdx.x * DT + threadIdx.x; u < total4; u += (long long) gridDim.x * DT)
    {
        cur = dense_find(tensors, nT, u, cur);
        const float4 v = dense_load_unit(tensors[cur], u);
        const int p = (int) (u / slice4);
        if (HALF)
            reinterpret_cast<uint2*>(dst.base[p])[u - (long long) p * slice4] = dense_to_half4(v);
        else
            reinterpret_cast<float4*>(dst.base[p])[u - (long long) p * slice4] = v;
    }
    dense_finish(counters, signal);
}

// recv: this rank's receive window, K slots of slice4 units (slot s = rank s's floats of this rank's slice)
template <bool HALF>
__global__ void __launch_bounds__(DT) k_dense_reduce(const float4* __restrict__ recv, int K, long long slice4, long long mine4, int rank,
                                                     const DensePeers dst, unsigned* __restrict__ counters, const Signal signal)
{
    for (long long j = (long long) blockIdx.x * DT + threadIdx.x; j < mine4; j += (long long) gridDim.x * DT)
    {
        if (HALF)
        {
            // slot src starts where it does in fp32 geometry: 2 * slice4 eight-byte units further on
            const uint2* recv2 = reinterpret_cast<const uint2*>(recv);
            float4 s = dense_from_half4(__ldcs(recv2 + j));
            for (int src = 1; src < K; ++src)
            {
                const float4 v = dense_from_half4(__ldcs(recv2 + 2 * (long long) src * slice4 + j));
                s.x = dense_half_round(__fadd_rn(s.x, v.x));
                s.y = dense_half_round(__fadd_rn(s.y, v.y));
                s.z = dense_half_round(__fadd_rn(s.z, v.z));
                s.w = dense_half_round(__fadd_rn(s.w, v.w));
            }
            const uint2 h = dense_to_half4(s);
            for (int p = 0; p < dst.K; ++p)
                reinterpret_cast<uint2*>(dst.base[p])[2 * (long long) rank * slice4 + j] = h;
            continue;
        }
        float4 s = __ldcs(recv + j);
        for (int src = 1; src < K; ++src)
        {
            const float4 v = __ldcs(recv + (long long) src * slice4 + j);
            s.x = __fadd_rn(s.x, v.x);
            s.y = __fadd_rn(s.y, v.y);
            s.z = __fadd_rn(s.z, v.z);
            s.w = __fadd_rn(s.w, v.w);
        }
        for (int p = 0; p < dst.K; ++p)
            reinterpret_cast<float4*>(dst.base[p])[(long long) rank * slice4 + j] = s;
    }
    dense_finish(counters, signal);
}

// HALF: unit u of slice p sits at eight-byte unit p * sliceStride + (u - p * slice4) of `flat` (sliceStride = 2 * slice4 in a
// window with fp32 geometry, slice4 in a contiguous buffer)
template <bool HALF>
__global__ void __launch_bounds__(DT) k_dense_unpack(const float4* __restrict__ flat, const DenseTensor* __restrict__ tensors, int nT, long long total4,
                                                     long long slice4, long long sliceStride)
{
    int cur = 0;
    for (long long u = (long long) blockIdx.x * DT + threadIdx.x; u < total4; u += (long long) gridDim.x * DT)
    {
        cur = dense_find(tensors, nT, u, cur);
        if (HALF)
        {
            const long long p = u / slice4;
            dense_store_unit(tensors[cur], u, dense_from_half4(__ldcs(reinterpret_cast<const uint2*>(flat) + p * sliceStride + (u - p * slice4))));
        }
        else
            dense_store_unit(tensors[cur], u, __ldcs(flat + u));
    }
}

// NCCL path: gradients -> flat buffer
template <bool HALF>
__global__ void __launch_bounds__(DT) k_dense_pack(float4* __restrict__ flat, const DenseTensor* __restrict__ tensors, int nT, long long total4)
{
    int cur = 0;
    for (long long u = (long long) blockIdx.x * DT + threadIdx.x; u < total4; u += (long long) gridDim.x * DT)
    {
        cur = dense_find(tensors, nT, u, cur);
        if (HALF)
            reinterpret_cast<uint2*>(flat)[u] = dense_to_half4(dense_load_unit(tensors[cur], u));
        else
            flat[u] = dense_load_unit(tensors[cur], u);
    }
}

inline int64_t align_up(int64_t v, int64_t a)
{
    return (v + a - 1) / a * a;
}

} // namespace

struct qagg_dense_aggregator
{
    qagg_comm* comm = nullptr;
    int rank = 0, K = 1, device = 0;
    bool local = false;
    ncclComm_t nccl = nullptr;
    int T = 0;
    std::vector<int64_t> elems;
    std::vector<DenseTensor> host;     // flat layout (pointers filled per step)
    long long total4 = 0, slice4 = 0;  // 16-byte units: all tensors; one slice
    static const int64_t kFlagBytes = 512;
    void* window = nullptr;            // [flags][receive: K slots of one slice][gather: K slices = the whole flat sequence]
    void* table = nullptr;             // device copy of `host`
    void* queue = nullptr;             // counters
    std::vector<float*> bound;
    bool peer = false;
    unsigned char* peerWin[QAGG_MAXK] = {};
    bool peerOpened[QAGG_MAXK] = {};
    unsigned stepNo = 0;
    long long waitPolls = 20000000;
    int numSMs = 0;
    bool fp16 = false; // values travel and are summed as halves

    float* recv(unsigned char* win) const { return reinterpret_cast<float*>(win + kFlagBytes); }
    float* gather(unsigned char* win) const { return recv(win) + (size_t) K * (size_t) slice4 * 4; }
    unsigned* flags(unsigned char* win) const { return reinterpret_cast<unsigned*>(win); }
    unsigned* status() const { return reinterpret_cast<unsigned*>(window) + 127; }
    ~qagg_dense_aggregator()
    {
        for (int p = 0; p < QAGG_MAXK; ++p)
            if (peerOpened[p])
                cudaIpcCloseMemHandle(peerWin[p]);
        cudaFree(window);
        cudaFree(table);
        cudaFree(queue);
    }
};

extern "C" {

int qagg_dense_create(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, qagg_dense_aggregator** out)
{
    if (!comm || !out || num_tensors < 0 || (num_tensors > 0 && (!M || !N)))
        return fail(QAGG_EINVAL, "qagg_dense_create: bad arguments");
    const qagg_comm* cv = comm;
    int rc = check_cuda(cudaSetDevice(cv->device), "cudaSetDevice");
    if (rc)
        return rc;
    std::unique_ptr<qagg_dense_aggregator> a(new qagg_dense_aggregator);
    a->comm = comm;
    a->rank = cv->rank;
    a->K = cv->K;
    a->device = cv->device;
    a->local = cv->local;
    a->nccl = cv->nccl;
    a->T = num_tensors;
    long long flat4 = 0;
    for (int i = 0; i < num_tensors; ++i)
    {
        if (M[i] < 0 || N[i] < 0 || M[i] > 0x3fffffffLL || N[i] > 0x7fffffffLL)
            return fail(QAGG_EINVAL, "qagg_dense_create: bad tensor shape");
        a->elems.push_back(M[i] * N[i]);
        a->host.push_back(DenseTensor{nullptr, flat4, M[i] * N[i]});
        flat4 += (M[i] * N[i] + 3) / 4;
    }
    a->total4 = flat4;
    a->slice4 = std::max<long long>(1, (flat4 + a->K - 1) / a->K);
    cudaDeviceProp prop;
    if ((rc = check_cuda(cudaGetDeviceProperties(&prop, cv->device), "cudaGetDeviceProperties")))
        return rc;
    a->numSMs = prop.multiProcessorCount;
    const size_t winBytes = (size_t) qagg_dense_aggregator::kFlagBytes + 2 * (size_t) a->K * (size_t) a->slice4 * 16;
    if ((rc = check_cuda(cudaMalloc(&a->window, winBytes), "cudaMalloc")) || (rc = check_cuda(cudaMemset(a->window, 0, winBytes), "cudaMemset")))
        return rc;
    if ((rc = check_cuda(cudaMalloc(&a->table, std::max<size_t>(16, sizeof(DenseTensor) * (size_t) num_tensors)), "cudaMalloc")))
        return rc;
    if ((rc = check_cuda(cudaMalloc(&a->queue, 2 * QAGG_COUNTER_UINTS * sizeof(unsigned)), "cudaMalloc")) ||
        (rc = check_cuda(cudaMemset(a->queue, 0, 2 * QAGG_COUNTER_UINTS * sizeof(unsigned)), "cudaMemset")))
        return rc;
    *out = a.release();
    return QAGG_OK;
}

int qagg_dense_peer_handle(qagg_dense_aggregator* a, void* out)
{
    if (!a || !out)
        return fail(QAGG_EINVAL, "qagg_dense_peer_handle: bad arguments");
    int rc = check_cuda(cudaSetDevice(a->device), "cudaSetDevice");
    if (rc)
        return rc;
    std::memset(out, 0, QAGG_PEER_HANDLE_BYTES);
    if (a->local)
    {
        std::memcpy(out, &a->window, sizeof(void*));
        return QAGG_OK;
    }
    cudaIpcMemHandle_t h;
    if ((rc = check_cuda(cudaIpcGetMemHandle(&h, a->window), "cudaIpcGetMemHandle")))
        return rc;
    std::memcpy(out, &h, sizeof(h));
    return QAGG_OK;
}

int qagg_dense_enable_peer(qagg_dense_aggregator* a, const void* handles)
{
    if (!a || !handles)
        return fail(QAGG_EINVAL, "qagg_dense_enable_peer: bad arguments");
    if (a->peer)
        return fail(QAGG_ESTATE, "qagg_dense_enable_peer: already enabled");
    if (a->K == 1)
        return QAGG_OK;
    int rc = check_cuda(cudaSetDevice(a->device), "cudaSetDevice");
    if (rc)
        return rc;
    const unsigned char* hb = static_cast<const unsigned char*>(handles);
    for (int p = 0; p < a->K; ++p)
    {
        if (p == a->rank)
        {
            a->peerWin[p] = static_cast<unsigned char*>(a->window);
            continue;
        }
        void* q = nullptr;
        if (a->local)
        {
            std::memcpy(&q, hb + (size_t) p * QAGG_PEER_HANDLE_BYTES, sizeof(void*));
        }
        else
        {
            cudaIpcMemHandle_t h;
            std::memcpy(&h, hb + (size_t) p * QAGG_PEER_HANDLE_BYTES, sizeof(h));
            if ((rc = check_cuda(cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")))
                return rc;
            a->peerOpened[p] = true;
        }
        if (!q)
            return fail(QAGG_EINVAL, "qagg_dense_enable_peer: null peer window");
        a->peerWin[p] = static_cast<unsigned char*>(q);
    }
    a->peer = true;
    return QAGG_OK;
}

static int dense_bind(qagg_dense_aggregator* a, float* const* grads, cudaStream_t st)
{
    bool same = a->bound.size() == (size_t) a->T;
    for (int i = 0; same && i < a->T; ++i)
        same = a->bound[i] == grads[i];
    if (same)
        return QAGG_OK;
    for (int i = 0; i < a->T; ++i)
    {
        if (!grads[i] && a->elems[i] > 0)
            return fail(QAGG_EINVAL, "qagg_dense_step: null gradient pointer");
        a->host[i].ptr = grads[i];
    }
    int rc = check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize"); // an earlier step may still read the table
    if (rc)
        return rc;
    if (a->T > 0 && (rc = check_cuda(cudaMemcpy(a->table, a->host.data(), sizeof(DenseTensor) * (size_t) a->T, cudaMemcpyHostToDevice), "table upload")))
        return rc;
    a->bound.assign(grads, grads + a->T);
    return QAGG_OK;
}

static int dense_grid(const qagg_dense_aggregator* a, long long units)
{
    long long g = (units + DT - 1) / DT;
    const long long most = (long long) a->numSMs * 8;
    return (int) std::max<long long>(1, std::min(g, most));
}

// the three phases of one rank's step, so that a local group can interleave them rank by rank
static int dense_scatter(qagg_dense_aggregator* a, cudaStream_t st)
{
    DensePeers dst = {};
    dst.K = a->K;
    Signal sg = {};
    for (int p = 0; p < a->K; ++p)
    {
        dst.base[p] = a->recv(a->peerWin[p]) + (size_t) a->rank * (size_t) a->slice4 * 4;
        if (p != a->rank)
            sg.flag[sg.n++] = a->flags(a->peerWin[p]) + a->rank;
    }
    sg.value = a->stepNo;
    if (a->fp16)
        k_dense_scatter<true><<<dense_grid(a, a->total4), DT, 0, st>>>(static_cast<const DenseTensor*>(a->table), a->T, a->total4, a->slice4, dst,
                                                                        static_cast<unsigned*>(a->queue), sg);
    else
        k_dense_scatter<false><<<dense_grid(a, a->total4), DT, 0, st>>>(static_cast<const DenseTensor*>(a->table), a->T, a->total4, a->slice4, dst,
                                                                         static_cast<unsigned*>(a->queue), sg);
    return check_cuda(cudaGetLastError(), "dense scatter launch");
}

static int dense_wait(qagg_dense_aggregator* a, bool gatherPhase, cudaStream_t st)
{
    return check_cuda(launch_wait_flags(st, a->flags(static_cast<unsigned char*>(a->window)) + (gatherPhase ? 64 : 0), a->K, a->rank, a->stepNo, a->waitPolls,
                                        a->status()), "flag wait launch");
}

static int dense_reduce(qagg_dense_aggregator* a, cudaStream_t st)
{
    DensePeers dst = {};
    dst.K = a->K;
    Signal sg = {};
    for (int p = 0; p < a->K; ++p)
    {
        dst.base[p] = a->gather(a->peerWin[p]);
        if (p != a->rank)
            sg.flag[sg.n++] = a->flags(a->peerWin[p]) + 64 + a->rank;
    }
    sg.value = a->stepNo;
    const long long first = (long long) a->rank * a->slice4;
    const long long mine4 = std::max<long long>(0, std::min(a->slice4, a->total4 - first));
    const float4* recv = reinterpret_cast<const float4*>(a->recv(static_cast<unsigned char*>(a->window)));
    unsigned* counters = static_cast<unsigned*>(a->queue) + QAGG_COUNTER_UINTS;
    if (a->fp16)
        k_dense_reduce<true><<<dense_grid(a, std::max<long long>(mine4, 1)), DT, 0, st>>>(recv, a->K, a->slice4, mine4, a->rank, dst, counters, sg);
    else
        k_dense_reduce<false><<<dense_grid(a, std::max<long long>(mine4, 1)), DT, 0, st>>>(recv, a->K, a->slice4, mine4, a->rank, dst, counters, sg);
    return check_cuda(cudaGetLastError(), "dense reduce launch");
}

// contiguous: the half units lie back to back (the all-reduced buffer of the NCCL path), not in fp32 slice geometry
static int dense_unpack(qagg_dense_aggregator* a, cudaStream_t st, bool contiguous = false)
{
    const float4* flat = reinterpret_cast<const float4*>(a->gather(static_cast<unsigned char*>(a->window)));
    const DenseTensor* table = static_cast<const DenseTensor*>(a->table);
    if (a->fp16)
        k_dense_unpack<true><<<dense_grid(a, a->total4), DT, 0, st>>>(flat, table, a->T, a->total4, a->slice4, contiguous ? a->slice4 : 2 * a->slice4);
    else
        k_dense_unpack<false><<<dense_grid(a, a->total4), DT, 0, st>>>(flat, table, a->T, a->total4, a->slice4, a->slice4);
    return check_cuda(cudaGetLastError(), "dense unpack launch");
}

int qagg_dense_step(qagg_dense_aggregator* a, float* const* grads, void* stream)
{
    if (!a || (a->T > 0 && !grads))
        return fail(QAGG_EINVAL, "qagg_dense_step: bad arguments");
    if (a->local && a->K > 1)
        return fail(QAGG_ESTATE, "aggregators of a local group must be stepped with qagg_dense_step_group");
    if (a->K == 1 || a->total4 == 0)
        return QAGG_OK;
    cudaStream_t st = (cudaStream_t) stream;
    int rc = check_cuda(cudaSetDevice(a->device), "cudaSetDevice");
    if (rc)
        return rc;
    if ((rc = dense_bind(a, grads, st)))
        return rc;
    a->stepNo++;
    if (a->peer)
    {
        if ((rc = dense_scatter(a, st)) || (rc = dense_wait(a, false, st)) || (rc = dense_reduce(a, st)) || (rc = dense_wait(a, true, st)))
            return rc;
        return dense_unpack(a, st);
    }
    // baseline path: one all-reduce of the flat buffer (kept in the gather area of the window)
    float* flat = a->gather(static_cast<unsigned char*>(a->window));
    if (a->fp16)
        k_dense_pack<true><<<dense_grid(a, a->total4), DT, 0, st>>>(reinterpret_cast<float4*>(flat), static_cast<const DenseTensor*>(a->table), a->T, a->total4);
    else
        k_dense_pack<false><<<dense_grid(a, a->total4), DT, 0, st>>>(reinterpret_cast<float4*>(flat), static_cast<const DenseTensor*>(a->table), a->T, a->total4);
    if ((rc = check_cuda(cudaGetLastError(), "dense pack launch")))
        return rc;
    const ncclResult_t nr = ncclAllReduce(flat, flat, (size_t) a->total4 * 4, a->fp16 ? ncclHalf : ncclFloat, ncclSum, a->nccl, st);
    if (nr != ncclSuccess)
        return fail(QAGG_ENCCL, std::string("ncclAllReduce: ") + ncclGetErrorString(nr));
    return dense_unpack(a, st, true);
}

int qagg_dense_step_group(qagg_dense_aggregator* const* aggs, int num_ranks, float* const* const* grads, void* stream)
{
    if (!aggs || !grads || num_ranks < 1)
        return fail(QAGG_EINVAL, "qagg_dense_step_group: bad arguments");
    const int K = num_ranks;
    for (int r = 0; r < K; ++r)
    {
        if (!aggs[r] || aggs[r]->K != K || aggs[r]->rank != r || !aggs[r]->local)
            return fail(QAGG_ESTATE, "qagg_dense_step_group: aggregators are not ranks 0..K-1 of one local group");
        if (aggs[r]->elems != aggs[0]->elems)
            return fail(QAGG_ESTATE, "qagg_dense_step_group: aggregators disagree on tensor shapes");
        if (K > 1 && !aggs[r]->peer)
            return fail(QAGG_ESTATE, "qagg_dense_step_group: enable peer mode on every rank first (the ranks of a local group exchange through their windows)");
    }
    if (K == 1 || aggs[0]->total4 == 0)
        return QAGG_OK;
    cudaStream_t st = (cudaStream_t) stream;
    int rc = check_cuda(cudaSetDevice(aggs[0]->device), "cudaSetDevice");
    if (rc)
        return rc;
    // every rank's kernels run one after the other on this one stream, so each flag is already set when its waiter starts
    for (int r = 0; r < K; ++r)
    {
        if ((rc = dense_bind(aggs[r], grads[r], st)))
            return rc;
        aggs[r]->stepNo++;
        if ((rc = dense_scatter(aggs[r], st)))
            return rc;
    }
    for (int r = 0; r < K; ++r)
        if ((rc = dense_wait(aggs[r], false, st)))
            return rc;
    for (int r = 0; r < K; ++r)
        if ((rc = dense_reduce(aggs[r], st)))
            return rc;
    for (int r = 0; r < K; ++r)
        if ((rc = dense_wait(aggs[r], true, st)))
            return rc;
    for (int r = 0; r < K; ++r)
        if ((rc = dense_unpack(aggs[r], st)))
            return rc;
    return QAGG_OK;
}

int qagg_dense_set_fp16(qagg_dense_aggregator* a, int enabled)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    a->fp16 = enabled != 0;
    return QAGG_OK;
}

int qagg_dense_check(qagg_dense_aggregator* a, void* stream)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    int rc = check_cuda(cudaSetDevice(a->device), "cudaSetDevice");
    if (rc)
        return rc;
    unsigned st = 0;
    if ((rc = check_cuda(cudaMemcpyAsync(&st, a->status(), sizeof(st), cudaMemcpyDeviceToHost, (cudaStream_t) stream), "status read")))
        return rc;
    if ((rc = check_cuda(cudaStreamSynchronize((cudaStream_t) stream), "cudaStreamSynchronize")))
        return rc;
    if (st & 1u)
        return fail(QAGG_ETIMEOUT, "a device-side wait for a peer's flag ran out: a peer did not reach the step (results of that step are invalid)");
    return QAGG_OK;
}

int64_t qagg_dense_wire_bytes(const qagg_dense_aggregator* a)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    // scatter: every slice but the own one leaves; gather: the own slice goes to every peer
    return a->K > 1 ? 2 * (int64_t) (a->K - 1) * a->slice4 * (a->fp16 ? 8 : 16) : 0;
}

int qagg_dense_destroy(qagg_dense_aggregator* a)
{
    delete a;
    return QAGG_OK;
}

} // extern "C"
