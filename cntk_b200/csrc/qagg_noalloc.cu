// qagg_noalloc.cu -- qagg_quantize_batch_noalloc: the batched column quantizer for callers that must not allocate.
//
// The table-driven quantize kernel needs scratch in device memory besides its inputs and outputs: one descriptor per
// matrix, the list of work items, and the work-queue counters.  The aggregator keeps those in buffers it cudaMallocs
// when it is created.  Some callers cannot do that: a plugin that is handed its device memory once and is forbidden
// to grow (the host framework's pool owns the rest of the card), a step that runs where a device-wide synchronising
// call such as cudaMalloc would stall every other stream of the process, or a component whose memory budget is audited
// and fixed before training starts.  For them the scratch lives in the fixed array below, which is part of the
// library's image: every GPU that loads libqagg.so holds these 64 KB until the process exits.
//
// Consequences the caller must know (also stated at the declaration in include/qagg.h):
//   * limits: at most QAGG_NOALLOC_MAX_MATRICES matrices and QAGG_NOALLOC_MAX_ITEMS work items per call; larger
//     batches are rejected with QAGG_EINVAL and a message, nothing is launched;
//   * the first call on each device looks up the array's device address and zeroes the counters.  That first call
//     should be made before any stream capture begins;
//   * all calls share the one array and it keeps the previous call's tables: two calls whose kernels could overlap
//     on the GPU (different streams, no dependency between them) race on it.  Calls on one stream are safe;
//   * the tables of a call are built in about 62 KB of the calling thread's stack and uploaded from there, so the
//     call needs that much stack, and a call on a stream that is being captured is refused with QAGG_ESTATE (the
//     recorded copy would point into a stack frame that no longer exists when the graph runs).
#include "../../include/qagg.h"
#include "qagg_internal.h"

#include <mutex>

using namespace qagg;

namespace {

constexpr int kMaxMatrices = QAGG_NOALLOC_MAX_MATRICES;
constexpr int kMaxItems = QAGG_NOALLOC_MAX_ITEMS;
constexpr size_t kCounterBytes = 2048; // QAGG_COUNTER_UINTS * 4 = 1088, rounded up
constexpr size_t kTensorBytes = (sizeof(QTensor) * kMaxMatrices + 255) / 256 * 256;
constexpr size_t kItemBytes = (sizeof(QItem) * kMaxItems + 255) / 256 * 256;
constexpr size_t kScratchBytes = kCounterBytes + kTensorBytes + kItemBytes;
static_assert(QAGG_COUNTER_UINTS * sizeof(unsigned) <= kCounterBytes, "counter block does not fit");
static_assert(kScratchBytes <= 64 * 1024, "the fixed scratch is meant to stay modest");

// In host code this name is only a stand-in for the symbol: it is NOT a device address and must never be handed to a
// kernel.  The device address is fetched per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct DeviceSetup
{
    bool ready = false;
    unsigned char* base = nullptr; // device address of g_noalloc_scratch on this device
    LaunchCfg cfg;
};
DeviceSetup g_setup[64];
std::mutex g_setupMutex;

// once per device, with that device current
int setup_current_device(DeviceSetup** out)
{
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc)
        return rc;
    if (dev < 0 || dev >= 64)
        return fail(QAGG_EINVAL, "device index out of range");
    std::lock_guard<std::mutex> lk(g_setupMutex);
    DeviceSetup& s = g_setup[dev];
    if (!s.ready)
    {
        void* p = nullptr;
        if ((rc = check_cuda(cudaGetSymbolAddress(&p, g_noalloc_scratch), "cudaGetSymbolAddress(g_noalloc_scratch)")))
            return rc;
        if (!p)
            return fail(QAGG_ECUDA, "cudaGetSymbolAddress returned a null address for the fixed scratch");
        if ((rc = check_cuda(cudaMemset(p, 0, kCounterBytes), "clearing the work-queue counters")))
            return rc;
        if ((rc = check_cuda(get_launch_cfg(dev, &s.cfg), "cudaGetDeviceProperties")))
            return rc;
        s.base = static_cast<unsigned char*>(p);
        s.ready = true;
    }
    *out = &s;
    return QAGG_OK;
}

} // namespace

extern "C" int qagg_quantize_batch_noalloc(void* stream, int num_matrices, const float* const* grads, const float* const* res_in,
                                           float* const* res_out, void* const* packed, const int64_t* M, const int64_t* N, int bits,
                                           int zero_threshold)
{
    if (num_matrices < 0 || (num_matrices > 0 && (!grads || !res_in || !res_out || !packed || !M || !N)))
        return fail(QAGG_EINVAL, "qagg_quantize_batch_noalloc: bad arguments");
    if (!bits_ok(bits))
        return fail(QAGG_EINVAL, "bits must be a power of two in 1..32");
    if (num_matrices > kMaxMatrices)
        return fail(QAGG_EINVAL, "qagg_quantize_batch_noalloc: " + std::to_string(num_matrices) + " matrices exceed the fixed scratch (at most " +
                                     std::to_string(kMaxMatrices) + " per call); split the batch");
    if (num_matrices == 0)
        return QAGG_OK;
    DeviceSetup* s = nullptr;
    int rc = setup_current_device(&s);
    if (rc)
        return rc;
    {
        // the table uploads below read this call's stack frame: they must run now, not when a captured graph is replayed
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if ((rc = check_cuda(cudaStreamIsCapturing((cudaStream_t) stream, &cap), "cudaStreamIsCapturing")))
            return rc;
        if (cap != cudaStreamCaptureStatusNone)
            return fail(QAGG_ESTATE, "qagg_quantize_batch_noalloc: the stream is being captured; this entry point uploads its tables from the "
                                     "caller's stack and cannot be recorded into a graph");
    }

    // tables are built on the stack: nothing is allocated on the host either
    QTensor tensors[kMaxMatrices];
    QItem items[kMaxItems];
    int nItems = 0;
    for (int i = 0; i < num_matrices; ++i)
    {
        if (M[i] < 0 || N[i] < 0 || M[i] > 0x3fffffffLL || N[i] > 0x7fffffffLL)
            return fail(QAGG_EINVAL, "qagg_quantize_batch_noalloc: bad matrix shape");
        QTensor& t = tensors[i];
        t = QTensor{};
        fill_layout(&t, M[i], N[i], bits);
        if (M[i] == 0 || N[i] == 0)
            continue;
        if (!grads[i] || !res_in[i] || !res_out[i] || !packed[i])
            return fail(QAGG_EINVAL, "qagg_quantize_batch_noalloc: null pointer");
        if ((reinterpret_cast<uintptr_t>(packed[i]) & 3) || (reinterpret_cast<uintptr_t>(grads[i]) & 3) || (reinterpret_cast<uintptr_t>(res_in[i]) & 3) ||
            (reinterpret_cast<uintptr_t>(res_out[i]) & 3))
            return fail(QAGG_EINVAL, "qagg_quantize_batch_noalloc: buffers must be 4-byte aligned");
        t.grad = grads[i];
        t.res_in = res_in[i];
        t.res_out = res_out[i];
        t.pk[0] = static_cast<unsigned char*>(packed[i]);
        const int c = cols_per_item(M[i], N[i], s->cfg.smemFloats, nullptr);
        const int64_t n = (N[i] + c - 1) / c;
        if (nItems + n > kMaxItems)
            return fail(QAGG_EINVAL, "qagg_quantize_batch_noalloc: the batch needs more than " + std::to_string(kMaxItems) +
                                         " work items, beyond the fixed scratch; split the batch");
        for (int64_t col0 = 0; col0 < N[i]; col0 += c)
            items[nItems++] = QItem{i, (int) col0, (int) ((N[i] - col0 < c) ? (N[i] - col0) : c)};
    }
    if (nItems == 0)
        return QAGG_OK;
    cudaStream_t st = (cudaStream_t) stream;
    unsigned* dCounters = reinterpret_cast<unsigned*>(s->base);
    QTensor* dTensors = reinterpret_cast<QTensor*>(s->base + kCounterBytes);
    QItem* dItems = reinterpret_cast<QItem*>(s->base + kCounterBytes + kTensorBytes);
    // stream-ordered uploads from pageable memory: the runtime has taken its copy of the source when the call returns
    if ((rc = check_cuda(cudaMemcpyAsync(dTensors, tensors, sizeof(QTensor) * (size_t) num_matrices, cudaMemcpyHostToDevice, st), "descriptor upload")))
        return rc;
    if ((rc = check_cuda(cudaMemcpyAsync(dItems, items, sizeof(QItem) * (size_t) nItems, cudaMemcpyHostToDevice, st), "work-item upload")))
        return rc;
    return check_cuda(launch_colquant(st, false, mode_of(bits, zero_threshold), nullptr, dTensors, dItems, nItems, 0, s->cfg, dCounters),
                      "quantize kernel launch");
}
