// qagg_agg_f64.cu -- the striped aggregation for DOUBLE gradients (ElemType = double, QWord = uint64: the precision the
// reference's own 1-bit end-to-end tests run, Tests/EndToEndTests/Speech/DNN/Parallel1BitQuantization).
//
// It follows AllReduceDistGradAggregator<double>::AggregateGradientsImpl (Source/1BitSGD/AllReduceDistGradAggregator.h:237-566)
// step for step, built from the two double-precision matrix kernels of qagg_f64.cu exactly as the reference builds it from
// its quantizer: every rank quantizes every gradient against its residual (:290-300); stripe p of every packed matrix goes
// to rank p (:303-365); the owner unquantizes its own stripe into its slice of the gradient (:366-375), adds the received
// stripes -- in ascending source order here, arrival order there (:389-421) -- requantizes the sum against its stripe
// residual (:429-435), the requantized stripes are gathered (:459-512) and everything is unquantized (:516-522).
// One kernel launch per matrix and step of the above: correct and bit-identical to the CPU checker, not tuned -- the fp32
// path (qagg_aggregator.cu) is the fast one.  Transport: NCCL send/recv between processes, device-to-device copies inside
// an in-process group.
#include "../../include/qagg.h"
#include "qagg_comm.h"
#include "qagg_internal.h"

#include <cstring>
#include <memory>
#include <vector>

using namespace qagg;

struct qagg_aggregator_f64
{
    qagg_comm* comm = nullptr;
    int T = 0, bits = 1, flags = 0;
    std::vector<int64_t> M, N, C;          // rows, columns, packed column bytes per tensor
    std::vector<int64_t> s0, sn;           // this rank's stripe of every tensor: first column, columns
    std::vector<double*> res, sres;        // residual (M x N) and stripe residual (M x sn) per tensor
    std::vector<unsigned char*> pk, gath;  // packed matrix as quantized here; packed matrix as gathered
    std::vector<unsigned char*> recv;      // K slots of this rank's stripe per tensor (slot = source rank)
    std::vector<void*> allocs;
    bool identity = false;

    ~qagg_aggregator_f64()
    {
        for (void* p : allocs)
            cudaFree(p);
    }
    template <class P>
    int alloc(P** out, size_t bytes)
    {
        void* p = nullptr;
        int rc = check_cuda(cudaMalloc(&p, bytes ? bytes : 16), "cudaMalloc");
        if (rc)
            return rc;
        if ((rc = check_cuda(cudaMemset(p, 0, bytes ? bytes : 16), "cudaMemset")))
            return rc;
        allocs.push_back(p);
        *out = static_cast<P*>(p);
        return QAGG_OK;
    }
    unsigned char* recv_slot(int i, int src) const { return recv[i] + (size_t) src * (size_t) (sn[i] * C[i]); }
};

namespace {

int nccl_ok(ncclResult_t r, const char* what)
{
    if (r == ncclSuccess)
        return QAGG_OK;
    return fail(QAGG_ENCCL, std::string(what) + ": " + ncclGetErrorString(r));
}

void stripe_of(int64_t N, int r, int K, int64_t* start, int64_t* n)
{
    qagg_stripe(N, r, K, start, n);
}

// steps 1: quantize everything
int quantize_all(qagg_aggregator_f64* a, double* const* grads, cudaStream_t st)
{
    for (int i = 0; i < a->T; ++i)
    {
        int rc = qagg_quantize_f64(st, grads[i], a->res[i], a->res[i], a->pk[i], a->M[i], a->N[i], a->bits, (a->flags & QAGG_ZERO_THRESHOLD) ? 1 : 0);
        if (rc)
            return rc;
    }
    return QAGG_OK;
}

// the owner's pass: own stripe, then the received ones in ascending source order, then requantize into the gathered matrix
int own_stripes(qagg_aggregator_f64* a, double* const* grads, cudaStream_t st)
{
    const int K = a->comm->K, r = a->comm->rank;
    for (int i = 0; i < a->T; ++i)
    {
        if (a->sn[i] == 0 || a->M[i] == 0)
            continue;
        double* agg = grads[i] + a->s0[i] * a->M[i]; // the stripe's slice of the gradient (ColumnSlice, :281)
        int rc;
        if (a->flags & QAGG_SELF_QUANTIZED)
            if ((rc = qagg_unquantize_f64(st, a->pk[i] + a->s0[i] * a->C[i], agg, a->M[i], a->sn[i], a->bits, 0)))
                return rc;
        for (int src = 0; src < K; ++src)
        {
            if (src == r)
                continue;
            if ((rc = qagg_unquantize_f64(st, a->recv_slot(i, src), agg, a->M[i], a->sn[i], a->bits, 1)))
                return rc;
        }
        if ((rc = qagg_quantize_f64(st, agg, a->sres[i], a->sres[i], a->gath[i] + a->s0[i] * a->C[i], a->M[i], a->sn[i], a->bits,
                                    (a->flags & QAGG_ZERO_THRESHOLD) ? 1 : 0)))
            return rc;
    }
    return QAGG_OK;
}

int unquantize_all(qagg_aggregator_f64* a, double* const* grads, const std::vector<unsigned char*>& from, cudaStream_t st)
{
    for (int i = 0; i < a->T; ++i)
    {
        int rc = qagg_unquantize_f64(st, from[i], grads[i], a->M[i], a->N[i], a->bits, 0);
        if (rc)
            return rc;
    }
    return QAGG_OK;
}

int check_args(const qagg_aggregator_f64* a, double* const* grads)
{
    if (!a || (a->T > 0 && !grads))
        return fail(QAGG_EINVAL, "qagg_agg_f64_step: bad arguments");
    for (int i = 0; i < a->T; ++i)
        if (a->M[i] * a->N[i] > 0 && (!grads[i] || (reinterpret_cast<uintptr_t>(grads[i]) & 7)))
            return fail(QAGG_EINVAL, "qagg_agg_f64_step: null or misaligned gradient pointer");
    return QAGG_OK;
}

} // namespace

extern "C" {

int qagg_agg_f64_create(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, int bits, int flags, qagg_aggregator_f64** out)
{
    if (!comm || !out || num_tensors < 0 || (num_tensors > 0 && (!M || !N)))
        return fail(QAGG_EINVAL, "qagg_agg_f64_create: bad arguments");
    if (bits < 1 || bits > 64 || (bits & (bits - 1)))
        return fail(QAGG_EINVAL, "bits must be a power of two in 1..64");
    for (int i = 0; i < num_tensors; ++i)
        if (M[i] < 0 || N[i] < 0 || M[i] > 0x3fffffffLL || N[i] > 0x7fffffffLL)
            return fail(QAGG_EINVAL, "qagg_agg_f64_create: bad tensor shape");
    int rc = check_cuda(cudaSetDevice(comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    std::unique_ptr<qagg_aggregator_f64> a(new qagg_aggregator_f64);
    a->comm = comm;
    a->T = num_tensors;
    a->bits = bits;
    a->flags = flags;
    a->identity = (comm->K == 1) && (flags & QAGG_V2_IDENTITY_K1);
    const int K = comm->K, r = comm->rank;
    a->M.assign(M, M + num_tensors);
    a->N.assign(N, N + num_tensors);
    a->C.resize(num_tensors);
    a->s0.resize(num_tensors);
    a->sn.resize(num_tensors);
    a->res.resize(num_tensors);
    a->sres.resize(num_tensors);
    a->pk.resize(num_tensors);
    a->gath.resize(num_tensors);
    a->recv.resize(num_tensors);
    for (int i = 0; i < num_tensors; ++i)
    {
        a->C[i] = 16 + 8 * ((M[i] * bits + 63) / 64);
        stripe_of(N[i], r, K, &a->s0[i], &a->sn[i]);
        if (a->identity)
            continue;
        if ((rc = a->alloc(&a->res[i], (size_t) (M[i] * N[i]) * 8)) || (rc = a->alloc(&a->pk[i], (size_t) (N[i] * a->C[i]))))
            return rc;
        if (K > 1)
        {
            if ((rc = a->alloc(&a->sres[i], (size_t) (M[i] * a->sn[i]) * 8)) || (rc = a->alloc(&a->gath[i], (size_t) (N[i] * a->C[i]))) ||
                (rc = a->alloc(&a->recv[i], (size_t) K * (size_t) (a->sn[i] * a->C[i]))))
                return rc;
        }
    }
    *out = a.release();
    return QAGG_OK;
}

int qagg_agg_f64_step(qagg_aggregator_f64* a, double* const* grads, void* stream)
{
    int rc = check_args(a, grads);
    if (rc)
        return rc;
    if (a->comm->local && a->comm->K > 1)
        return fail(QAGG_ESTATE, "aggregators of a local group must be stepped with qagg_agg_f64_step_group");
    if (a->identity)
        return QAGG_OK;
    cudaStream_t st = (cudaStream_t) stream;
    if ((rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice")) || (rc = quantize_all(a, grads, st)))
        return rc;
    const int K = a->comm->K, r = a->comm->rank;
    if (K == 1)
        return unquantize_all(a, grads, a->pk, st); // one rank, V1 semantics: quantize -> unquantize (:366-375, :516-522)
    // stripe p of every packed matrix -> rank p
    if ((rc = nccl_ok(ncclGroupStart(), "ncclGroupStart")))
        return rc;
    for (int i = 0; i < a->T; ++i)
        for (int p = 0; p < K; ++p)
        {
            if (p == r)
                continue;
            int64_t ps, pn;
            stripe_of(a->N[i], p, K, &ps, &pn);
            if (pn > 0 && (rc = nccl_ok(ncclSend(a->pk[i] + ps * a->C[i], (size_t) (pn * a->C[i]), ncclUint8, p, a->comm->nccl, st), "ncclSend")))
                return rc;
            if (a->sn[i] > 0 && (rc = nccl_ok(ncclRecv(a->recv_slot(i, p), (size_t) (a->sn[i] * a->C[i]), ncclUint8, p, a->comm->nccl, st), "ncclRecv")))
                return rc;
        }
    if ((rc = nccl_ok(ncclGroupEnd(), "ncclGroupEnd")) || (rc = own_stripes(a, grads, st)))
        return rc;
    // the requantized stripes -> every rank
    if ((rc = nccl_ok(ncclGroupStart(), "ncclGroupStart")))
        return rc;
    for (int i = 0; i < a->T; ++i)
        for (int p = 0; p < K; ++p)
        {
            if (p == r)
                continue;
            int64_t ps, pn;
            stripe_of(a->N[i], p, K, &ps, &pn);
            if (a->sn[i] > 0 &&
                (rc = nccl_ok(ncclSend(a->gath[i] + a->s0[i] * a->C[i], (size_t) (a->sn[i] * a->C[i]), ncclUint8, p, a->comm->nccl, st), "ncclSend")))
                return rc;
            if (pn > 0 && (rc = nccl_ok(ncclRecv(a->gath[i] + ps * a->C[i], (size_t) (pn * a->C[i]), ncclUint8, p, a->comm->nccl, st), "ncclRecv")))
                return rc;
        }
    if ((rc = nccl_ok(ncclGroupEnd(), "ncclGroupEnd")))
        return rc;
    return unquantize_all(a, grads, a->gath, st);
}

int qagg_agg_f64_step_group(qagg_aggregator_f64* const* aggs, int num_ranks, double* const* const* grads, void* stream)
{
    if (!aggs || !grads || num_ranks < 1)
        return fail(QAGG_EINVAL, "qagg_agg_f64_step_group: bad arguments");
    const int K = num_ranks;
    cudaStream_t st = (cudaStream_t) stream;
    for (int r = 0; r < K; ++r)
    {
        if (!aggs[r] || aggs[r]->comm->K != K || aggs[r]->comm->rank != r || !aggs[r]->comm->local)
            return fail(QAGG_ESTATE, "qagg_agg_f64_step_group: aggregators are not ranks 0..K-1 of one local group");
        if (aggs[r]->T != aggs[0]->T || aggs[r]->bits != aggs[0]->bits || aggs[r]->M != aggs[0]->M || aggs[r]->N != aggs[0]->N)
            return fail(QAGG_ESTATE, "qagg_agg_f64_step_group: aggregators disagree on tensor shapes or bits");
        int rc = check_args(aggs[r], grads[r]);
        if (rc)
            return rc;
    }
    if (aggs[0]->identity)
        return QAGG_OK;
    int rc = check_cuda(cudaSetDevice(aggs[0]->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    for (int r = 0; r < K; ++r)
        if ((rc = quantize_all(aggs[r], grads[r], st)))
            return rc;
    if (K == 1)
        return unquantize_all(aggs[0], grads[0], aggs[0]->pk, st);
    const int T = aggs[0]->T;
    for (int r = 0; r < K; ++r)
        for (int i = 0; i < T; ++i)
            for (int p = 0; p < K; ++p)
            {
                const qagg_aggregator_f64* dst = aggs[p];
                if (p == r || dst->sn[i] == 0)
                    continue;
                if ((rc = check_cuda(cudaMemcpyAsync(dst->recv_slot(i, r), aggs[r]->pk[i] + dst->s0[i] * dst->C[i], (size_t) (dst->sn[i] * dst->C[i]),
                                                     cudaMemcpyDeviceToDevice, st), "stripe copy")))
                    return rc;
            }
    for (int r = 0; r < K; ++r)
        if ((rc = own_stripes(aggs[r], grads[r], st)))
            return rc;
    for (int r = 0; r < K; ++r)
        for (int i = 0; i < T; ++i)
            for (int p = 0; p < K; ++p)
            {
                const qagg_aggregator_f64* src = aggs[r];
                if (p == r || src->sn[i] == 0)
                    continue;
                const size_t off = (size_t) (src->s0[i] * src->C[i]);
                if ((rc = check_cuda(cudaMemcpyAsync(aggs[p]->gath[i] + off, src->gath[i] + off, (size_t) (src->sn[i] * src->C[i]), cudaMemcpyDeviceToDevice,
                                                     st), "aggregated stripe copy")))
                    return rc;
            }
    for (int r = 0; r < K; ++r)
        if ((rc = unquantize_all(aggs[r], grads[r], aggs[r]->gath, st)))
            return rc;
    return QAGG_OK;
}

int qagg_agg_f64_reset_residuals(qagg_aggregator_f64* a, void* stream)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    for (int i = 0; !rc && i < a->T; ++i)
    {
        if (a->res[i])
            rc = check_cuda(cudaMemsetAsync(a->res[i], 0, (size_t) (a->M[i] * a->N[i]) * 8, (cudaStream_t) stream), "cudaMemsetAsync");
        if (!rc && a->sres[i])
            rc = check_cuda(cudaMemsetAsync(a->sres[i], 0, (size_t) (a->M[i] * a->sn[i]) * 8, (cudaStream_t) stream), "cudaMemsetAsync");
    }
    return rc;
}

int qagg_agg_f64_residuals(qagg_aggregator_f64* a, int tensor, double** residual, double** stripe_residual)
{
    if (!a || tensor < 0 || tensor >= a->T)
        return fail(QAGG_EINVAL, "qagg_agg_f64_residuals: bad arguments");
    if (residual)
        *residual = a->res[tensor];
    if (stripe_residual)
        *stripe_residual = a->sres[tensor];
    return QAGG_OK;
}

int qagg_agg_f64_copy_residual(qagg_aggregator_f64* a, int tensor, int which, double* dst, void* stream)
{
    if (!a || tensor < 0 || tensor >= a->T || which < 0 || which > 1 || !dst)
        return fail(QAGG_EINVAL, "qagg_agg_f64_copy_residual: bad arguments");
    const double* src = which ? a->sres[tensor] : a->res[tensor];
    const int64_t cols = which ? a->sn[tensor] : a->N[tensor];
    if (!src || cols * a->M[tensor] == 0)
        return QAGG_OK;
    return check_cuda(cudaMemcpyAsync(dst, src, (size_t) (cols * a->M[tensor]) * 8, cudaMemcpyDeviceToDevice, (cudaStream_t) stream), "residual copy");
}

int qagg_agg_f64_destroy(qagg_aggregator_f64* a)
{
    delete a;
    return QAGG_OK;
}

} // extern "C"
