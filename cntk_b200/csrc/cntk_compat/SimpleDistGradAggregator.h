// SimpleDistGradAggregator.h -- the unquantized aggregator SGD creates for gradientBits = 8 * sizeof(ElemType)
// (Source/SGDLib/SGD.cpp:2351-2356), with the constructor and AggregateGradients contract of
// Source/SGDLib/SimpleDistGradAggregator.h:24-40, 62-147, 262-485, implemented over libqagg's unquantized arm
// (qagg_dense_*: all tensors laid end to end, summed in rank order by kernels over peer windows, or one ncclAllReduce).
//
// Kept from the reference: gradients are summed IN PLACE; a rank with numSamples == 0 contributes zero gradients
// (:283-299); the header is summed over the ranks and the return value is "any samples processed" (:146); sparse gradients
// are refused; syncStatsTrace > 0 prints "Actual gradient aggregation time" every that many calls.  The pack threshold is
// accepted and ignored: every tensor is packed.  useFP16AllReduce casts to half, sums as halves and casts back
// (Source/CNTKv2LibraryDll/DistributedCommunicator.cpp:411-429).  useAsyncAggregation (double buffering) is not built for this
// arm: asking for it throws, as an unsupported mode should.
#pragma once

#include <chrono>
#include <cstdio>
#include <vector>

#include "IDistGradAggregator.h"

namespace Microsoft { namespace MSR { namespace CNTK {

template <class ElemType>
class SimpleDistGradAggregator : public IDistGradAggregator<ElemType>
{
    using IDistGradAggregator<ElemType>::m_mpi;

public:
    SimpleDistGradAggregator(const MPIWrapperPtr& mpi, bool useAsyncAggregation, int deviceId, int syncStatsTrace, size_t packThresholdSizeInBytes = 0,
                             bool useFP16AllReduce = false)
        : IDistGradAggregator<ElemType>(mpi), m_deviceId(deviceId), m_syncStatsTrace(syncStatsTrace)
    {
        (void) packThresholdSizeInBytes;
        if (useAsyncAggregation)
            LogicError("SimpleDistGradAggregator: buffered asynchronous aggregation is not implemented for the unquantized arm in this build");
        m_fp16 = useFP16AllReduce;
    }
    ~SimpleDistGradAggregator() override
    {
        if (m_agg)
            qagg_dense_destroy(m_agg);
    }

    // the handles of all ranks' windows, in rank order (QAGG_PEER_HANDLE_BYTES each): switches to the peer-memory kernels
    void PeerHandle(void* out)
    {
        QaggCheck(qagg_dense_peer_handle(m_agg, out), "qagg_dense_peer_handle");
    }
    void EnablePeer(const void* handles)
    {
        QaggCheck(qagg_dense_enable_peer(m_agg, handles), "qagg_dense_enable_peer");
    }
    // creates the aggregator ahead of the first AggregateGradients call (needed to exchange peer handles first)
    void Initialize(const std::vector<Matrix<ElemType>*>& gradients)
    {
        if (m_agg)
            return;
        std::vector<int64_t> M, N;
        for (auto* g : gradients)
        {
            if (g->GetMatrixType() != DENSE)
                RuntimeError("Gradient aggregation for sparse gradient matrices is currently unsupported!");
            M.push_back((int64_t) g->GetNumRows());
            N.push_back((int64_t) g->GetNumCols());
        }
        QaggCheck(qagg_dense_create(m_mpi->Handle(), (int) gradients.size(), M.data(), N.data(), &m_agg), "qagg_dense_create");
        QaggCheck(qagg_dense_set_fp16(m_agg, m_fp16 ? 1 : 0), "qagg_dense_set_fp16");
        m_ptrs.resize(gradients.size());
    }

    bool AggregateGradients(const std::vector<Matrix<ElemType>*>& gradients, DistGradHeader* headerCPU, bool /*resetState*/) override
    {
        Initialize(gradients);
        if (gradients.size() != m_ptrs.size())
            LogicError("AggregateGradients: the number of gradient matrices changed");
        const bool showStats = (m_syncStatsTrace > 0) && ((m_iterationCount % m_syncStatsTrace) == 0);
        m_iterationCount++;
        std::chrono::steady_clock::time_point t0;
        if (showStats)
        {
            cudaDeviceSynchronize();
            t0 = std::chrono::steady_clock::now();
        }
        if (headerCPU->numSamples == 0)
            for (auto* g : gradients)
                g->SetValue(0);
        for (size_t i = 0; i < gradients.size(); ++i)
            m_ptrs[i] = gradients[i]->Data();
        QaggCheck(qagg_dense_step(m_agg, m_ptrs.data(), nullptr), "AggregateGradients");
        std::vector<double> h(3 + 2 * (size_t) headerCPU->numEvalNode);
        h[0] = headerCPU->criterion;
        h[1] = (double) headerCPU->numSamples;
        h[2] = (double) headerCPU->numSamplesWithLabel;
        for (int i = 0; i < headerCPU->numEvalNode; ++i)
        {
            h[3 + 2 * i] = headerCPU->evalErrors[i].first;
            h[4 + 2 * i] = (double) headerCPU->evalErrors[i].second;
        }
        QaggCheck(qagg_comm_allreduce_f64(m_mpi->Handle(), h.data(), (int) h.size(), nullptr), "header aggregation");
        headerCPU->criterion = h[0];
        headerCPU->numSamples = (size_t) h[1];
        headerCPU->numSamplesWithLabel = (size_t) h[2];
        for (int i = 0; i < headerCPU->numEvalNode; ++i)
        {
            headerCPU->evalErrors[i].first = h[3 + 2 * i];
            headerCPU->evalErrors[i].second = (size_t) h[4 + 2 * i];
        }
        if (cudaStreamSynchronize(nullptr) != cudaSuccess)
            RuntimeError("AggregateGradients: the aggregation step failed on the device");
        QaggCheck(qagg_dense_check(m_agg, nullptr), "AggregateGradients");
        if (showStats)
            fprintf(stderr, "Actual gradient aggregation time: %.6g\n", std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
        return headerCPU->numSamples != 0;
    }

private:
    int m_deviceId, m_syncStatsTrace;
    bool m_fp16 = false; // useFP16AllReduce: values travel and are summed as halves
    size_t m_iterationCount = 0;
    qagg_dense_aggregator* m_agg = nullptr;
    std::vector<float*> m_ptrs;
};

}}}
