// AllReduceDistGradAggregator.h -- 1-bit SGD aggregator with the constructor and AggregateGradients contract of
// Source/1BitSGD/AllReduceDistGradAggregator.h:40-43, 150-235, implemented over the C ABI of libqagg.
//
// Kept from the reference: gradients are aggregated IN PLACE; residuals, packed buffers and stripe residuals belong to
// the aggregator and are created on the first call from the gradient shapes (which must not change, :69-71); resetState on
// a later call zeroes the residuals (:121-136); a rank with numSamples == 0 contributes zero gradients (:250-259); the
// header is summed over ranks; the return value is "any samples processed" (:233); sparse gradients are refused (:82-83);
// syncStatsTrace > 0 prints "Actual gradient aggregation time" every that many calls (:153, 241-246, 560-565).
// Not built yet: useAsyncAggregation (double-buffered aggregation, :156-229) -- requesting it throws.
#pragma once

#include <chrono>
#include <cstdio>
#include <vector>

#include "IDistGradAggregator.h"

namespace Microsoft { namespace MSR { namespace CNTK {

template <class ElemType>
class AllReduceDistGradAggregator : public IDistGradAggregator<ElemType>
{
    using IDistGradAggregator<ElemType>::m_mpi;

public:
    AllReduceDistGradAggregator(const MPIWrapperPtr& mpi, int nBits, bool zeroThresholdFor1Bit, bool useQuantizationForSelfStripe,
                                bool useAsyncAggregation, int traceLevel, int syncStatsTrace)
        : IDistGradAggregator<ElemType>(mpi), m_nBits(nBits), m_zeroThr(zeroThresholdFor1Bit), m_selfQuant(useQuantizationForSelfStripe),
          m_traceLevel(traceLevel), m_syncStatsTrace(syncStatsTrace)
    {
        if (useAsyncAggregation)
            LogicError("AllReduceDistGradAggregator: buffered asynchronous aggregation is not implemented in this build");
    }
    ~AllReduceDistGradAggregator() override
    {
        if (m_agg)
            qagg_agg_destroy(m_agg);
    }

    bool AggregateGradients(const std::vector<Matrix<ElemType>*>& gradients, DistGradHeader* headerCPU, bool resetState) override
    {
        const bool showStats = (m_syncStatsTrace > 0) && ((m_iterationCount % m_syncStatsTrace) == 0);
        m_iterationCount++;
        if (!m_agg)
            Initialize(gradients);
        else if (resetState)
            QaggCheck(qagg_agg_reset_residuals(m_agg, nullptr), "ResetResidue");
        if (gradients.size() != m_ptrs.size())
            LogicError("AggregateGradients: the number of gradient matrices changed");

        std::chrono::steady_clock::time_point t0;
        if (showStats)
        {
            cudaDeviceSynchronize();
            t0 = std::chrono::steady_clock::now();
        }
        if (headerCPU->numSamples == 0)
            for (auto* g : gradients)
                g->SetValue(0);

        // header: numSamples, numSamplesWithLabel, criterion and the eval pairs, summed over ranks
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

        for (size_t i = 0; i < gradients.size(); ++i)
        {
            if (gradients[i]->GetNumRows() != m_rows[i] || gradients[i]->GetNumCols() != m_cols[i])
                LogicError("AggregateGradients: gradient matrix %zu changed shape", i);
            m_ptrs[i] = gradients[i]->Data();
        }
        QaggCheck(qagg_agg_step(m_agg, m_ptrs.data(), nullptr), "AggregateGradients");
        if (cudaStreamSynchronize(nullptr) != cudaSuccess)
            RuntimeError("AggregateGradients: the aggregation step failed on the device");
        if (showStats)
        {
            const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            fprintf(stderr, "Actual gradient aggregation time: %.6g\n", s);
        }
        return headerCPU->numSamples != 0;
    }

private:
    void Initialize(const std::vector<Matrix<ElemType>*>& gradients)
    {
        std::vector<int64_t> M, N;
        for (auto* g : gradients)
        {
            if (g->GetMatrixType() != DENSE)
                RuntimeError("Gradient aggregation for sparse gradient matrices is currently unsupported!");
            M.push_back((int64_t) g->GetNumRows());
            N.push_back((int64_t) g->GetNumCols());
            m_rows.push_back(g->GetNumRows());
            m_cols.push_back(g->GetNumCols());
        }
        const int flags = (m_zeroThr ? QAGG_ZERO_THRESHOLD : 0) | (m_selfQuant ? QAGG_SELF_QUANTIZED : 0);
        QaggCheck(qagg_agg_create(m_mpi->Handle(), (int) gradients.size(), M.data(), N.data(), m_nBits, flags, &m_agg), "qagg_agg_create");
        m_ptrs.resize(gradients.size());
        (void) m_traceLevel;
    }

    int m_nBits;
    bool m_zeroThr, m_selfQuant;
    int m_traceLevel, m_syncStatsTrace;
    size_t m_iterationCount = 0;
    qagg_aggregator* m_agg = nullptr;
    std::vector<float*> m_ptrs;
    std::vector<size_t> m_rows, m_cols;
};

}}}
