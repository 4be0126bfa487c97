// V2AllReduceDistGradAggregator.h -- IDistGradAggregator over the V2 quantized communicator, with the constructor and
// AggregateGradients contract of Source/1BitSGD/V2AllReduceDistGradAggregator.h:31-44, 100-189, 191-272.
//
// Kept from the reference: the first call initialises, a later call with resetState zeroes the quantization residuals
// (:78-98; here they live inside the communicator, so this is ResetResiduals()); a rank with numSamples == 0 contributes
// zero gradients (:206-222); the header (criterion, numSamples, numSamplesWithLabel, eval pairs) is summed over the
// workers through AggregateInPlace (:224-250); the gradient matrices are handed to QuantizedAggregateInPlace as views
// over the same device memory (:252-266), so a single worker gets them back untouched; the return value is "any samples
// processed"; sparse gradients are refused (:63-64); syncStatsTrace > 0 prints the aggregation time.
// Not built: useAsyncAggregation = true for this adapter (the V1 aggregator has it) -- requesting it throws.
#pragma once

#include <chrono>
#include <cstdio>
#include <vector>

#include "IDistGradAggregator.h"
#include "QuantizedDistributedCommunicator.h"

namespace Microsoft { namespace MSR { namespace CNTK {

template <class ElemType>
class V2AllReduceDistGradAggregator : public IDistGradAggregator<ElemType>
{
public:
    V2AllReduceDistGradAggregator(::CNTK::QuantizedDistributedCommunicatorPtr communicator, bool useAsyncAggregation, int traceLevel, int syncStatsTrace)
        : IDistGradAggregator<ElemType>(nullptr), m_communicator(communicator), m_traceLevel(traceLevel), m_syncStatsTrace(syncStatsTrace)
    {
        if (useAsyncAggregation)
            LogicError("V2AllReduceDistGradAggregator: buffered asynchronous aggregation is not implemented in this build");
    }

    bool AggregateGradients(const std::vector<Matrix<ElemType>*>& gradients, DistGradHeader* headerCPU, bool resetState) override
    {
        if (!m_initialized)
        {
            for (auto* g : gradients)
                if (g->GetMatrixType() != DENSE)
                    RuntimeError("Gradient aggregation for sparse gradient matrices is currently unsupported!");
            m_initialized = true;
        }
        else if (resetState)
        {
            m_communicator->ResetResiduals();
        }
        const bool showStats = (m_syncStatsTrace > 0) && ((m_iterationCount % m_syncStatsTrace) == 0);
        m_iterationCount++;
        std::chrono::steady_clock::time_point t0;
        if (showStats)
        {
            cudaDeviceSynchronize();
            t0 = std::chrono::steady_clock::now();
        }

        // if this node did not process any samples, its gradients are zero
        if (headerCPU->numSamples == 0)
            for (auto* g : gradients)
                g->SetValue(0);

        std::vector<double> h(3 + 2 * (size_t) headerCPU->numEvalNode);
        h[0] = headerCPU->criterion;
        h[1] = (double) headerCPU->numSamples;
        h[2] = (double) headerCPU->numSamplesWithLabel;
        for (int i = 0; i < headerCPU->numEvalNode; ++i)
        {
            h[3 + 2 * i] = headerCPU->evalErrors[i].first;
            h[4 + 2 * i] = (double) headerCPU->evalErrors[i].second;
        }
        m_communicator->AggregateInPlace(h, m_communicator->Workers());
        headerCPU->criterion = h[0];
        headerCPU->numSamples = (size_t) h[1];
        headerCPU->numSamplesWithLabel = (size_t) h[2];
        for (int i = 0; i < headerCPU->numEvalNode; ++i)
        {
            headerCPU->evalErrors[i].first = h[3 + 2 * i];
            headerCPU->evalErrors[i].second = (size_t) h[4 + 2 * i];
        }

        std::vector<::CNTK::NDArrayViewPtr> values;
        for (auto* g : gradients)
            values.push_back(std::make_shared<Matrix<ElemType>>(g->GetNumRows(), g->GetNumCols(), g->Data(), g->GetDeviceId()));
        m_communicator->QuantizedAggregateInPlace(values, m_communicator->Workers());

        if (showStats)
            fprintf(stderr, "Actual gradient aggregation time: %.6g\n", std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
        (void) m_traceLevel;
        return headerCPU->numSamples != 0;
    }

private:
    ::CNTK::QuantizedDistributedCommunicatorPtr m_communicator;
    int m_traceLevel, m_syncStatsTrace;
    bool m_initialized = false;
    size_t m_iterationCount = 0;
};

}}}
