// V2AllReduceDistGradAggregator.h -- IDistGradAggregator over the V2 quantized communicator, with the constructor and
// AggregateGradients contract of Source/1BitSGD/V2AllReduceDistGradAggregator.h:31-44, 50-98, 100-189, 191-272.
//
// Kept from the reference: the aggregator owns the two residual sets (m_residuals, m_stripeResiduals), which the
// communicator creates on the first call, and a later call with resetState zeroes them (:78-98); a rank with
// numSamples == 0 contributes zero gradients (:206-222); the header (criterion, numSamples, numSamplesWithLabel, eval
// pairs) is summed over the workers through AggregateInPlace (:224-250); the gradient matrices are handed to
// QuantizedAggregateInPlace as views over the same device memory (:252-266), so a single worker gets them back untouched;
// the return value is "any samples processed"; sparse gradients are refused (:63-64); syncStatsTrace > 0 prints the
// aggregation time.
// useAsyncAggregation (:110-183): a call first waits for the aggregation launched by the previous call, then SWAPS the
// contents of the caller's gradient matrices and header with the buffered ones (so the caller continues with the aggregate
// of the previous minibatch: one step stale, zeros after a reset) and starts the aggregation of what it just received on
// another host thread (std::async, as the reference does), which first makes the communicator's stream wait for an event
// recorded on the compute stream at the time of the call.  Resetting while an aggregation is pending is a logic error.
#pragma once

#include <chrono>
#include <cstdio>
#include <future>
#include <memory>
#include <unordered_map>
#include <vector>

#include "IDistGradAggregator.h"
#include "QuantizedDistributedCommunicator.h"

namespace Microsoft { namespace MSR { namespace CNTK {

template <class ElemType>
class V2AllReduceDistGradAggregator : public IDistGradAggregator<ElemType>
{
public:
    V2AllReduceDistGradAggregator(::CNTK::QuantizedDistributedCommunicatorPtr communicator, bool useAsyncAggregation, int traceLevel, int syncStatsTrace)
        : IDistGradAggregator<ElemType>(nullptr), m_communicator(communicator), m_useAsyncAggregation(useAsyncAggregation), m_traceLevel(traceLevel),
          m_syncStatsTrace(syncStatsTrace)
    {
    }
    ~V2AllReduceDistGradAggregator() override
    {
        if (m_pendingAsyncAggregation.valid())
            m_pendingAsyncAggregation.wait();
        if (m_bufferedGradHeader)
            DistGradHeader::Destroy(m_bufferedGradHeader);
        if (m_mainDone)
            cudaEventDestroy(m_mainDone);
    }

    bool AggregateGradients(const std::vector<Matrix<ElemType>*>& gradients, DistGradHeader* headerCPU, bool resetState) override
    {
        if (!m_initialized)
            Initialize(gradients, headerCPU->numEvalNode);
        else if (resetState)
            ResetState(gradients);
        const bool showSyncPerfStats = (m_syncStatsTrace > 0) && ((m_iterationCount % m_syncStatsTrace) == 0);
        m_iterationCount++;
        if (!m_useAsyncAggregation)
        {
            AggregateGradientsImpl(gradients, headerCPU, showSyncPerfStats, nullptr);
            return headerCPU->numSamples != 0;
        }
        // wait for the pending aggregation, swap in its results, start the aggregation of the new gradients
        if (m_pendingAsyncAggregation.valid())
        {
            const auto t0 = std::chrono::steady_clock::now();
            m_pendingAsyncAggregation.get();
            if (showSyncPerfStats)
                fprintf(stderr, "Async gradient aggregation wait time: %.6g\n",
                        std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
        }
        std::vector<Matrix<ElemType>*> newGradients;
        for (size_t i = 0; i < gradients.size(); i++)
        {
            Matrix<ElemType>* buffered = m_bufferedGradients[gradients[i]].get();
            if ((buffered == nullptr) || (buffered->GetNumCols() != gradients[i]->GetNumCols()) || (buffered->GetNumRows() != gradients[i]->GetNumRows()) ||
                (buffered->GetDeviceId() != gradients[i]->GetDeviceId()))
                LogicError("No buffered gradient matrix found corresponding to a gradient matrix to be aggregated!");
            swap(*(gradients[i]), *buffered); // contents, not objects
            newGradients.push_back(buffered);
        }
        swap(*headerCPU, *m_bufferedGradHeader);
        // initiate aggregation only if any samples were processed in the previous iteration
        if (resetState || (headerCPU->numSamples != 0))
        {
            const int deviceId = gradients[0]->GetDeviceId();
            DistGradHeader* newGradHeader = m_bufferedGradHeader;
            // the gradients must have been computed before the other thread's stream touches them
            if (cudaEventRecord(m_mainDone, nullptr) != cudaSuccess)
                RuntimeError("AggregateGradients: cannot record on the compute stream");
            cudaEvent_t ready = m_mainDone;
            m_pendingAsyncAggregation = std::async(std::launch::async, [=] {
                Matrix<ElemType>::SetDevice(deviceId);
                AggregateGradientsImpl(newGradients, newGradHeader, showSyncPerfStats, ready);
            });
            return true;
        }
        return false;
    }

    // the residual views this aggregator holds (call MaterializeResiduals() on the communicator before reading them)
    const std::vector<::CNTK::NDArrayViewPtr>& Residuals() const { return m_residuals; }
    const std::vector<::CNTK::NDArrayViewPtr>& StripeResiduals() const { return m_stripeResiduals; }

private:
    void Initialize(const std::vector<Matrix<ElemType>*>& gradients, int numEvalNodes)
    {
        m_initialized = true;
        const int deviceId = gradients[0]->GetDeviceId();
        for (size_t i = 0; i < gradients.size(); i++)
        {
            if (gradients[i]->GetMatrixType() != DENSE)
                RuntimeError("Gradient aggregation for sparse gradient matrices is currently unsupported!");
            if (m_useAsyncAggregation)
                m_bufferedGradients[gradients[i]].reset(new Matrix<ElemType>(gradients[i]->GetNumRows(), gradients[i]->GetNumCols(), deviceId));
        }
        if (m_useAsyncAggregation)
        {
            m_bufferedGradHeader = DistGradHeader::Create(numEvalNodes);
            m_bufferedGradHeader->Clear();
            if (cudaEventCreateWithFlags(&m_mainDone, cudaEventDisableTiming) != cudaSuccess)
                RuntimeError("V2AllReduceDistGradAggregator: cannot create the compute-stream event");
        }
    }

    void ResetState(const std::vector<Matrix<ElemType>*>& gradients)
    {
        if (m_useAsyncAggregation && m_pendingAsyncAggregation.valid())
            LogicError("Unexpected pending async gradient aggregation found when resetting aggregator state!");
        for (size_t i = 0; i < m_residuals.size(); ++i)
            if (m_residuals[i])
                m_residuals[i]->SetValue(static_cast<ElemType>(0.0));
        for (size_t i = 0; i < m_stripeResiduals.size(); ++i)
            if (m_stripeResiduals[i])
                m_stripeResiduals[i]->SetValue(static_cast<ElemType>(0.0));
        if (m_useAsyncAggregation)
        {
            for (size_t i = 0; i < gradients.size(); i++)
                m_bufferedGradients[gradients[i]]->SetValue(static_cast<ElemType>(0));
            m_bufferedGradHeader->Clear();
        }
    }

    void AggregateGradientsImpl(const std::vector<Matrix<ElemType>*>& gradients, DistGradHeader* headerCPU, bool showSyncPerfStats, cudaEvent_t inputsReady)
    {
        std::chrono::steady_clock::time_point t0;
        if (showSyncPerfStats)
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

        std::vector<::CNTK::NDArrayViewPtr> gradientValues;
        for (auto* g : gradients)
            gradientValues.push_back(std::make_shared<Matrix<ElemType>>(g->GetNumRows(), g->GetNumCols(), g->Data(), g->GetDeviceId()));
        auto* impl = dynamic_cast<::CNTK::QuantizedMPICommunicatorImpl*>(m_communicator.get());
        if (inputsReady && impl)
            impl->QuantizedAggregateAfter(inputsReady, gradientValues, m_residuals, m_stripeResiduals, gradientValues, m_residuals, m_stripeResiduals,
                                          m_communicator->Workers());
        else
            m_communicator->QuantizedAggregateInPlace(gradientValues, m_residuals, m_stripeResiduals, m_communicator->Workers());

        if (showSyncPerfStats)
            fprintf(stderr, "Actual gradient aggregation time: %.6g\n", std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
        (void) m_traceLevel;
    }

    ::CNTK::QuantizedDistributedCommunicatorPtr m_communicator;
    bool m_useAsyncAggregation;
    int m_traceLevel, m_syncStatsTrace;
    bool m_initialized = false;
    size_t m_iterationCount = 0;
    // residuals of quantized gradients and of the aggregated stripes this node owns
    std::vector<::CNTK::NDArrayViewPtr> m_residuals;
    std::vector<::CNTK::NDArrayViewPtr> m_stripeResiduals;
    // buffered asynchronous aggregation
    std::unordered_map<Matrix<ElemType>*, std::unique_ptr<Matrix<ElemType>>> m_bufferedGradients;
    DistGradHeader* m_bufferedGradHeader = nullptr;
    std::future<void> m_pendingAsyncAggregation;
    cudaEvent_t m_mainDone = nullptr;
};

}}}
