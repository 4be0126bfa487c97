// AllReduceDistGradAggregator.h -- 1-bit SGD aggregator with the constructor and AggregateGradients contract of
// Source/1BitSGD/AllReduceDistGradAggregator.h:40-43, 150-235, implemented over the C ABI of libqagg.
//
// Kept from the reference: gradients are aggregated IN PLACE; residuals, packed buffers and stripe residuals belong to
// the aggregator and are created on the first call from the gradient shapes (which must not change, :69-71); resetState on
// a later call zeroes the residuals (:121-136); a rank with numSamples == 0 contributes zero gradients (:250-259); the
// header is summed over ranks; the return value is "any samples processed" (:233); sparse gradients are refused (:82-83);
// syncStatsTrace > 0 prints "Actual gradient aggregation time" every that many calls (:153, 241-246, 560-565).
//
// useAsyncAggregation (double-buffered aggregation, :156-229): a call first waits for the aggregation launched by the
// previous call, then SWAPS the contents of the caller's gradient matrices and header with the aggregator's buffered ones
// (so the caller continues with the aggregate of the previous minibatch -- one step stale, zeros after a reset), and
// launches the aggregation of the gradients it just received; it returns without waiting for it.  Where the reference
// runs the aggregation on a std::async thread whose quantization stream waits for an event on the main compute stream
// (:203-221), this build enqueues it on a side CUDA stream that waits for the same kind of event: the caller-visible
// behaviour is the same, and no host thread is needed.  Resetting the state while an aggregation is pending is a logic
// error, as in the reference (:126-127).
#pragma once

#include <chrono>
#include <cstdio>
#include <memory>
#include <vector>

#include "IDistGradAggregator.h"

namespace Microsoft { namespace MSR { namespace CNTK {

// which entry points of the library an element type goes through: float -> the tuned aggregator, double -> the aggregator
// composed from the double-precision matrix kernels (ElemType = double is what the reference's 1-bit end-to-end tests run)
template <class ElemType>
struct QaggAggregatorApi;
template <>
struct QaggAggregatorApi<float>
{
    typedef qagg_aggregator* Handle;
    static int Create(qagg_comm* c, int n, const int64_t* M, const int64_t* N, int bits, int flags, Handle* out) { return qagg_agg_create(c, n, M, N, bits, flags, out); }
    static int Step(Handle h, float* const* g, void* st) { return qagg_agg_step(h, g, st); }
    static int Reset(Handle h) { return qagg_agg_reset_residuals(h, nullptr); }
    static void Destroy(Handle h) { qagg_agg_destroy(h); }
};
template <>
struct QaggAggregatorApi<double>
{
    typedef qagg_aggregator_f64* Handle;
    static int Create(qagg_comm* c, int n, const int64_t* M, const int64_t* N, int bits, int flags, Handle* out) { return qagg_agg_f64_create(c, n, M, N, bits, flags, out); }
    static int Step(Handle h, double* const* g, void* st) { return qagg_agg_f64_step(h, g, st); }
    static int Reset(Handle h) { return qagg_agg_f64_reset_residuals(h, nullptr); }
    static void Destroy(Handle h) { qagg_agg_f64_destroy(h); }
};

template <class ElemType>
class AllReduceDistGradAggregator : public IDistGradAggregator<ElemType>
{
    typedef QaggAggregatorApi<ElemType> Api;
    using IDistGradAggregator<ElemType>::m_mpi;

public:
    AllReduceDistGradAggregator(const MPIWrapperPtr& mpi, int nBits, bool zeroThresholdFor1Bit, bool useQuantizationForSelfStripe,
                                bool useAsyncAggregation, int traceLevel, int syncStatsTrace)
        : IDistGradAggregator<ElemType>(mpi), m_nBits(nBits), m_zeroThr(zeroThresholdFor1Bit), m_selfQuant(useQuantizationForSelfStripe),
          m_useAsync(useAsyncAggregation), m_traceLevel(traceLevel), m_syncStatsTrace(syncStatsTrace)
    {
    }
    ~AllReduceDistGradAggregator() override
    {
        if (m_pending)
            cudaStreamSynchronize(m_aggStream);
        if (m_agg)
            Api::Destroy(m_agg);
        if (m_bufferedHeader)
            DistGradHeader::Destroy(m_bufferedHeader);
        if (m_mainDone)
            cudaEventDestroy(m_mainDone);
        if (m_aggStream)
            cudaStreamDestroy(m_aggStream);
    }

    bool AggregateGradients(const std::vector<Matrix<ElemType>*>& gradients, DistGradHeader* headerCPU, bool resetState) override
    {
        const bool showStats = (m_syncStatsTrace > 0) && ((m_iterationCount % m_syncStatsTrace) == 0);
        m_iterationCount++;
        if (!m_agg)
        {
            Initialize(gradients, headerCPU->numEvalNode);
        }
        else if (resetState)
        {
            if (m_useAsync && m_pending)
                LogicError("Unexpected pending async gradient aggregation found when resetting aggregator state!");
            QaggCheck(Api::Reset(m_agg), "ResetResidue");
            if (m_useAsync)
            {
                for (auto& b : m_buffered)
                    b->SetValue(0);
                m_bufferedHeader->Clear();
            }
        }
        if (gradients.size() != m_ptrs.size())
            LogicError("AggregateGradients: the number of gradient matrices changed");
        for (size_t i = 0; i < gradients.size(); ++i)
            if (gradients[i]->GetNumRows() != m_rows[i] || gradients[i]->GetNumCols() != m_cols[i])
                LogicError("AggregateGradients: gradient matrix %zu changed shape", i);

        if (!m_useAsync)
        {
            std::chrono::steady_clock::time_point t0;
            if (showStats)
            {
                cudaDeviceSynchronize();
                t0 = std::chrono::steady_clock::now();
            }
            Launch(gradients, headerCPU, nullptr);
            Finish(headerCPU, nullptr);
            if (showStats)
            {
                const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
                fprintf(stderr, "Actual gradient aggregation time: %.6g\n", s);
            }
            return headerCPU->numSamples != 0;
        }

        // ---- buffered asynchronous aggregation ----
        if (m_pending)
        {
            const auto t0 = std::chrono::steady_clock::now();
            Finish(m_bufferedHeader, m_aggStream);
            m_pending = false;
            if (showStats)
                fprintf(stderr, "Async gradient aggregation wait time: %.6g\n",
                        std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
        }
        std::vector<Matrix<ElemType>*> newGradients;
        for (size_t i = 0; i < gradients.size(); ++i)
        {
            Matrix<ElemType>* buffered = m_buffered[i].get();
            if (buffered->GetNumCols() != gradients[i]->GetNumCols() || buffered->GetNumRows() != gradients[i]->GetNumRows() ||
                buffered->GetDeviceId() != gradients[i]->GetDeviceId())
                LogicError("No buffered gradient matrix found corresponding to a gradient matrix to be aggregated!");
            swap(*gradients[i], *buffered); // contents, not objects: the caller's matrix now holds the previous aggregate
            newGradients.push_back(buffered);
        }
        swap(*headerCPU, *m_bufferedHeader);
        // initiate aggregation only if any samples were processed in the previous iteration
        if (resetState || headerCPU->numSamples != 0)
        {
            // the gradients must have been computed before the side stream touches them
            if (cudaEventRecord(m_mainDone, nullptr) != cudaSuccess || cudaStreamWaitEvent(m_aggStream, m_mainDone, 0) != cudaSuccess)
                RuntimeError("AggregateGradients: cannot order the aggregation stream after the compute stream");
            Launch(newGradients, m_bufferedHeader, m_aggStream);
            m_pending = true;
            return true;
        }
        return false;
    }

private:
    // enqueue one aggregation of `gradients` on `stream` (header values are captured; they are summed in Finish)
    void Launch(const std::vector<Matrix<ElemType>*>& gradients, DistGradHeader* header, cudaStream_t stream)
    {
        if (header->numSamples == 0)
            for (auto* g : gradients)
                if (g->GetNumElements() && cudaMemsetAsync(g->Data(), 0, g->GetNumElements() * sizeof(ElemType), stream) != cudaSuccess)
                    RuntimeError("AggregateGradients: clearing the gradients of a rank without samples failed");
        for (size_t i = 0; i < gradients.size(); ++i)
            m_ptrs[i] = gradients[i]->Data();
        QaggCheck(Api::Step(m_agg, m_ptrs.data(), stream), "AggregateGradients");
    }
    // header: numSamples, numSamplesWithLabel, criterion and the eval pairs, summed over ranks; then wait for the step
    void Finish(DistGradHeader* header, cudaStream_t stream)
    {
        std::vector<double> h(3 + 2 * (size_t) header->numEvalNode);
        h[0] = header->criterion;
        h[1] = (double) header->numSamples;
        h[2] = (double) header->numSamplesWithLabel;
        for (int i = 0; i < header->numEvalNode; ++i)
        {
            h[3 + 2 * i] = header->evalErrors[i].first;
            h[4 + 2 * i] = (double) header->evalErrors[i].second;
        }
        QaggCheck(qagg_comm_allreduce_f64(m_mpi->Handle(), h.data(), (int) h.size(), stream), "header aggregation");
        header->criterion = h[0];
        header->numSamples = (size_t) h[1];
        header->numSamplesWithLabel = (size_t) h[2];
        for (int i = 0; i < header->numEvalNode; ++i)
        {
            header->evalErrors[i].first = h[3 + 2 * i];
            header->evalErrors[i].second = (size_t) h[4 + 2 * i];
        }
        if (cudaStreamSynchronize(stream) != cudaSuccess)
            RuntimeError("AggregateGradients: the aggregation step failed on the device");
    }

    void Initialize(const std::vector<Matrix<ElemType>*>& gradients, int numEvalNodes)
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
        QaggCheck(Api::Create(m_mpi->Handle(), (int) gradients.size(), M.data(), N.data(), m_nBits, flags, &m_agg), "qagg_agg_create");
        m_ptrs.resize(gradients.size());
        if (m_useAsync)
        {
            for (auto* g : gradients)
                m_buffered.push_back(std::unique_ptr<Matrix<ElemType>>(new Matrix<ElemType>(g->GetNumRows(), g->GetNumCols(), g->GetDeviceId())));
            m_bufferedHeader = DistGradHeader::Create(numEvalNodes);
            m_bufferedHeader->Clear();
            if (cudaStreamCreateWithFlags(&m_aggStream, cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&m_mainDone, cudaEventDisableTiming) != cudaSuccess)
                RuntimeError("AllReduceDistGradAggregator: cannot create the aggregation stream");
        }
        (void) m_traceLevel;
    }

    int m_nBits;
    bool m_zeroThr, m_selfQuant, m_useAsync;
    int m_traceLevel, m_syncStatsTrace;
    size_t m_iterationCount = 0;
    typename Api::Handle m_agg = nullptr;
    std::vector<ElemType*> m_ptrs;
    std::vector<size_t> m_rows, m_cols;
    // buffered asynchronous aggregation
    std::vector<std::unique_ptr<Matrix<ElemType>>> m_buffered;
    DistGradHeader* m_bufferedHeader = nullptr;
    cudaStream_t m_aggStream = nullptr;
    cudaEvent_t m_mainDone = nullptr;
    bool m_pending = false;
};

}}}
