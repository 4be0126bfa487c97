// DataParallelSGD.h -- the data-parallel bookkeeping of SGD<ElemType> around the aggregator: which aggregator exists in which
// epoch, and the per-minibatch call.  It restates, over the mirror classes of this directory,
//   * the ParallelTrain / DataParallelSGD configuration and its checks (Source/SGDLib/SGD.cpp:3294-3343): gradientBits is a
//     PER-EPOCH array whose last value repeats (argvector indexing), each value in [1, 8 * sizeof(ElemType)];
//     parallelizationStartEpoch is 1-based and at least 1;
//   * InitDistGradAgg (SGD.cpp:2336-2359): gradientBits == 8 * sizeof(ElemType) creates the unquantized
//     SimpleDistGradAggregator, anything else _GetAllReduceDistGradAggregator (:2318-2328: the V2 aggregator over
//     QuantizedMPICommunicator when useV2Aggregator is set, else AllReduceDistGradAggregator with
//     useQuantizationForSelfStripe = true), and a fresh DistGradHeader for numEvalNodes;
//   * the (re-)initialisation at the start of training and whenever the epoch's gradientBits differ from the current
//     aggregator's (SGD.cpp:427-432, 553-559).  A new aggregator starts with zero residuals: the quantization error carried
//     by the old one is dropped, as in the reference;
//   * warm start: epochs before parallelizationStartEpoch do not aggregate (UsingGradientAggregation, SGD.h:634-637);
//   * the per-minibatch call m_distGradAgg->AggregateGradients(gradients, header, isFirstMinibatch) (SGD.cpp:1362-1376).
#pragma once

#include <memory>
#include <vector>

#include "AllReduceDistGradAggregator.h"
#include "SimpleDistGradAggregator.h"
#include "V2AllReduceDistGradAggregator.h"

namespace Microsoft { namespace MSR { namespace CNTK {

struct DataParallelSGDConfig
{
    std::vector<int> gradientBits;                        // per epoch; empty = 8 * sizeof(ElemType) = no quantization
    bool useZeroThresholdFor1BitQuantization = true;      // SGD.cpp:3297
    bool useBufferedAsyncGradientAggregation = false;     // SGD.cpp:3298
    int parallelizationStartEpoch = 1;                    // 1-based, as the user writes it (SGD.cpp:3317)
    bool useV2Aggregator = false;                         // SGD.cpp:3324-3326
    int syncPerfStats = 0;                                // SGD.cpp:3323
    int traceLevel = 0;
};

template <class ElemType>
class DataParallelSGD
{
public:
    DataParallelSGD(const MPIWrapperPtr& mpi, const DataParallelSGDConfig& config, int numEvalNodes, int deviceId)
        : m_mpi(mpi), m_config(config), m_numEvalNodes(numEvalNodes), m_deviceId(deviceId)
    {
        const int defaultGradientBits = 8 * (int) sizeof(ElemType);
        if (m_config.gradientBits.empty())
            m_config.gradientBits.push_back(defaultGradientBits);
        if (m_config.parallelizationStartEpoch < 1)
            InvalidArgument("parallelizationStartEpoch must be greater or equal to 1");
        for (int b : m_config.gradientBits)
            if (b < 1 || b > defaultGradientBits)
                InvalidArgument("gradientBits values must be in the range [1, 32] when using precision=float and in range [1, 64] when using precision=double.");
    }

    // gradientBits of a (0-based) epoch: the array's last value repeats
    int NumGradientBits(size_t epoch) const
    {
        return epoch < m_config.gradientBits.size() ? m_config.gradientBits[epoch] : m_config.gradientBits.back();
    }
    bool UsingGradientAggregation(size_t epoch) const { return (int) epoch >= m_config.parallelizationStartEpoch - 1; }

    // start of training at `startEpoch` (0-based; > 0 when resuming from a checkpoint)
    void BeginTraining(size_t startEpoch)
    {
        m_currentNumGradientBits = NumGradientBits(startEpoch);
        InitDistGradAgg(m_currentNumGradientBits);
    }
    // start of every epoch: a change of bit width replaces the aggregator
    void BeginEpoch(size_t epoch)
    {
        if (!m_distGradAgg)
            LogicError("DataParallelSGD: BeginTraining has not been called");
        if (m_currentNumGradientBits != NumGradientBits(epoch))
        {
            m_currentNumGradientBits = NumGradientBits(epoch);
            InitDistGradAgg(m_currentNumGradientBits);
        }
        m_epoch = epoch;
    }

    // One minibatch.  The caller has filled Header().  In an aggregating epoch the gradients and the header come back summed
    // over the workers; before parallelizationStartEpoch both are left as they are.  Returns whether any worker processed
    // samples.
    bool AggregateMinibatch(const std::vector<Matrix<ElemType>*>& gradients, bool isFirstMinibatch)
    {
        if (!UsingGradientAggregation(m_epoch))
            return m_gradHeader->numSamples > 0;
        return m_distGradAgg->AggregateGradients(gradients, m_gradHeader.get(), isFirstMinibatch);
    }

    DistGradHeader& Header() { return *m_gradHeader; }
    int CurrentNumGradientBits() const { return m_currentNumGradientBits; }
    IDistGradAggregator<ElemType>* Aggregator() { return m_distGradAgg.get(); }
    size_t TimesInitialized() const { return m_inits; }

private:
    void InitDistGradAgg(int numGradientBits)
    {
        m_distGradAgg.reset(); // the old aggregator's device buffers go before the new one's are allocated
        if (numGradientBits != 8 * (int) sizeof(ElemType))
        {
            if (m_config.traceLevel > 0)
                fprintf(stderr, "Initializing dataParallelSGD for %d-bit quantization.\n", numGradientBits);
            if (m_config.useV2Aggregator)
            {
                auto communicator = ::CNTK::QuantizedMPICommunicator(m_mpi, m_config.useZeroThresholdFor1BitQuantization, true, (size_t) numGradientBits);
                m_distGradAgg = std::make_shared<V2AllReduceDistGradAggregator<ElemType>>(communicator, m_config.useBufferedAsyncGradientAggregation,
                                                                                          m_config.traceLevel, m_config.syncPerfStats);
            }
            else
            {
                m_distGradAgg = std::make_shared<AllReduceDistGradAggregator<ElemType>>(m_mpi, numGradientBits, m_config.useZeroThresholdFor1BitQuantization, true,
                                                                                        m_config.useBufferedAsyncGradientAggregation, m_config.traceLevel,
                                                                                        m_config.syncPerfStats);
            }
        }
        else
        {
            if (m_config.traceLevel > 0)
                fprintf(stderr, "Initializing dataParallelSGD with FP%d aggregation.\n", numGradientBits);
            m_distGradAgg = std::make_shared<SimpleDistGradAggregator<ElemType>>(m_mpi, m_config.useBufferedAsyncGradientAggregation, m_deviceId,
                                                                                 m_config.syncPerfStats);
        }
        m_gradHeader.reset(DistGradHeader::Create(m_numEvalNodes), [](DistGradHeader* p) { DistGradHeader::Destroy(p); });
        ++m_inits;
    }

    MPIWrapperPtr m_mpi;
    DataParallelSGDConfig m_config;
    int m_numEvalNodes, m_deviceId;
    int m_currentNumGradientBits = 0;
    size_t m_epoch = 0, m_inits = 0;
    std::shared_ptr<IDistGradAggregator<ElemType>> m_distGradAgg;
    std::shared_ptr<DistGradHeader> m_gradHeader;
};

}}} // namespace Microsoft::MSR::CNTK
