// QuantizedDistributedCommunicator.h -- the V2 face of the same exchange: QuantizedAggregateInPlace with the contract of
// CNTK::QuantizedDistributedCommunicator (Source/CNTKv2LibraryDll/API/CNTKLibrary.h:6246-6259) and the factory
// QuantizedMPICommunicator(zeroThresholdFor1Bit, useQuantizationForSelfStripe, numQuantizationBits) (:6273), as
// implemented by QuantizedMPICommunicatorImpl (Source/1BitSGD/QuantizedDistributedCommunicator.h:47-99, 285-539).
//
// NDArrayView is reduced to what the path needs: a dense fp32 matrix view in device memory.  Differences kept from
// the reference: a single worker returns its inputs untouched (:75-81); all values must be float (:86-91, the double
// path is not built); sparse is refused (:215-216).  Residuals: the reference lets the caller own them as NDArrayViews
// created on first use (:246-261); here they live inside the aggregator (same lifetime as the communicator) and
// ResetResiduals() is what QuantizedDataParallelDistributedLearner::CreateCheckpoint does to them
// (Source/1BitSGD/QuantizedDataParallelDistributedLearner.h:73-91).
#pragma once

#include <memory>
#include <unordered_set>
#include <vector>

#include "MPIWrapper.h"
#include "Matrix.h"

namespace CNTK {

struct DistributedWorkerDescriptor
{
    size_t m_globalRank;
    bool IsMain() const { return m_globalRank == 0; }
    bool operator==(const DistributedWorkerDescriptor& o) const { return m_globalRank == o.m_globalRank; }
};

} // namespace CNTK

namespace std {
template <>
struct hash<::CNTK::DistributedWorkerDescriptor>
{
    size_t operator()(const ::CNTK::DistributedWorkerDescriptor& x) const { return std::hash<size_t>()(x.m_globalRank); }
};
} // namespace std

namespace CNTK {

typedef std::shared_ptr<Microsoft::MSR::CNTK::Matrix<float>> NDArrayViewPtr; // dense fp32 device matrix view

class QuantizedDistributedCommunicator
{
public:
    virtual ~QuantizedDistributedCommunicator() {}
    virtual const std::unordered_set<DistributedWorkerDescriptor>& Workers() const = 0;
    virtual const DistributedWorkerDescriptor& CurrentWorker() const = 0;
    virtual void QuantizedAggregateInPlace(std::vector<NDArrayViewPtr>& inValues, const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) = 0;
    virtual void AggregateInPlace(std::vector<double>& hostValues, const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) = 0;
    virtual void ResetResiduals() = 0;
    virtual void Barrier() = 0;
};
typedef std::shared_ptr<QuantizedDistributedCommunicator> QuantizedDistributedCommunicatorPtr;

class QuantizedMPICommunicatorImpl final : public QuantizedDistributedCommunicator
{
    using MPIWrapperPtr = Microsoft::MSR::CNTK::MPIWrapperPtr;

public:
    QuantizedMPICommunicatorImpl(const MPIWrapperPtr& mpi, bool zeroThresholdFor1Bit, bool useQuantizationForSelfStripe, size_t numQuantizationBits)
        : m_mpi(mpi), m_zeroThr(zeroThresholdFor1Bit), m_selfQuant(useQuantizationForSelfStripe), m_bits(numQuantizationBits)
    {
        for (size_t r = 0; r < mpi->NumNodesInUse(); ++r)
            m_workers.insert(DistributedWorkerDescriptor{r});
        m_me = DistributedWorkerDescriptor{mpi->CurrentNodeRank()};
    }
    ~QuantizedMPICommunicatorImpl() override
    {
        if (m_agg)
            qagg_agg_destroy(m_agg);
    }

    const std::unordered_set<DistributedWorkerDescriptor>& Workers() const override { return m_workers; }
    const DistributedWorkerDescriptor& CurrentWorker() const override { return m_me; }

    void QuantizedAggregateInPlace(std::vector<NDArrayViewPtr>& inValues, const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) override
    {
        using namespace Microsoft::MSR::CNTK;
        CheckWorkers(sendToWorkers);
        if (m_workers.size() == 1 || inValues.empty()) // no need to aggregate anything
            return;
        if (!m_agg)
        {
            std::vector<int64_t> M, N;
            for (auto& v : inValues)
            {
                if (v->GetMatrixType() != DENSE)
                    RuntimeError("Aggregation for sparse matrices is currently not supported!");
                M.push_back((int64_t) v->GetNumRows());
                N.push_back((int64_t) v->GetNumCols());
            }
            const int flags = (m_zeroThr ? QAGG_ZERO_THRESHOLD : 0) | (m_selfQuant ? QAGG_SELF_QUANTIZED : 0) | QAGG_V2_IDENTITY_K1;
            QaggCheck(qagg_agg_create(m_mpi->Handle(), (int) inValues.size(), M.data(), N.data(), (int) m_bits, flags, &m_agg), "qagg_agg_create");
            m_ptrs.resize(inValues.size());
        }
        if (inValues.size() != m_ptrs.size())
            LogicError("Number of aggregated values should be equal number of quantized residuals.");
        for (size_t i = 0; i < inValues.size(); ++i)
            m_ptrs[i] = inValues[i]->Data();
        QaggCheck(qagg_agg_step(m_agg, m_ptrs.data(), nullptr), "QuantizedAggregateInPlace");
        if (cudaStreamSynchronize(nullptr) != cudaSuccess)
            RuntimeError("QuantizedAggregateInPlace: the aggregation step failed on the device");
    }

    void AggregateInPlace(std::vector<double>& hostValues, const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) override
    {
        CheckWorkers(sendToWorkers);
        Microsoft::MSR::CNTK::QaggCheck(qagg_comm_allreduce_f64(m_mpi->Handle(), hostValues.data(), (int) hostValues.size(), nullptr), "AggregateInPlace");
    }

    void ResetResiduals() override
    {
        if (m_agg)
            Microsoft::MSR::CNTK::QaggCheck(qagg_agg_reset_residuals(m_agg, nullptr), "ResetResiduals");
    }

    void Barrier() override { m_mpi->WaitAll(); }

private:
    void CheckWorkers(const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) const
    {
        // Currently all operations should be executed on all workers (DistributedCommunicator.cpp:163-168)
        if (sendToWorkers != m_workers)
            Microsoft::MSR::CNTK::LogicError("Currently all operations should be executed on all workers");
    }

    MPIWrapperPtr m_mpi;
    bool m_zeroThr, m_selfQuant;
    size_t m_bits;
    std::unordered_set<DistributedWorkerDescriptor> m_workers;
    DistributedWorkerDescriptor m_me;
    qagg_aggregator* m_agg = nullptr;
    std::vector<float*> m_ptrs;
};

inline QuantizedDistributedCommunicatorPtr QuantizedMPICommunicator(const Microsoft::MSR::CNTK::MPIWrapperPtr& mpi, bool zeroThresholdFor1Bit,
                                                                    bool useQuantizationForSelfStripe, size_t numQuantizationBits)
{
    return std::make_shared<QuantizedMPICommunicatorImpl>(mpi, zeroThresholdFor1Bit, useQuantizationForSelfStripe, numQuantizationBits);
}

} // namespace CNTK
