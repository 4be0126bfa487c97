// QuantizedDistributedCommunicator.h -- the V2 face of the exchange: QuantizedAggregate / QuantizedAggregateInPlace with the
// argument lists of CNTK::QuantizedDistributedCommunicator (Source/CNTKv2LibraryDll/API/CNTKLibrary.h:6246-6259) and the
// factory QuantizedMPICommunicator(zeroThresholdFor1Bit, useQuantizationForSelfStripe, numQuantizationBits) (:6273), as
// implemented by QuantizedMPICommunicatorImpl (Source/1BitSGD/QuantizedDistributedCommunicator.h:47-99, 179-283, 285-539).
//
// NDArrayView is reduced to what the path needs: a dense fp32 matrix view in device memory.  Kept from the reference:
//   * the residuals are the CALLER's: valueQuantizationResidues[i] (rows x columns of value i) and
//     stripeQuantizationResidues[i] (rows x the columns of value i this worker owns; stays null where it owns none).  Where
//     an entry is null the communicator creates it, zeroed, on first use and hands it back through the vector (:246-261);
//   * a single worker returns its inputs untouched, residuals included (:75-81);
//   * QuantizedAggregateInPlace is QuantizedAggregate with outputs = inputs (:51-61);
//   * "Number of aggregated values should be equal number of quantized residuals" (:186-193); all values must be float
//     (:86-91; double is not built); sparse is refused (:215-216); sendToWorkers must be all workers
//     (DistributedCommunicator.cpp:163-168).
// What the residual views hold: for 1 bit with threshold 0 the library keeps the error-feedback state in a deferred form
// between calls (see qagg_agg_bind_residuals in qagg.h).  Zeroing a view through SetValue(0) -- all the reference's callers
// ever do with one (QuantizedDataParallelDistributedLearner.h:73-91, V2AllReduceDistGradAggregator.h:78-98) -- is noticed
// and honoured; MaterializeResiduals() turns all views into plain residuals for a caller that wants to read them.
// MPI is replaced by the qagg communicator, so the factory takes the MPIWrapper that owns it as a first argument.
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

typedef Microsoft::MSR::CNTK::Matrix<float> NDArrayView; // dense fp32 device matrix view
typedef std::shared_ptr<NDArrayView> NDArrayViewPtr;

class DistributedCommunicator
{
public:
    virtual ~DistributedCommunicator() {}
    virtual const std::unordered_set<DistributedWorkerDescriptor>& Workers() const = 0;
    virtual const DistributedWorkerDescriptor& CurrentWorker() const = 0;
    // in-place sum of host values over all workers (the reference aggregates NDArrayViews on any device; the path only
    // ever passes the header's doubles, V2AllReduceDistGradAggregator.h:222-248, QuantizedDataParallelDistributedLearner.h:40-49)
    virtual void AggregateInPlace(std::vector<double>& hostValues, const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) = 0;
    virtual void Barrier() = 0;
};

class QuantizedDistributedCommunicator : public DistributedCommunicator
{
public:
    virtual void QuantizedAggregate(const std::vector<NDArrayViewPtr>& inValues, const std::vector<NDArrayViewPtr>& valueQuantizationResidues,
                                    const std::vector<NDArrayViewPtr>& stripeQuantizationResidues, std::vector<NDArrayViewPtr>& aggregatedOutputs,
                                    std::vector<NDArrayViewPtr>& newQuantizationResidues, std::vector<NDArrayViewPtr>& newStripeQuantizationResidues,
                                    const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) = 0;
    virtual void QuantizedAggregateInPlace(std::vector<NDArrayViewPtr>& inValues, std::vector<NDArrayViewPtr>& valueQuantizationResidues,
                                           std::vector<NDArrayViewPtr>& stripeQuantizationResidues,
                                           const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) = 0;
};
typedef std::shared_ptr<QuantizedDistributedCommunicator> QuantizedDistributedCommunicatorPtr;

class QuantizedMPICommunicatorImpl final : public QuantizedDistributedCommunicator
{
    using MPIWrapperPtr = Microsoft::MSR::CNTK::MPIWrapperPtr;

public:
    QuantizedMPICommunicatorImpl(const MPIWrapperPtr& mpi, bool zeroThresholdFor1Bit, bool useQuantizationForSelfStripe, size_t numQuantizationBits)
        : m_mpi(mpi), m_zeroThr(zeroThresholdFor1Bit), m_selfQuant(useQuantizationForSelfStripe), m_bits(numQuantizationBits),
          m_dirty(std::make_shared<bool>(false))
    {
        for (size_t r = 0; r < mpi->NumNodesInUse(); ++r)
            m_workers.insert(DistributedWorkerDescriptor{r});
        m_me = DistributedWorkerDescriptor{mpi->CurrentNodeRank()};
    }
    ~QuantizedMPICommunicatorImpl() override
    {
        if (m_agg)
            qagg_agg_destroy(m_agg);
        if (m_ready)
            cudaEventDestroy(m_ready);
        if (m_stream)
            cudaStreamDestroy(m_stream);
    }

    const std::unordered_set<DistributedWorkerDescriptor>& Workers() const override { return m_workers; }
    const DistributedWorkerDescriptor& CurrentWorker() const override { return m_me; }

    void QuantizedAggregateInPlace(std::vector<NDArrayViewPtr>& inValues, std::vector<NDArrayViewPtr>& valueQuantizationResidues,
                                   std::vector<NDArrayViewPtr>& stripeQuantizationResidues,
                                   const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) override
    {
        QuantizedAggregate(inValues, valueQuantizationResidues, stripeQuantizationResidues, inValues, valueQuantizationResidues,
                           stripeQuantizationResidues, sendToWorkers);
    }

    void QuantizedAggregate(const std::vector<NDArrayViewPtr>& inValues, const std::vector<NDArrayViewPtr>& formalValueQuantizationResidues,
                            const std::vector<NDArrayViewPtr>& formalStripeQuantizationResidues, std::vector<NDArrayViewPtr>& aggregatedOutputs,
                            std::vector<NDArrayViewPtr>& newQuantizationResidues, std::vector<NDArrayViewPtr>& newStripeQuantizationResidues,
                            const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) override
    {
        QuantizedAggregateAfter(nullptr, inValues, formalValueQuantizationResidues, formalStripeQuantizationResidues, aggregatedOutputs,
                                newQuantizationResidues, newStripeQuantizationResidues, sendToWorkers);
    }

    // The same, ordered after `inputsReady` (an event recorded where the inputs were produced) instead of after everything
    // the calling thread's default stream holds at the time of the call: what a caller on another host thread needs
    // (V2AllReduceDistGradAggregator's buffered asynchronous mode).  Returns when the results are complete.
    void QuantizedAggregateAfter(cudaEvent_t inputsReady, const std::vector<NDArrayViewPtr>& inValues,
                                 const std::vector<NDArrayViewPtr>& formalValueQuantizationResidues,
                                 const std::vector<NDArrayViewPtr>& formalStripeQuantizationResidues, std::vector<NDArrayViewPtr>& aggregatedOutputs,
                                 std::vector<NDArrayViewPtr>& newQuantizationResidues, std::vector<NDArrayViewPtr>& newStripeQuantizationResidues,
                                 const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers)
    {
        using namespace Microsoft::MSR::CNTK;
        CheckWorkers(sendToWorkers);
        if (m_workers.size() == 1) // no need to aggregate anything
        {
            aggregatedOutputs = inValues;
            newQuantizationResidues = formalValueQuantizationResidues;
            newStripeQuantizationResidues = formalStripeQuantizationResidues;
            return;
        }
        if (inValues.empty())
            return;
        const size_t n = inValues.size();
        const bool inPlaceResidues = (&formalValueQuantizationResidues == &newQuantizationResidues);
        auto valueResidues = formalValueQuantizationResidues;
        auto stripeResidues = formalStripeQuantizationResidues;
        // InitializeBuffers (:179-283)
        if (std::max(n, valueResidues.size()) != n)
            LogicError("Number of aggregated values should be equal number of quantized residuals.");
        if (std::max(n, stripeResidues.size()) != n)
            LogicError("Number of aggregated values should be equal number of striped quantized residuals.");
        if (aggregatedOutputs.size() != n)
            LogicError("QuantizedAggregate: one output view per value is expected.");
        valueResidues.resize(n);
        stripeResidues.resize(n);
        if (newQuantizationResidues.empty())
            newQuantizationResidues.resize(n);
        if (newStripeQuantizationResidues.empty())
            newStripeQuantizationResidues.resize(n);
        const int rank = (int) m_me.m_globalRank, K = (int) m_workers.size();
        std::vector<int64_t> M(n), N(n), stripeCols(n);
        for (size_t i = 0; i < n; ++i)
        {
            const auto& v = inValues[i];
            if (v->GetMatrixType() != DENSE)
                RuntimeError("Aggregation for sparse matrices is currently not supported!");
            M[i] = (int64_t) v->GetNumRows();
            N[i] = (int64_t) v->GetNumCols();
            int64_t start = 0;
            QaggCheck(qagg_stripe(N[i], rank, K, &start, &stripeCols[i]), "qagg_stripe");
            if (!valueResidues[i])
            {
                valueResidues[i] = MakeResidual(v->GetNumRows(), v->GetNumCols(), v->GetDeviceId());
                newQuantizationResidues[i] = inPlaceResidues ? valueResidues[i] : MakeResidual(v->GetNumRows(), v->GetNumCols(), v->GetDeviceId());
            }
            if (!stripeResidues[i] && stripeCols[i] > 0)
            {
                stripeResidues[i] = MakeResidual(v->GetNumRows(), (size_t) stripeCols[i], v->GetDeviceId());
                newStripeQuantizationResidues[i] = inPlaceResidues ? stripeResidues[i] : MakeResidual(v->GetNumRows(), (size_t) stripeCols[i], v->GetDeviceId());
            }
            if (!newQuantizationResidues[i] || (stripeCols[i] > 0 && !newStripeQuantizationResidues[i]))
                LogicError("QuantizedAggregate: an output residual view is missing.");
        }
        if (!m_agg)
        {
            const int flags = (m_zeroThr ? QAGG_ZERO_THRESHOLD : 0) | (m_selfQuant ? QAGG_SELF_QUANTIZED : 0) | QAGG_V2_IDENTITY_K1;
            QaggCheck(qagg_agg_create(m_mpi->Handle(), (int) n, M.data(), N.data(), (int) m_bits, flags, &m_agg), "qagg_agg_create");
            m_rows = M;
            m_cols = N;
            m_ptrs.resize(n);
            if (cudaStreamCreateWithFlags(&m_stream, cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&m_ready, cudaEventDisableTiming) != cudaSuccess)
                RuntimeError("QuantizedAggregate: cannot create the aggregation stream");
        }
        if (M != m_rows || N != m_cols)
            LogicError("QuantizedAggregate: the shapes of the values changed between calls");

        // the step runs on the communicator's own stream, after the inputs have been produced
        if (!inputsReady)
        {
            if (cudaEventRecord(m_ready, nullptr) != cudaSuccess)
                RuntimeError("QuantizedAggregate: cannot record on the compute stream");
            inputsReady = m_ready;
        }
        if (cudaStreamWaitEvent(m_stream, inputsReady, 0) != cudaSuccess)
            RuntimeError("QuantizedAggregate: cannot order the aggregation stream after the compute stream");

        // out of place: outputs and new residuals start as copies of the inputs, then everything happens in place in them
        for (size_t i = 0; i < n; ++i)
        {
            CopyIfDistinct(*aggregatedOutputs[i], *inValues[i]);
            CopyIfDistinct(*newQuantizationResidues[i], *valueResidues[i]);
            if (stripeCols[i] > 0)
                CopyIfDistinct(*newStripeQuantizationResidues[i], *stripeResidues[i]);
        }
        // (re)bind the residual buffers when they are not the ones of the previous call, or were written to since
        std::vector<float*> vres(n), sres(n);
        for (size_t i = 0; i < n; ++i)
        {
            vres[i] = newQuantizationResidues[i]->Data();
            sres[i] = stripeCols[i] > 0 ? newStripeQuantizationResidues[i]->Data() : nullptr;
        }
        const bool foreign = !inPlaceResidues; // distinct output residuals: plain residuals must be in them when the call returns
        if (vres != m_boundValue || sres != m_boundStripe || *m_dirty || foreign != m_boundPlain)
        {
            if (!m_boundValue.empty() && !*m_dirty && !m_boundPlain)
                QaggCheck(qagg_agg_materialize_residuals(m_agg, m_stream), "qagg_agg_materialize_residuals"); // leave the old buffers readable
            QaggCheck(qagg_agg_bind_residuals(m_agg, vres.data(), sres.data(), foreign ? 1 : 0), "qagg_agg_bind_residuals");
            m_boundValue = vres;
            m_boundStripe = sres;
            m_boundPlain = foreign;
            *m_dirty = false;
        }
        for (size_t i = 0; i < n; ++i)
            m_ptrs[i] = aggregatedOutputs[i]->Data();
        // a fused learner step, armed for this call only
        if (m_fuse.armed)
        {
            m_fuse.armed = false;
            if (m_fuse.params.size() != n || m_fuse.smoothed.size() != n)
                LogicError("QuantizedAggregate: one parameter and one smoothed-gradient view per value is expected");
            std::vector<float*> pp(n), ss(n);
            for (size_t i = 0; i < n; ++i)
            {
                if (m_fuse.params[i]->GetNumRows() != inValues[i]->GetNumRows() || m_fuse.params[i]->GetNumCols() != inValues[i]->GetNumCols() ||
                    m_fuse.smoothed[i]->GetNumElements() != inValues[i]->GetNumElements())
                    LogicError("QuantizedAggregate: a parameter view has a different shape than its gradient");
                pp[i] = m_fuse.params[i]->Data();
                ss[i] = m_fuse.smoothed[i]->Data();
            }
            if (pp != m_boundParams || ss != m_boundSmoothed)
            {
                QaggCheck(qagg_agg_bind_update(m_agg, pp.data(), ss.data()), "qagg_agg_bind_update");
                m_boundParams = pp;
                m_boundSmoothed = ss;
            }
            // the parameters were last written on the calling thread's stream: inputsReady already orders this step after that
            QaggCheck(qagg_agg_set_update(m_agg, 1, m_fuse.lr, m_fuse.momentum, m_fuse.unitGain), "qagg_agg_set_update");
        }
        else if (!m_boundParams.empty())
        {
            QaggCheck(qagg_agg_set_update(m_agg, 0, 0.0f, 0.0f, 1.0f), "qagg_agg_set_update");
        }
        QaggCheck(qagg_agg_step(m_agg, m_ptrs.data(), m_stream), "QuantizedAggregate");
        if (cudaStreamSynchronize(m_stream) != cudaSuccess)
            RuntimeError("QuantizedAggregate: the aggregation step failed on the device");
        QaggCheck(qagg_agg_check(m_agg, m_stream), "QuantizedAggregate");
        // hand created residual views back through the formal vectors, as the reference does for the in-place form
        if (inPlaceResidues)
        {
            newQuantizationResidues = valueResidues;
            newStripeQuantizationResidues = stripeResidues;
        }
    }

    void AggregateInPlace(std::vector<double>& hostValues, const std::unordered_set<DistributedWorkerDescriptor>& sendToWorkers) override
    {
        CheckWorkers(sendToWorkers);
        Microsoft::MSR::CNTK::QaggCheck(qagg_comm_allreduce_f64(m_mpi->Handle(), hostValues.data(), (int) hostValues.size(), nullptr), "AggregateInPlace");
    }

    // Arms the NEXT QuantizedAggregate / QuantizedAggregateInPlace call (more than one worker) to end in the momentum-SGD
    // update of `parameters` and `smoothedGradients` (one view per value, same shapes) instead of writing the aggregated
    // gradients: see qagg_agg_set_update.  No reference counterpart.
    void FuseUpdateIntoNextAggregate(const std::vector<NDArrayViewPtr>& parameters, const std::vector<NDArrayViewPtr>& smoothedGradients,
                                     float learningRate, float momentum, float unitGainFactor)
    {
        m_fuse.params = parameters;
        m_fuse.smoothed = smoothedGradients;
        m_fuse.lr = learningRate;
        m_fuse.momentum = momentum;
        m_fuse.unitGain = unitGainFactor;
        m_fuse.armed = true;
    }

    // turns every bound residual view into plain residuals (what a caller must do before reading them)
    void MaterializeResiduals()
    {
        if (!m_agg)
            return;
        Microsoft::MSR::CNTK::QaggCheck(qagg_agg_materialize_residuals(m_agg, m_stream), "qagg_agg_materialize_residuals");
        if (cudaStreamSynchronize(m_stream) != cudaSuccess)
            Microsoft::MSR::CNTK::RuntimeError("MaterializeResiduals failed on the device");
    }

    void Barrier() override { m_mpi->WaitAll(); }

private:
    // a zeroed residual view whose SetValue tells this communicator that its derived state is stale
    NDArrayViewPtr MakeResidual(size_t rows, size_t cols, DEVICEID_TYPE deviceId)
    {
        auto view = std::make_shared<NDArrayView>(rows, cols, deviceId);
        std::weak_ptr<bool> dirty = m_dirty;
        view->NotifyOnWrite([dirty]() {
            if (auto d = dirty.lock())
                *d = true;
        });
        return view;
    }

    void CopyIfDistinct(NDArrayView& dst, const NDArrayView& src)
    {
        using namespace Microsoft::MSR::CNTK;
        if (dst.Data() == src.Data())
            return;
        if (dst.GetNumRows() != src.GetNumRows() || dst.GetNumCols() != src.GetNumCols())
            LogicError("QuantizedAggregate: an output view has a different shape than its input");
        if (src.GetNumElements() &&
            cudaMemcpyAsync(dst.Data(), src.Data(), src.GetNumElements() * sizeof(float), cudaMemcpyDeviceToDevice, m_stream) != cudaSuccess)
            RuntimeError("QuantizedAggregate: copying an input into its output view failed");
    }

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
    struct
    {
        bool armed = false;
        std::vector<NDArrayViewPtr> params, smoothed;
        float lr = 0.0f, momentum = 0.0f, unitGain = 1.0f;
    } m_fuse;
    std::vector<float*> m_boundParams, m_boundSmoothed;
    std::vector<int64_t> m_rows, m_cols;
    std::vector<float*> m_ptrs, m_boundValue, m_boundStripe;
    bool m_boundPlain = false;
    std::shared_ptr<bool> m_dirty; // a residual view was written through SetValue since it was bound
    cudaStream_t m_stream = nullptr;
    cudaEvent_t m_ready = nullptr;
};

inline QuantizedDistributedCommunicatorPtr QuantizedMPICommunicator(const Microsoft::MSR::CNTK::MPIWrapperPtr& mpi, bool zeroThresholdFor1Bit,
                                                                    bool useQuantizationForSelfStripe, size_t numQuantizationBits)
{
    return std::make_shared<QuantizedMPICommunicatorImpl>(mpi, zeroThresholdFor1Bit, useQuantizationForSelfStripe, numQuantizationBits);
}

// the reference's own signature (Source/CNTKv2LibraryDll/API/CNTKLibrary.h:6273): over the process-wide MPIWrapper instance
inline QuantizedDistributedCommunicatorPtr QuantizedMPICommunicator(bool zeroThresholdFor1Bit, bool useQuantizationForSelfStripe, size_t numQuantizationBits)
{
    auto mpi = Microsoft::MSR::CNTK::MPIWrapper::GetInstance();
    if (!mpi)
        Microsoft::MSR::CNTK::RuntimeError("QuantizedMPICommunicator: no MPIWrapper instance has been registered (MPIWrapper::SetInstance)");
    return QuantizedMPICommunicator(mpi, zeroThresholdFor1Bit, useQuantizationForSelfStripe, numQuantizationBits);
}

} // namespace CNTK
