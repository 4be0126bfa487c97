// QuantizedDataParallelDistributedLearner.h -- the V2 distributed learner of the quantized path, with the Update and
// CreateCheckpoint contract of Source/1BitSGD/QuantizedDataParallelDistributedLearner.h:19-91 and the factory
// CreateQuantizedDataParallelDistributedLearner (Source/CNTKv2LibraryDll/API/CNTKLibrary.h:5477).
//
// The V2 library's types are reduced to what this path touches: a Learner is anything with
// Update(gradients, sampleCount, sweepEnd); MinibatchInfo carries the sample count, the two criterion values and the
// end-of-sweep flag; the gradients arrive as an ordered vector of dense fp32 device views (the reference orders its
// parameter map first, ConvertToOrdered, :38).
// Kept from the reference: aggregation starts only once distributeAfterSamples samples have been seen (:31); an empty
// minibatch contributes zero gradients (:35-36); evalCriterion, trainingLoss and the sample count are summed over the
// workers BEFORE the gradients (:40-50) and the local learner is updated with the aggregated count (:69); an empty
// (aggregated) minibatch skips the local update and returns false (:66-67); the learner OWNS the two residual sets
// (m_residuals, m_stripeResiduals: created by the communicator on the first call and handed back through the vectors,
// :56-60) and CreateCheckpoint zeroes them, because they are not part of the checkpoint (:73-91);
// useAsyncBufferedParameterUpdate = true is a LogicError, as in the reference (:24-25).
#pragma once

#include <memory>
#include <vector>

#include "QuantizedDistributedCommunicator.h"

namespace CNTK {

struct MinibatchInfo
{
    bool atEndOfData = false;
    bool atEndOfSweep = false;
    size_t numberOfSamples = 0;
    double trainingLossValue = 0.0;
    double evalCriterionValue = 0.0;
    bool IsEmpty() const { return numberOfSamples == 0; }
};

class Learner
{
public:
    virtual ~Learner() {}
    // updates the parameters from their (aggregated) gradients; returns whether any parameter was updated
    virtual bool Update(std::vector<NDArrayViewPtr>& gradientValues, size_t trainingSampleCount, bool sweepEnd) = 0;
};
typedef std::shared_ptr<Learner> LearnerPtr;

class QuantizedDataParallelDistributedLearner
{
public:
    QuantizedDataParallelDistributedLearner(QuantizedDistributedCommunicatorPtr communicator, LearnerPtr learner, size_t distributeAfterSamples,
                                            bool useAsyncBufferedParameterUpdate)
        : m_communicator(communicator), m_learner(learner), m_distributeAfterSamples(distributeAfterSamples)
    {
        if (useAsyncBufferedParameterUpdate)
            Microsoft::MSR::CNTK::LogicError("Asynchronous parameter update is not yet supported.");
    }

    // called per minibatch after the gradients have been computed and before the model parameters are updated
    bool Update(std::vector<NDArrayViewPtr>& gradientValues, MinibatchInfo& info)
    {
        if (m_sampleCount >= m_distributeAfterSamples)
        {
            if (info.IsEmpty())
                for (auto& g : gradientValues)
                    g->SetValue(0);
            std::vector<double> header{info.evalCriterionValue, info.trainingLossValue, (double) info.numberOfSamples};
            m_communicator->AggregateInPlace(header, m_communicator->Workers());
            info.evalCriterionValue = header[0];
            info.trainingLossValue = header[1];
            info.numberOfSamples = (size_t) header[2];
            m_communicator->QuantizedAggregateInPlace(gradientValues, m_residuals, m_stripeResiduals, m_communicator->Workers());
        }
        m_sampleCount += info.numberOfSamples;
        if (info.IsEmpty())
            return false;
        return m_learner->Update(gradientValues, info.numberOfSamples, info.atEndOfSweep);
    }

    // The residuals are not checkpointed: zero them so that the in-memory state matches what a restart would see.
    // Returns the one piece of state the base class checkpoints here, the total sample count.
    size_t CreateCheckpoint()
    {
        for (auto& r : m_residuals)
            if (r)
                r->SetValue(0.0f);
        for (auto& r : m_stripeResiduals)
            if (r)
                r->SetValue(0.0f);
        return m_sampleCount;
    }
    void RestoreFromCheckpoint(size_t totalNumberOfSamplesSeen) { m_sampleCount = totalNumberOfSamplesSeen; }

    size_t TotalNumberOfSamplesSeen() const { return m_sampleCount; }
    // the residual views the learner holds (for inspection; call MaterializeResiduals() on the communicator before reading)
    const std::vector<NDArrayViewPtr>& Residuals() const { return m_residuals; }
    const std::vector<NDArrayViewPtr>& StripeResiduals() const { return m_stripeResiduals; }
    QuantizedDistributedCommunicatorPtr GetCommunicator() const { return m_communicator; }

private:
    QuantizedDistributedCommunicatorPtr m_communicator;
    LearnerPtr m_learner;
    size_t m_distributeAfterSamples;
    size_t m_sampleCount = 0;
    // residuals of quantized gradients and of the aggregated stripes this worker owns
    std::vector<NDArrayViewPtr> m_residuals;
    std::vector<NDArrayViewPtr> m_stripeResiduals;
};
typedef std::shared_ptr<QuantizedDataParallelDistributedLearner> DistributedLearnerPtr;

inline DistributedLearnerPtr CreateQuantizedDataParallelDistributedLearner(QuantizedDistributedCommunicatorPtr communicator, LearnerPtr learner,
                                                                          size_t distributeAfterSamples, bool useAsyncBufferedParameterUpdate = false)
{
    return std::make_shared<QuantizedDataParallelDistributedLearner>(communicator, learner, distributeAfterSamples, useAsyncBufferedParameterUpdate);
}

} // namespace CNTK
