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

// A learner whose update the quantized exchange can apply itself (no reference counterpart: the reference always writes the
// aggregated gradients and then calls Update).  The rule must be a function of the aggregated sample count alone, which the
// distributed learner knows before the gradients are exchanged (the header is summed first, :40-50 of the reference file).
class FusableLearner
{
public:
    virtual ~FusableLearner() {}
    virtual void UpdateRuleFor(size_t trainingSampleCount, float& learningRate, float& momentum, float& unitGainFactor) const = 0;
    virtual const std::vector<NDArrayViewPtr>& Parameters() const = 0;
    virtual const std::vector<NDArrayViewPtr>& SmoothedGradients() const = 0;
    virtual void NoteUpdate(size_t trainingSampleCount) = 0; // the bookkeeping Update would have done
};

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
            // consumer fusion: with the aggregated sample count known, the exchange's last kernel can take the learner's step
            // itself; the gradient views then keep the local gradients
            auto* fusable = m_fuseUpdate ? dynamic_cast<FusableLearner*>(m_learner.get()) : nullptr;
            auto* impl = dynamic_cast<QuantizedMPICommunicatorImpl*>(m_communicator.get());
            if (fusable && impl && !info.IsEmpty() && m_communicator->Workers().size() > 1)
            {
                float lr, momentum, unitGainFactor;
                fusable->UpdateRuleFor(info.numberOfSamples, lr, momentum, unitGainFactor);
                impl->FuseUpdateIntoNextAggregate(fusable->Parameters(), fusable->SmoothedGradients(), lr, momentum, unitGainFactor);
                m_communicator->QuantizedAggregateInPlace(gradientValues, m_residuals, m_stripeResiduals, m_communicator->Workers());
                fusable->NoteUpdate(info.numberOfSamples);
                m_sampleCount += info.numberOfSamples;
                return true;
            }
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

    // Lets the exchange apply the local learner's step when that learner is a FusableLearner (off by default: the
    // reference's behaviour -- aggregated gradients written, then Update -- is the default).
    void SetConsumerFusion(bool on) { m_fuseUpdate = on; }

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
    bool m_fuseUpdate = false;
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
