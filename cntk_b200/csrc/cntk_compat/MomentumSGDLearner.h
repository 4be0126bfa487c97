// MomentumSGDLearner.h -- the local learner the distributed learner hands the aggregated gradients to, reduced to the plain
// momentum-SGD rule: LearnerMomentumSGD::Update (Source/CNTKv2LibraryDll/Learner.cpp:610-622) ->
// Matrix<ElemType>::MomentumSGDUpdate (Source/Math/Matrix.cpp:1681-1698), i.e. per parameter matrix
//     smoothed = ScaleAndAdd(unitGainFactor * learningRate, gradient, momentum, smoothed);   parameter -= smoothed
// with unitGainFactor = 1 - momentum when the learner was created with unit gain, else 1 (Learner.h:203-212).
// Learning rate and momentum are per-call constants here (the reference looks both up in schedules keyed by the sample
// count; a schedule is a function of the count, which UpdateRuleFor receives).  Not covered, as in the fused kernel: mean-
// gradient scaling, clipping, regularisation, noise injection (LearnerBase::PreProcess, Learner.cpp:300-345).
//
// The class also implements FusableLearner: a distributed learner that aggregates through the quantized exchange may ask
// for the rule and the matrices BEFORE the exchange and let the exchange's last kernel apply the update straight from the
// packed aggregate (qagg_agg_set_update), instead of calling Update afterwards.
#pragma once

#include <functional>
#include <vector>

#include "QuantizedDataParallelDistributedLearner.h"

namespace CNTK {

class MomentumSGDLearner : public Learner, public FusableLearner
{
public:
    // parameters: one view per gradient, same order and shapes; the smoothed gradients start at zero
    MomentumSGDLearner(std::vector<NDArrayViewPtr> parameters, double learningRatePerSample, double momentum, bool unitGain)
        : m_parameters(std::move(parameters)), m_learningRate(learningRatePerSample), m_momentum(momentum), m_unitGain(unitGain)
    {
        for (const auto& p : m_parameters)
        {
            m_smoothed.push_back(std::make_shared<NDArrayView>(p->GetNumRows(), p->GetNumCols(), p->GetDeviceId()));
            m_smoothed.back()->SetValue(0.0f);
        }
    }

    bool Update(std::vector<NDArrayViewPtr>& gradientValues, size_t trainingSampleCount, bool /*sweepEnd*/) override
    {
        using namespace Microsoft::MSR::CNTK;
        if (gradientValues.size() != m_parameters.size())
            LogicError("MomentumSGDLearner: one gradient per parameter is expected");
        if (trainingSampleCount == 0)
            return false;
        float lr, momentum, unitGainFactor;
        UpdateRuleFor(trainingSampleCount, lr, momentum, unitGainFactor);
        for (size_t i = 0; i < m_parameters.size(); ++i)
        {
            if (gradientValues[i]->GetNumElements() != m_parameters[i]->GetNumElements())
                LogicError("MomentumSGDLearner: a gradient has a different size than its parameter");
            QaggCheck(qagg_sgd_update(nullptr, m_parameters[i]->Data(), gradientValues[i]->Data(), m_smoothed[i]->Data(),
                                      (int64_t) m_parameters[i]->GetNumElements(), lr, momentum, unitGainFactor),
                      "MomentumSGDUpdate");
        }
        NoteUpdate(trainingSampleCount);
        return true;
    }

    // FusableLearner
    void UpdateRuleFor(size_t /*trainingSampleCount*/, float& learningRate, float& momentum, float& unitGainFactor) const override
    {
        learningRate = (float) m_learningRate;
        momentum = (float) m_momentum;
        unitGainFactor = m_unitGain ? 1.0f - momentum : 1.0f;
    }
    const std::vector<NDArrayViewPtr>& Parameters() const override { return m_parameters; }
    const std::vector<NDArrayViewPtr>& SmoothedGradients() const override { return m_smoothed; }
    void NoteUpdate(size_t trainingSampleCount) override
    {
        m_sampleCount += trainingSampleCount;
        ++m_minibatchCount;
    }

    size_t TotalNumberOfSamplesSeen() const { return m_sampleCount; }
    size_t TotalNumberOfMinibatchesSeen() const { return m_minibatchCount; }

private:
    std::vector<NDArrayViewPtr> m_parameters, m_smoothed;
    double m_learningRate, m_momentum;
    bool m_unitGain;
    size_t m_sampleCount = 0, m_minibatchCount = 0;
};

} // namespace CNTK
