// qagg_update.cu -- the learner step that follows aggregation, for the plain momentum-SGD learner
// (SGD<ElemType>::TypedUpdateWeights with GradientsUpdateType::None, Source/SGDLib/SGD.cpp:2509-2527; V2:
// LearnerMomentumSGD::Update, Source/CNTKv2LibraryDll/Learner.cpp:610-645; both end in Matrix<ElemType>::MomentumSGDUpdate,
// Source/Math/Matrix.cpp:1681-1698).
//
// Two forms of the same arithmetic (qagg_internal.h: UpdateRule, qagg_device.cuh: sgd_apply):
//   * fused into the unquantize kernel (qagg_unquantize.cu, mode UNQ_UPDATE): the aggregated gradient is consumed as it is
//     expanded and never written; per value the step then moves 16 bytes + its share of the packed words instead of
//     4 (gradient write) + 20 (gradient read, smoothed and parameter read and write);
//   * the plain kernel below over a gradient that is in memory -- the unfused arm the fused one is compared with, and the
//     update for gradients that did not come through the quantized exchange.
// Not covered (the caller keeps its own update for these): gradient clipping, L1/L2 regularisation, update noise, Nesterov
// momentum, AdaGrad/RmsProp/FSAdaGrad (SGD.cpp:2490-2508, 2528-2570).
#include "../../include/qagg.h"
#include "qagg_device.cuh"

#include <algorithm>

namespace qagg {

UpdateRule make_update_rule(float learnRatePerSample, float momentum, float unitGainFactor)
{
    UpdateRule r;
    const float alpha = unitGainFactor * learnRatePerSample;
    r.beta = momentum;
    if (momentum == 1.0f)
    {
        r.kind = 0;
        r.a = alpha;
    }
    else if (momentum == 0.0f)
    {
        r.kind = 1;
        r.a = alpha;
    }
    else
    {
        r.kind = 2;
        r.a = alpha / momentum;
    }
    return r;
}

// Grid-stride over 16-byte vectors; the ragged head and tail (unaligned base, n not a multiple of 4) go value by value.
__global__ void __launch_bounds__(NT) k_sgd_update(float* __restrict__ params, const float* __restrict__ grads, float* __restrict__ smoothed, long long n,
                                                   const UpdateRule rule, int vec)
{
    const long long tid = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long) gridDim.x * blockDim.x;
    if (vec)
    {
        const long long n4 = n >> 2;
        float4* p4 = reinterpret_cast<float4*>(params);
        const float4* g4 = reinterpret_cast<const float4*>(grads);
        float4* s4 = reinterpret_cast<float4*>(smoothed);
        for (long long i = tid; i < n4; i += nthreads)
        {
            const float4 g = __ldcs(g4 + i);
            float4 s = __ldcs(s4 + i);
            float4 w = __ldcs(p4 + i);
            w.x = sgd_apply(rule, g.x, s.x, w.x);
            w.y = sgd_apply(rule, g.y, s.y, w.y);
            w.z = sgd_apply(rule, g.z, s.z, w.z);
            w.w = sgd_apply(rule, g.w, s.w, w.w);
            __stcs(s4 + i, s);
            __stcs(p4 + i, w);
        }
        for (long long i = (n4 << 2) + tid; i < n; i += nthreads)
        {
            float s = smoothed[i];
            params[i] = sgd_apply(rule, grads[i], s, params[i]);
            smoothed[i] = s;
        }
    }
    else
    {
        for (long long i = tid; i < n; i += nthreads)
        {
            float s = smoothed[i];
            params[i] = sgd_apply(rule, grads[i], s, params[i]);
            smoothed[i] = s;
        }
    }
}

cudaError_t launch_sgd_update(cudaStream_t st, float* params, const float* grads, float* smoothed, long long n, const UpdateRule& rule, int numSMs)
{
    if (n <= 0)
        return cudaSuccess;
    const int vec = (((uintptr_t) params | (uintptr_t) grads | (uintptr_t) smoothed) & 15) == 0;
    const long long perThread = vec ? 4 : 1;
    const long long need = (n + NT * perThread - 1) / (NT * perThread);
    const int grid = (int) std::min<long long>(need, (long long) numSMs * 8);
    k_sgd_update<<<grid, NT, 0, st>>>(params, grads, smoothed, n, rule, vec);
    return cudaGetLastError();
}

} // namespace qagg

using namespace qagg;

extern "C" {

int qagg_sgd_update(void* stream, float* params, const float* grads, float* smoothed, int64_t n, float learn_rate_per_sample, float momentum,
                    float unit_gain_factor)
{
    if (n < 0)
        return fail(QAGG_EINVAL, "qagg_sgd_update: negative size");
    if (n == 0)
        return QAGG_OK;
    if (!params || !grads || !smoothed)
        return fail(QAGG_EINVAL, "qagg_sgd_update: null pointer");
    if (!(momentum >= 0.0f && momentum <= 1.0f))
        return fail(QAGG_EINVAL, "qagg_sgd_update: momentum must lie in [0, 1]");
    LaunchCfg cfg;
    int rc = launch_cfg_for_current_device(&cfg);
    if (rc)
        return rc;
    return check_cuda(launch_sgd_update((cudaStream_t) stream, params, grads, smoothed, n, make_update_rule(learn_rate_per_sample, momentum, unit_gain_factor),
                                        cfg.numSMs), "update kernel launch");
}

int qagg_unquantize_sgd(void* stream, const void* packed, float* params, float* smoothed, int64_t M, int64_t N, int bits, float learn_rate_per_sample,
                        float momentum, float unit_gain_factor)
{
    int rc = check_dims(M, N, bits);
    if (rc)
        return rc;
    if (M == 0 || N == 0)
        return QAGG_OK;
    if (!packed || !params || !smoothed)
        return fail(QAGG_EINVAL, "qagg_unquantize_sgd: null pointer");
    if (!(momentum >= 0.0f && momentum <= 1.0f))
        return fail(QAGG_EINVAL, "qagg_unquantize_sgd: momentum must lie in [0, 1]");
    LaunchCfg cfg;
    rc = launch_cfg_for_current_device(&cfg);
    if (rc)
        return rc;
    QTensor t = {};
    fill_layout(&t, M, N, bits);
    t.out = params;
    t.res_out = smoothed;
    t.pk[0] = static_cast<unsigned char*>(const_cast<void*>(packed));
    const UpdateRule rule = make_update_rule(learn_rate_per_sample, momentum, unit_gain_factor);
    return check_cuda(launch_unquantize((cudaStream_t) stream, UNQ_UPDATE, bits, &t, nullptr, 1, unq_units(M, N, bits), unq_smem_words(M, bits), cfg, &rule),
                      "unquantize-update kernel launch");
}

} // extern "C"
