// host_logic_check.cpp -- the parts of the C++ mirror that need no device: the data-parallel configuration checks and epoch
// bookkeeping of DataParallelSGD (Source/SGDLib/SGD.cpp:3294-3343; SGD.h:634-637), DistGradHeader's arithmetic
// (Source/SGDLib/DistGradHeader.h:5-95) and the process-wide MPIWrapper slot.  Exit code 0 = all checks hold.
#include <cstdio>

#include "../../cntk_b200/csrc/cntk_compat/DataParallelSGD.h"

using namespace Microsoft::MSR::CNTK;

int main()
{
    MPIWrapperPtr none;
    // gradientBits: per-epoch array, the last value repeats; parallelizationStartEpoch is 1-based
    DataParallelSGDConfig cfg;
    cfg.gradientBits = {1, 1, 4, 32};
    cfg.parallelizationStartEpoch = 3;
    DataParallelSGD<float> dp(none, cfg, 2, 0);
    const int want[] = {1, 1, 4, 32, 32, 32};
    for (int e = 0; e < 6; ++e)
        if (dp.NumGradientBits((size_t) e) != want[e])
            return 1;
    if (dp.UsingGradientAggregation(0) || dp.UsingGradientAggregation(1) || !dp.UsingGradientAggregation(2) || !dp.UsingGradientAggregation(7))
        return 2;
    // default: no quantization (8 * sizeof(ElemType) bits), aggregation from the first epoch
    DataParallelSGD<float> dflt(none, DataParallelSGDConfig(), 1, 0);
    if (dflt.NumGradientBits(0) != 32 || !dflt.UsingGradientAggregation(0))
        return 3;
    DataParallelSGD<double> dfltD(none, DataParallelSGDConfig(), 1, 0);
    if (dfltD.NumGradientBits(5) != 64)
        return 4;
    // range checks
    int refused = 0;
    for (int bad = 0; bad < 4; ++bad)
    {
        DataParallelSGDConfig c;
        if (bad == 0)
            c.gradientBits = {0};
        else if (bad == 1)
            c.gradientBits = {1, 33};
        else if (bad == 2)
            c.parallelizationStartEpoch = 0;
        else
            c.gradientBits = {-4};
        try { DataParallelSGD<float> x(none, c, 1, 0); } catch (const std::invalid_argument&) { ++refused; }
    }
    if (refused != 4)
        return 5;
    { // 64 bits are fine for double, 33..64 are not for float
        DataParallelSGDConfig c;
        c.gradientBits = {64};
        DataParallelSGD<double> ok(none, c, 1, 0);
        bool threw = false;
        try { DataParallelSGD<float> x(none, c, 1, 0); } catch (const std::invalid_argument&) { threw = true; }
        if (!threw)
            return 6;
    }
    // BeginEpoch before BeginTraining is a logic error
    {
        bool threw = false;
        try { dp.BeginEpoch(0); } catch (const std::logic_error&) { threw = true; }
        if (!threw)
            return 7;
    }
    // DistGradHeader: Aggregate(add) sums every field, Clear zeroes them
    DistGradHeader* a = DistGradHeader::Create(2);
    DistGradHeader* b = DistGradHeader::Create(2);
    a->Clear();
    b->Clear();
    a->numSamples = 3; a->numSamplesWithLabel = 2; a->criterion = 1.5; a->evalErrors[0] = {0.25, 4}; a->evalErrors[1] = {1.0, 1};
    b->numSamples = 5; b->numSamplesWithLabel = 5; b->criterion = 2.0; b->evalErrors[0] = {0.5, 6}; b->evalErrors[1] = {2.0, 3};
    a->Aggregate(b, true);
    if (a->numSamples != 8 || a->numSamplesWithLabel != 7 || a->criterion != 3.5 || a->evalErrors[0].first != 0.75 || a->evalErrors[0].second != 10 ||
        a->evalErrors[1].first != 3.0 || a->evalErrors[1].second != 4)
        return 8;
    a->Aggregate(b, false); // add = false: assignment
    if (a->numSamples != 5 || a->criterion != 2.0 || a->evalErrors[1].second != 3)
        return 9;
    a->Clear();
    if (a->numSamples != 0 || a->criterion != 0.0 || a->evalErrors[0].second != 0)
        return 10;
    DistGradHeader::Destroy(a);
    DistGradHeader::Destroy(b);
    // the process-wide MPIWrapper slot starts empty
    if (MPIWrapper::GetInstance())
        return 11;
    bool threw = false;
    try { ::CNTK::QuantizedMPICommunicator(true, true, 1); } catch (const std::runtime_error&) { threw = true; }
    if (!threw)
        return 12;
    printf("host logic ok\n");
    return 0;
}
