// DistGradHeader.h -- per-minibatch scalars that travel with the gradients; same fields, layout and operations as
// Source/SGDLib/DistGradHeader.h:5-95 (a variable-size POD created with Create(numEvalNode) and freed with Destroy).
#pragma once

#include <cstddef>
#include <cstring>
#include <new>
#include <utility>

#include "Basics.h"

namespace Microsoft { namespace MSR { namespace CNTK {

struct DistGradHeader
{
    size_t numSamples;
    size_t numSamplesWithLabel; // denominator of `criterion`
    double criterion;
    int numEvalNode;
    std::pair<double, size_t> evalErrors[1]; // numEvalNode entries follow (numerator, denominator)

    static size_t BytesFor(int numEvalNode)
    {
        const int extra = numEvalNode > 1 ? numEvalNode - 1 : 0;
        return sizeof(DistGradHeader) + sizeof(std::pair<double, size_t>) * (size_t) extra;
    }
    static DistGradHeader* Create(int numEvalNode)
    {
        char* raw = new char[BytesFor(numEvalNode)];
        DistGradHeader* h = reinterpret_cast<DistGradHeader*>(raw);
        h->numEvalNode = numEvalNode;
        return h;
    }
    static void Destroy(DistGradHeader* h) { delete[] reinterpret_cast<char*>(h); }

    size_t Size() const { return BytesFor(numEvalNode); }

    void Clear()
    {
        numSamples = numSamplesWithLabel = 0;
        criterion = 0;
        for (int i = 0; i < numEvalNode; ++i)
            evalErrors[i] = std::make_pair(0.0, (size_t) 0);
    }

    // copy (add == false) or accumulate (add == true) another header of the same shape
    void Aggregate(DistGradHeader* other, bool add = false)
    {
        if (other->numEvalNode != numEvalNode)
            RuntimeError("mismatched size");
        if (!add)
        {
            std::memcpy((void*) this, (const void*) other, Size());
            return;
        }
        numSamples += other->numSamples;
        numSamplesWithLabel += other->numSamplesWithLabel;
        criterion += other->criterion;
        for (int i = 0; i < numEvalNode; ++i)
        {
            evalErrors[i].first += other->evalErrors[i].first;
            evalErrors[i].second += other->evalErrors[i].second;
        }
    }

    friend void swap(DistGradHeader& a, DistGradHeader& b)
    {
        if (a.numEvalNode != b.numEvalNode)
            LogicError("Cannot swap DistGradHeader objects with different number of evalNodes!");
        std::swap(a.numSamples, b.numSamples);
        std::swap(a.numSamplesWithLabel, b.numSamplesWithLabel);
        std::swap(a.criterion, b.criterion);
        for (int i = 0; i < a.numEvalNode; ++i)
            std::swap(a.evalErrors[i], b.evalErrors[i]);
    }

private:
    DistGradHeader() = delete;
    ~DistGradHeader() = delete;
    DISABLE_COPY_AND_MOVE(DistGradHeader);
};

}}}
