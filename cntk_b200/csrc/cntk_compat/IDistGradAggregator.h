// IDistGradAggregator.h -- interface of Source/SGDLib/IDistGradAggregator.h:8-39.
#pragma once

#include <vector>

#include "DistGradHeader.h"
#include "MPIWrapper.h"
#include "Matrix.h"

namespace Microsoft { namespace MSR { namespace CNTK {

template <class ElemType>
class IDistGradAggregator
{
public:
    IDistGradAggregator(const MPIWrapperPtr& mpi) : m_mpi(mpi) {}
    virtual ~IDistGradAggregator() {}

    // aggregates in place over all ranks; returns whether any samples were processed
    virtual bool AggregateGradients(const std::vector<Matrix<ElemType>*>& gradients, DistGradHeader* headerCPU, bool resetState) = 0;

    size_t NumProc() { return m_mpi->NumNodesInUse(); }
    size_t MyRank() { return m_mpi->CurrentNodeRank(); }
    void WaitAll() { m_mpi->WaitAll(); }

protected:
    MPIWrapperPtr m_mpi;
};

}}}
