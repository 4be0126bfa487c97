// MPIWrapper.h -- the slice of CNTK's MPIWrapper (Source/Common/Include/MPIWrapper.h:74-177) that
// IDistGradAggregator uses: rank / size / main-node queries and WaitAll.  There is no MPI here: the object wraps a
// qagg communicator (NCCL between device buffers).  The unique id that ties the ranks together is made on one rank with
// MPIWrapper::NewUniqueId() and handed to the others by whatever launcher started them (file, socket, torchrun store),
// as the reference does for NCCL with an MPI broadcast (Source/Math/NcclComm.cpp:96-111).
#pragma once

#include <memory>
#include <string>

#include "Basics.h"

namespace Microsoft { namespace MSR { namespace CNTK {

class MPIWrapper
{
public:
    static std::string NewUniqueId()
    {
        std::string id(QAGG_UNIQUE_ID_BYTES, '\0');
        QaggCheck(qagg_unique_id(&id[0]), "qagg_unique_id");
        return id;
    }

    // one rank of `numNodes` on CUDA device `deviceId`; numNodes == 1 needs no id
    MPIWrapper(const std::string& uniqueId, int rank, int numNodes, int deviceId)
    {
        QaggCheck(qagg_comm_create(numNodes > 1 ? uniqueId.data() : nullptr, rank, numNodes, deviceId, &m_comm), "qagg_comm_create");
    }
    ~MPIWrapper() { qagg_comm_destroy(m_comm); }
    DISABLE_COPY_AND_MOVE(MPIWrapper);

    size_t NumNodesInUse() const { return (size_t) qagg_comm_size(m_comm); }
    size_t CurrentNodeRank() const { return (size_t) qagg_comm_rank(m_comm); }
    bool IsMainNode() const { return CurrentNodeRank() == MainNodeRank(); }
    size_t MainNodeRank() const { return 0; }
    bool UsingAllNodes() const { return true; }
    void WaitAll() { QaggCheck(qagg_comm_barrier(m_comm, nullptr), "WaitAll"); }

    qagg_comm* Handle() const { return m_comm; }

    // The process-wide instance, as MPIWrapper::GetInstance (Source/Common/MPIWrapper.cpp:375-430) keeps one: the reference
    // creates it from MPI_COMM_WORLD on first use; here the launcher creates it (it knows rank, size and the unique id) and
    // registers it, and the factories that take no MPIWrapper argument (QuantizedMPICommunicator's reference signature) find
    // it.  GetInstance() returns null when none was registered.
    static std::shared_ptr<MPIWrapper>& InstanceSlot()
    {
        static std::shared_ptr<MPIWrapper> s_instance;
        return s_instance;
    }
    static void SetInstance(const std::shared_ptr<MPIWrapper>& mpi) { InstanceSlot() = mpi; }
    static std::shared_ptr<MPIWrapper> GetInstance() { return InstanceSlot(); }
    static void DeleteInstance() { InstanceSlot().reset(); }

private:
    qagg_comm* m_comm = nullptr;
};

typedef std::shared_ptr<MPIWrapper> MPIWrapperPtr;

}}}
