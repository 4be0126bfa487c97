// qagg_comm.h -- the communicator object behind include/qagg.h's qagg_comm, shared by the quantized aggregator
// (qagg_aggregator.cu) and the unquantized one (qagg_dense.cu).
#pragma once

#include <nccl.h>

struct qagg_comm
{
    int rank = 0;
    int K = 1;
    int device = 0;
    ncclComm_t nccl = nullptr;
    bool local = false; // member of an in-process group (device-to-device copies instead of NCCL)
    double* scalars = nullptr; // small device buffer for the header all-reduce
    static const int kMaxScalars = 512;
};
