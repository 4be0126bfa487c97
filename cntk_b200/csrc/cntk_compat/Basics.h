// Basics.h -- the handful of helpers the aggregation path uses from CNTK's Common/Include/Basics.h:
// exception helpers with printf-style messages (Basics.h:84-122), CPUDEVICE / DEVICEID_TYPE, DISABLE_COPY_AND_MOVE.
#pragma once

#include <cstdarg>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "../../../include/qagg.h"

#define DEVICEID_TYPE int
#define CPUDEVICE (-1)

#define DISABLE_COPY_AND_MOVE(TypeName)              \
    TypeName(const TypeName&) = delete;              \
    TypeName& operator=(const TypeName&) = delete;   \
    TypeName(TypeName&&) = delete;                   \
    TypeName& operator=(TypeName&&) = delete

namespace Microsoft { namespace MSR { namespace CNTK {

enum MatrixType { UNDETERMINED, DENSE, SPARSE };

template <class E>
[[noreturn]] inline void ThrowFormatted(const char* format, va_list args)
{
    char buffer[1024];
    vsnprintf(buffer, sizeof(buffer), format, args);
    throw E(buffer);
}

[[noreturn]] inline void RuntimeError(const char* format, ...)
{
    va_list args;
    va_start(args, format);
    ThrowFormatted<std::runtime_error>(format, args);
}
[[noreturn]] inline void LogicError(const char* format, ...)
{
    va_list args;
    va_start(args, format);
    ThrowFormatted<std::logic_error>(format, args);
}
[[noreturn]] inline void InvalidArgument(const char* format, ...)
{
    va_list args;
    va_start(args, format);
    ThrowFormatted<std::invalid_argument>(format, args);
}

// non-zero status of a C-ABI call -> the exception the reference would have thrown (its CUDA and MPI failures
// become RuntimeError: MatrixQuantizerGPU.cu:21-52, MPIWrapper.cpp:277-309)
inline void QaggCheck(int rc, const char* what)
{
    if (rc == QAGG_OK)
        return;
    if (rc == QAGG_EINVAL)
        InvalidArgument("%s: %s", what, qagg_last_error());
    if (rc == QAGG_ESTATE)
        LogicError("%s: %s", what, qagg_last_error());
    RuntimeError("%s: %s", what, qagg_last_error());
}

}}}
