// QuantizedMatrix.h -- QuantizedMatrix<float / double> with the reference's interface and byte layout
// (Source/Math/QuantizedMatrix.h:53-124, QuantizedMatrix.cpp:8-107): N packed columns of
// QuantizedColumnSize(bits, rows) bytes each; ColumnSlice(start, n) is the byte range [start*C, (start+n)*C).
// deviceId == CPUDEVICE puts the buffer in pinned host memory (what the reference aggregator uses as MPI buffers,
// AllReduceDistGradAggregator.h:88); deviceId >= 0 puts it in device memory.
#pragma once

#include <cuda_runtime.h>

#include <memory>

#include "Basics.h"

namespace Microsoft { namespace MSR { namespace CNTK {

class QuantizedMatrixBase
{
};

template <class ElemType>
class QuantizedMatrix : public QuantizedMatrixBase
{
    static_assert(sizeof(ElemType) == 4 || sizeof(ElemType) == 8, "ElemType is float (QWord = uint32) or double (QWord = uint64)");

public:
    QuantizedMatrix(size_t numRows, size_t numCols, size_t nbits, DEVICEID_TYPE deviceId, void* /*allocator*/ = nullptr)
        : m_numRows(numRows), m_numCols(numCols), m_numBits(nbits), m_deviceId(deviceId)
    {
        const int64_t c = sizeof(ElemType) == 8 ? qagg_packed_col_bytes_f64((int64_t) numRows, (int) nbits) : qagg_packed_col_bytes((int64_t) numRows, (int) nbits);
        if (c < 0)
            LogicError("QuantizedMatrix: nbits=%zu must be a power of two dividing the %zu-bit word", nbits, 8 * sizeof(ElemType)); // QuantizedMatrix.cpp:12-15
        m_qColSize = (size_t) c;
        const size_t bytes = m_qColSize * numCols != 0 ? m_qColSize * numCols : 1;
        void* p = nullptr;
        if (deviceId == CPUDEVICE)
        {
            if (cudaHostAlloc(&p, bytes, cudaHostAllocDefault) != cudaSuccess)
                RuntimeError("QuantizedMatrix: cudaHostAlloc of %zu bytes failed", bytes);
            m_owner = std::shared_ptr<void>(p, [](void* q) { cudaFreeHost(q); });
        }
        else
        {
            if (cudaSetDevice(deviceId) != cudaSuccess || cudaMalloc(&p, bytes) != cudaSuccess)
                RuntimeError("QuantizedMatrix: cudaMalloc of %zu bytes failed", bytes);
            m_owner = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
        }
        m_buffer = static_cast<char*>(p);
    }

    QuantizedMatrix(QuantizedMatrix&&) = default;
    QuantizedMatrix& operator=(QuantizedMatrix&&) = default;
    QuantizedMatrix(const QuantizedMatrix&) = delete;
    QuantizedMatrix& operator=(const QuantizedMatrix&) = delete;

    int GetDeviceId() const { return m_deviceId; }
    size_t GetNumRows() const { return m_numRows; }
    size_t GetNumCols() const { return m_numCols; }
    size_t GetNumBits() const { return m_numBits; }
    size_t GetSize() const { return m_qColSize * m_numCols; }
    char* Buffer() const { return m_buffer; }

    QuantizedMatrix ColumnSlice(size_t startColumn, size_t numCols) const
    {
        if (startColumn + numCols > m_numCols)
            LogicError("QuantizedMatrix::ColumnSlice: out of range");
        QuantizedMatrix s(*this, 0);
        s.m_buffer = m_buffer + startColumn * m_qColSize;
        s.m_numCols = numCols;
        return s;
    }

private:
    QuantizedMatrix(const QuantizedMatrix& o, int) // slice constructor
        : m_numRows(o.m_numRows), m_numCols(o.m_numCols), m_numBits(o.m_numBits), m_deviceId(o.m_deviceId),
          m_qColSize(o.m_qColSize), m_buffer(o.m_buffer), m_owner(o.m_owner)
    {
    }

    size_t m_numRows, m_numCols, m_numBits;
    DEVICEID_TYPE m_deviceId;
    size_t m_qColSize = 0;
    char* m_buffer = nullptr;
    std::shared_ptr<void> m_owner;
};

}}}
