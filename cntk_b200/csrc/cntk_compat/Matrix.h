// Matrix.h -- the part of CNTK's Matrix<ElemType> (Source/Math/Matrix.h) that the aggregation path touches:
// Data / GetNumRows / GetNumCols / GetNumElements / GetDeviceId / GetMatrixType / ColumnSlice / SetValue(0) / swap.
// Dense, column-major, in device memory (deviceId >= 0).  A Matrix either owns its buffer or is a column-slice view
// of another one (as Matrix::ColumnSlice returns in the reference: AllReduceDistGradAggregator.h:281).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <functional>
#include <memory>
#include <utility>

#include "Basics.h"

namespace Microsoft { namespace MSR { namespace CNTK {

template <class ElemType>
class Matrix
{
public:
    Matrix(size_t numRows, size_t numCols, DEVICEID_TYPE deviceId, MatrixType type = DENSE)
        : m_rows(numRows), m_cols(numCols), m_deviceId(deviceId)
    {
        if (type != DENSE)
            RuntimeError("Matrix: only dense matrices exist on this path");
        if (deviceId < 0)
            RuntimeError("Matrix: this build has no CPU path; pass a CUDA device id");
        if (cudaSetDevice(deviceId) != cudaSuccess)
            RuntimeError("Matrix: cudaSetDevice(%d) failed", deviceId);
        void* p = nullptr;
        const size_t bytes = (numRows * numCols != 0 ? numRows * numCols : 1) * sizeof(ElemType);
        if (cudaMalloc(&p, bytes) != cudaSuccess)
            RuntimeError("Matrix: cudaMalloc of %zu bytes failed", bytes);
        cudaMemset(p, 0, bytes); // CNTK matrices start zeroed (the residual relies on it, 1BitSGD/MatrixQuantizer.h:27-30)
        m_owner = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
        m_data = static_cast<ElemType*>(p);
    }

    // view over caller-owned device memory (what V2AllReduceDistGradAggregator does with NDArrayView, :251-258)
    Matrix(size_t numRows, size_t numCols, ElemType* deviceData, DEVICEID_TYPE deviceId)
        : m_rows(numRows), m_cols(numCols), m_deviceId(deviceId), m_data(deviceData)
    {
    }

    Matrix(const Matrix&) = default; // shallow, like a slice
    Matrix& operator=(const Matrix&) = default;

    ElemType* Data() const { return m_data; }
    size_t GetNumRows() const { return m_rows; }
    size_t GetNumCols() const { return m_cols; }
    size_t GetNumElements() const { return m_rows * m_cols; }
    DEVICEID_TYPE GetDeviceId() const { return m_deviceId; }
    MatrixType GetMatrixType() const { return DENSE; }

    Matrix ColumnSlice(size_t startColumn, size_t numCols) const
    {
        if (startColumn + numCols > m_cols)
            LogicError("ColumnSlice: columns [%zu, %zu) outside a matrix of %zu columns", startColumn, startColumn + numCols, m_cols);
        Matrix s(*this);
        s.m_data = m_data + startColumn * m_rows;
        s.m_cols = numCols;
        return s;
    }

    void SetValue(ElemType v)
    {
        if (v != ElemType(0))
            LogicError("Matrix::SetValue: only 0 is needed on this path");
        if (GetNumElements() && cudaMemset(m_data, 0, GetNumElements() * sizeof(ElemType)) != cudaSuccess)
            RuntimeError("Matrix::SetValue: cudaMemset failed");
        if (m_onWrite && *m_onWrite)
            (*m_onWrite)();
    }

    // A matrix that something else keeps derived state about (the communicator's residual views) tells it when its content
    // is overwritten through this interface.
    void NotifyOnWrite(std::function<void()> fn) { m_onWrite = std::make_shared<std::function<void()>>(std::move(fn)); }

    static void SetDevice(DEVICEID_TYPE deviceId)
    {
        if (cudaSetDevice(deviceId) != cudaSuccess)
            RuntimeError("Matrix::SetDevice(%d) failed", deviceId);
    }

    friend void swap(Matrix& a, Matrix& b)
    {
        std::swap(a.m_rows, b.m_rows);
        std::swap(a.m_cols, b.m_cols);
        std::swap(a.m_deviceId, b.m_deviceId);
        std::swap(a.m_data, b.m_data);
        std::swap(a.m_owner, b.m_owner);
        std::swap(a.m_onWrite, b.m_onWrite);
    }

private:
    size_t m_rows, m_cols;
    DEVICEID_TYPE m_deviceId;
    ElemType* m_data = nullptr;
    std::shared_ptr<void> m_owner;
    std::shared_ptr<std::function<void()>> m_onWrite;
};

}}}
