// MatrixQuantizer.h -- the residual-owning wrapper, interface of Source/1BitSGD/MatrixQuantizer.h:24-85.
#pragma once

#include <memory>

#include "MatrixQuantizerImpl.h"

namespace Microsoft { namespace MSR { namespace CNTK {

class MatrixQuantizerBase
{
};

template <class ElemType>
class MatrixQuantizer final : public MatrixQuantizerBase
{
public:
    MatrixQuantizer(size_t numRows, size_t numCols, int deviceId, bool useAsync) : MatrixQuantizer(deviceId, useAsync)
    {
        m_residual = std::make_shared<Matrix<ElemType>>(numRows, numCols, deviceId, DENSE);
    }
    MatrixQuantizer(int deviceId, bool useAsync) : m_residual(nullptr)
    {
        m_quantizerImpl.reset(MatrixQuantizerImpl<ElemType>::Create(deviceId, useAsync));
    }
    DISABLE_COPY_AND_MOVE(MatrixQuantizer);

    void QuantizeAsync(const Matrix<ElemType>& inMatrix, QuantizedMatrix<ElemType>& outQMatrix, bool zeroThresholdFor1Bit)
    {
        m_quantizerImpl->QuantizeAsync(inMatrix, *m_residual, outQMatrix, *m_residual, zeroThresholdFor1Bit);
    }
    void QuantizeAsync(const Matrix<ElemType>& inMatrix, const Matrix<ElemType>& inResidual, QuantizedMatrix<ElemType>& outQMatrix,
                       Matrix<ElemType>& outResidual, bool zeroThresholdFor1Bit)
    {
        m_quantizerImpl->QuantizeAsync(inMatrix, inResidual, outQMatrix, outResidual, zeroThresholdFor1Bit);
    }
    void WaitQuantizeAsyncDone() { m_quantizerImpl->WaitQuantizeAsyncDone(); }
    void UnquantizeAsync(QuantizedMatrix<ElemType>& inQMatrix, Matrix<ElemType>& outMatrix, bool add = false)
    {
        m_quantizerImpl->UnquantizeAsync(inQMatrix, outMatrix, add);
    }
    void WaitUnquantizeAsyncDone() { m_quantizerImpl->WaitUnquantizeAsyncDone(); }
    int GetDeviceId() const { return m_quantizerImpl->GetDeviceId(); }
    void ResetResidue() { m_residual->SetValue(0.0); }
    const Matrix<ElemType>& GetResidualMatrix() const { return *m_residual; }

private:
    std::unique_ptr<MatrixQuantizerImpl<ElemType>> m_quantizerImpl;
    std::shared_ptr<Matrix<ElemType>> m_residual;
};

}}}
