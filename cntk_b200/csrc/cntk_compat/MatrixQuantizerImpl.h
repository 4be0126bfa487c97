// MatrixQuantizerImpl.h -- MatrixQuantizerImpl<float / double> with the reference's interface
// (Source/Math/MatrixQuantizerImpl.h:18-49), implemented over the C ABI of libqagg.
//   QuantizeAsync(in, inResidual, outQ, outResidual, zeroThresholdFor1Bit)   inResidual may alias outResidual
//   WaitQuantizeAsyncDone()
//   UnquantizeAsync(inQ, out, add = false)
//   WaitUnquantizeAsyncDone()
// The packed matrix may live on the CPU (pinned; the reference's only supported case, MatrixQuantizerGPU.cu:243) or
// on the device.  Create(CPUDEVICE, ...) throws: this build has no CPU quantizer.
#pragma once

#include <cuda_runtime.h>

#include "Matrix.h"
#include "QuantizedMatrix.h"

namespace Microsoft { namespace MSR { namespace CNTK {

// the C entry points of the two element types behind one name
inline int QaggQuantize(void* st, const float* g, const float* ri, float* ro, void* p, int64_t M, int64_t N, int bits, int z)
{
    return qagg_quantize(st, g, ri, ro, p, M, N, bits, z);
}
inline int QaggQuantize(void* st, const double* g, const double* ri, double* ro, void* p, int64_t M, int64_t N, int bits, int z)
{
    return qagg_quantize_f64(st, g, ri, ro, p, M, N, bits, z);
}
inline int QaggUnquantize(void* st, const void* p, float* out, int64_t M, int64_t N, int bits, int add)
{
    return qagg_unquantize(st, p, out, M, N, bits, add);
}
inline int QaggUnquantize(void* st, const void* p, double* out, int64_t M, int64_t N, int bits, int add)
{
    return qagg_unquantize_f64(st, p, out, M, N, bits, add);
}

template <class ElemType>
class MatrixQuantizerImpl
{
public:
    static MatrixQuantizerImpl<ElemType>* Create(int deviceId, bool useAsync);
    virtual ~MatrixQuantizerImpl() {}
    DISABLE_COPY_AND_MOVE(MatrixQuantizerImpl);

    virtual void QuantizeAsync(const Matrix<ElemType>& inMatrix, const Matrix<ElemType>& inResidual, QuantizedMatrix<ElemType>& outQMatrix,
                               Matrix<ElemType>& outResidual, bool zeroThresholdFor1Bit) = 0;
    virtual void WaitQuantizeAsyncDone() = 0;
    virtual void UnquantizeAsync(QuantizedMatrix<ElemType>& inQMatrix, Matrix<ElemType>& outMatrix, bool add = false) = 0;
    virtual void WaitUnquantizeAsyncDone() = 0;

    int GetDeviceId() const { return m_deviceId; }

protected:
    MatrixQuantizerImpl(int deviceId) : m_deviceId(deviceId) {}

private:
    int m_deviceId;
};

// the B200 implementation: one private stream; a grow-only device staging buffer when the packed matrix is on the host
// (the counterpart of MatrixQuantizerGPU::GetTempGPUQuantizedMatrix, MatrixQuantizerGPU.cu:158-179)
template <class ElemType>
class MatrixQuantizerB200 final : public MatrixQuantizerImpl<ElemType>
{
public:
    MatrixQuantizerB200(int deviceId, bool /*useAsync*/) : MatrixQuantizerImpl<ElemType>(deviceId)
    {
        if (cudaSetDevice(deviceId) != cudaSuccess || cudaStreamCreateWithFlags(&m_stream, cudaStreamNonBlocking) != cudaSuccess)
            RuntimeError("MatrixQuantizerB200: cannot create a stream on device %d", deviceId);
    }
    ~MatrixQuantizerB200() override
    {
        cudaStreamSynchronize(m_stream);
        cudaStreamDestroy(m_stream);
        if (m_scratch)
            cudaFree(m_scratch);
    }

    void QuantizeAsync(const Matrix<ElemType>& in, const Matrix<ElemType>& inResidual, QuantizedMatrix<ElemType>& outQ,
                       Matrix<ElemType>& outResidual, bool zeroThresholdFor1Bit) override
    {
        const size_t M = in.GetNumRows(), N = in.GetNumCols();
        if (outQ.GetNumRows() != M || outQ.GetNumCols() != N || inResidual.GetNumRows() != M || inResidual.GetNumCols() != N ||
            outResidual.GetNumRows() != M || outResidual.GetNumCols() != N)
            LogicError("QuantizeAsync: mismatched dimensions");
        const int bits = (int) outQ.GetNumBits();
        if (outQ.GetDeviceId() == CPUDEVICE)
        {
            // kernel, then copy to the host buffer on the same stream; completion is observed in WaitQuantizeAsyncDone
            QaggCheck(QaggQuantize(m_stream, in.Data(), inResidual.Data(), outResidual.Data(), Scratch(outQ.GetSize()), (int64_t) M, (int64_t) N, bits,
                                    zeroThresholdFor1Bit ? 1 : 0), "QuantizeAsync");
            if (outQ.GetSize() && cudaMemcpyAsync(outQ.Buffer(), m_scratch, outQ.GetSize(), cudaMemcpyDeviceToHost, m_stream) != cudaSuccess)
                RuntimeError("QuantizeAsync: copy of the packed matrix to the host failed");
        }
        else
        {
            QaggCheck(QaggQuantize(m_stream, in.Data(), inResidual.Data(), outResidual.Data(), outQ.Buffer(), (int64_t) M, (int64_t) N, bits,
                                    zeroThresholdFor1Bit ? 1 : 0), "QuantizeAsync");
        }
    }
    void WaitQuantizeAsyncDone() override { Sync("WaitQuantizeAsyncDone"); }

    void UnquantizeAsync(QuantizedMatrix<ElemType>& inQ, Matrix<ElemType>& out, bool add = false) override
    {
        const size_t M = inQ.GetNumRows(), N = inQ.GetNumCols();
        if (out.GetNumRows() != M || out.GetNumCols() != N)
            LogicError("UnquantizeAsync: mismatched dimensions");
        const int bits = (int) inQ.GetNumBits();
        const void* packed = inQ.Buffer();
        if (inQ.GetDeviceId() == CPUDEVICE)
        {
            if (inQ.GetSize() && cudaMemcpyAsync(Scratch(inQ.GetSize()), inQ.Buffer(), inQ.GetSize(), cudaMemcpyHostToDevice, m_stream) != cudaSuccess)
                RuntimeError("UnquantizeAsync: copy of the packed matrix to the device failed");
            packed = m_scratch;
        }
        QaggCheck(QaggUnquantize(m_stream, packed, out.Data(), (int64_t) M, (int64_t) N, bits, add ? 1 : 0), "UnquantizeAsync");
    }
    void WaitUnquantizeAsyncDone() override { Sync("WaitUnquantizeAsyncDone"); }

    cudaStream_t Stream() const { return m_stream; }

private:
    void* Scratch(size_t bytes)
    {
        if (bytes > m_scratchBytes)
        {
            cudaStreamSynchronize(m_stream);
            if (m_scratch)
                cudaFree(m_scratch);
            m_scratch = nullptr;
            if (cudaMalloc(&m_scratch, bytes) != cudaSuccess)
                RuntimeError("MatrixQuantizerB200: cudaMalloc of %zu staging bytes failed", bytes);
            m_scratchBytes = bytes;
        }
        return m_scratch;
    }
    void Sync(const char* what)
    {
        if (cudaStreamSynchronize(m_stream) != cudaSuccess)
            RuntimeError("%s: cudaStreamSynchronize failed", what);
    }

    cudaStream_t m_stream = nullptr;
    void* m_scratch = nullptr;
    size_t m_scratchBytes = 0;
};

template <class ElemType>
MatrixQuantizerImpl<ElemType>* MatrixQuantizerImpl<ElemType>::Create(int deviceId, bool useAsync)
{
    if (deviceId == CPUDEVICE)
        RuntimeError("MatrixQuantizerImpl::Create: this build has no CPU quantizer (no CPU fallback); pass a CUDA device id");
    return new MatrixQuantizerB200<ElemType>(deviceId, useAsync);
}

}}}
