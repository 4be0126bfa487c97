// compat_check.cpp -- drives the C++ mirror of the reference interfaces the way the reference's own callers do and dumps
// the results for tests/test_gpu_compat.py to compare with the CPU oracle.
//   mode "quantizer": the loop of TestRunQuantization (Tests/UnitTests/MathTests/MatrixQuantizerTests.cpp:268-316):
//       MatrixQuantizerImpl::Create, QuantizeAsync(in, residue, CPU QuantizedMatrix, residue), UnquantizeAsync(add = it > 0)
//   mode "aggregator": AllReduceDistGradAggregator::AggregateGradients on one rank (SGD.cpp:1376), two calls
//   mode "aggregator_async": the same with useAsyncAggregation = true (one-step-stale results, AllReduceDistGradAggregator.h:156-229)
// usage: compat_check <mode> <in.bin> <out.bin> M N bits zeroThr iters
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../cntk_b200/csrc/cntk_compat/AllReduceDistGradAggregator.h"
#include "../../cntk_b200/csrc/cntk_compat/QuantizedDataParallelDistributedLearner.h"
#include "../../cntk_b200/csrc/cntk_compat/V2AllReduceDistGradAggregator.h"
#include "../../cntk_b200/csrc/cntk_compat/MatrixQuantizer.h"
#include "../../cntk_b200/csrc/cntk_compat/QuantizedDistributedCommunicator.h"

using namespace Microsoft::MSR::CNTK;

static std::vector<float> download(const Matrix<float>& m)
{
    std::vector<float> h(m.GetNumElements());
    cudaMemcpy(h.data(), m.Data(), h.size() * 4, cudaMemcpyDeviceToHost);
    return h;
}

int main(int argc, char** argv)
{
    if (argc < 9)
        return 2;
    const std::string mode = argv[1];
    const size_t M = atol(argv[4]), N = atol(argv[5]);
    const int bits = atoi(argv[6]), zeroThr = atoi(argv[7]), iters = atoi(argv[8]);
    FILE* fi = fopen(argv[2], "rb");
    FILE* fo = fopen(argv[3], "wb");
    if (!fi || !fo)
        return 3;
    std::vector<float> in(M * N);
    try
    {
        if (mode == "quantizer")
        {
            std::unique_ptr<MatrixQuantizerImpl<float>> q(MatrixQuantizerImpl<float>::Create(0, false));
            Matrix<float> inM(M, N, 0), residue(M, N, 0), out(M, N, 0);
            for (int it = 0; it < iters; ++it)
            {
                if (fread(in.data(), 4, in.size(), fi) != in.size())
                    return 4;
                cudaMemcpy(inM.Data(), in.data(), in.size() * 4, cudaMemcpyHostToDevice);
                QuantizedMatrix<float> packed(M, N, bits, CPUDEVICE);
                q->QuantizeAsync(inM, residue, packed, residue, zeroThr != 0);
                q->WaitQuantizeAsyncDone();
                q->UnquantizeAsync(packed, out, it > 0);
                q->WaitUnquantizeAsyncDone();
                fwrite(packed.Buffer(), 1, packed.GetSize(), fo);
                auto r = download(residue), o = download(out);
                fwrite(r.data(), 4, r.size(), fo);
                fwrite(o.data(), 4, o.size(), fo);
            }
            // error behaviour: a CPU quantizer does not exist, and 3 bits is not a legal width
            bool threw = false;
            try { MatrixQuantizerImpl<float>::Create(CPUDEVICE, false); } catch (const std::runtime_error&) { threw = true; }
            if (!threw) return 5;
            threw = false;
            try { QuantizedMatrix<float> bad(8, 8, 3, CPUDEVICE); } catch (const std::logic_error&) { threw = true; }
            if (!threw) return 6;
        }
        else if (mode == "aggregator")
        {
            auto mpi = std::make_shared<MPIWrapper>(std::string(), 0, 1, 0);
            AllReduceDistGradAggregator<float> agg(mpi, bits, zeroThr != 0, true, false, 0, 0);
            Matrix<float> g0(M, N, 0), g1(M, 1, 0);
            std::vector<Matrix<float>*> grads{&g0, &g1};
            DistGradHeader* hdr = DistGradHeader::Create(1);
            for (int it = 0; it < iters; ++it)
            {
                if (fread(in.data(), 4, in.size(), fi) != in.size())
                    return 4;
                cudaMemcpy(g0.Data(), in.data(), in.size() * 4, cudaMemcpyHostToDevice);
                cudaMemcpy(g1.Data(), in.data(), M * 4, cudaMemcpyHostToDevice);
                hdr->Clear();
                hdr->numSamples = 7;
                hdr->criterion = 1.5;
                const bool any = agg.AggregateGradients(grads, hdr, it == 0);
                if (!any || hdr->numSamples != 7 || hdr->criterion != 1.5)
                    return 7;
                auto a = download(g0), b = download(g1);
                fwrite(a.data(), 4, a.size(), fo);
                fwrite(b.data(), 4, b.size(), fo);
            }
            // a rank without samples contributes zeros and reports "nothing processed"
            hdr->Clear();
            if (agg.AggregateGradients(grads, hdr, false))
                return 8;
            DistGradHeader::Destroy(hdr);
            // V2 face: one worker leaves its inputs untouched
            auto comm = ::CNTK::QuantizedMPICommunicator(mpi, true, true, 1);
            auto view = std::make_shared<Matrix<float>>(M, N, 0);
            cudaMemcpy(view->Data(), in.data(), in.size() * 4, cudaMemcpyHostToDevice);
            std::vector<::CNTK::NDArrayViewPtr> vals{view};
            comm->QuantizedAggregateInPlace(vals, comm->Workers());
            auto v = download(*view);
            if (memcmp(v.data(), in.data(), in.size() * 4) != 0)
                return 9;

            // V2AllReduceDistGradAggregator: the IDistGradAggregator face of the V2 communicator (one worker: identity)
            {
                V2AllReduceDistGradAggregator<float> v2agg(comm, false, 0, 0);
                std::vector<Matrix<float>*> vg{view.get()};
                DistGradHeader* h2 = DistGradHeader::Create(1);
                h2->Clear();
                h2->numSamples = 5;
                h2->criterion = 0.25;
                if (!v2agg.AggregateGradients(vg, h2, true) || h2->numSamples != 5 || h2->criterion != 0.25)
                    return 12;
                v = download(*view);
                if (memcmp(v.data(), in.data(), in.size() * 4) != 0)
                    return 13;
                h2->Clear(); // a worker without samples: zero gradients, "nothing processed"
                if (v2agg.AggregateGradients(vg, h2, false))
                    return 14;
                v = download(*view);
                for (float x : v)
                    if (x != 0.0f)
                        return 15;
                DistGradHeader::Destroy(h2);
                bool threwAsync = false;
                try { V2AllReduceDistGradAggregator<float> bad(comm, true, 0, 0); } catch (const std::logic_error&) { threwAsync = true; }
                if (!threwAsync)
                    return 16;
            }
            // QuantizedDataParallelDistributedLearner: warm-start threshold, aggregated sample count, empty minibatch, checkpoint
            {
                struct CountingLearner : ::CNTK::Learner
                {
                    int calls = 0;
                    size_t lastCount = 0;
                    bool Update(std::vector<::CNTK::NDArrayViewPtr>&, size_t n, bool) override
                    {
                        ++calls;
                        lastCount = n;
                        return true;
                    }
                };
                auto learner = std::make_shared<CountingLearner>();
                auto dl = ::CNTK::CreateQuantizedDataParallelDistributedLearner(comm, learner, /*distributeAfterSamples=*/10);
                cudaMemcpy(view->Data(), in.data(), in.size() * 4, cudaMemcpyHostToDevice);
                ::CNTK::MinibatchInfo info;
                for (int step = 0; step < 3; ++step) // steps 0 and 1 run before the threshold, step 2 after it
                {
                    info.numberOfSamples = 6;
                    info.trainingLossValue = 2.0;
                    info.evalCriterionValue = 0.5;
                    if (!dl->Update(vals, info) || info.numberOfSamples != 6 || learner->lastCount != 6)
                        return 17;
                }
                if (learner->calls != 3 || dl->TotalNumberOfSamplesSeen() != 18)
                    return 18;
                v = download(*view);
                if (memcmp(v.data(), in.data(), in.size() * 4) != 0) // one worker: gradients untouched
                    return 19;
                info = ::CNTK::MinibatchInfo(); // empty minibatch: zero gradients, no local update
                if (dl->Update(vals, info) || learner->calls != 3)
                    return 20;
                v = download(*view);
                for (float x : v)
                    if (x != 0.0f)
                        return 21;
                if (dl->CreateCheckpoint() != 18)
                    return 22;
                bool threwAsync = false;
                try { ::CNTK::CreateQuantizedDataParallelDistributedLearner(comm, learner, 0, true); } catch (const std::logic_error&) { threwAsync = true; }
                if (!threwAsync)
                    return 23;
            }
        }
        else if (mode == "aggregator_async")
        {
            // useAsyncAggregation = true (AllReduceDistGradAggregator.h:156-229): every call hands back the aggregate of the
            // PREVIOUS call's gradients (zeros after the reset) and launches the aggregation of the ones it received
            auto mpi = std::make_shared<MPIWrapper>(std::string(), 0, 1, 0);
            AllReduceDistGradAggregator<float> agg(mpi, bits, zeroThr != 0, true, true, 0, 0);
            Matrix<float> g0(M, N, 0), g1(M, 1, 0);
            std::vector<Matrix<float>*> grads{&g0, &g1};
            DistGradHeader* hdr = DistGradHeader::Create(1);
            for (int it = 0; it <= iters; ++it)
            {
                hdr->Clear();
                if (it < iters)
                {
                    if (fread(in.data(), 4, in.size(), fi) != in.size())
                        return 4;
                    cudaMemcpy(g0.Data(), in.data(), in.size() * 4, cudaMemcpyHostToDevice);
                    cudaMemcpy(g1.Data(), in.data(), M * 4, cudaMemcpyHostToDevice);
                    hdr->numSamples = 7;
                    hdr->criterion = 1.5;
                }
                const bool any = agg.AggregateGradients(grads, hdr, it == 0);
                if (!any)
                    return 7;
                // the header that comes back is the previous call's, aggregated (cleared after the reset)
                if (it == 0 ? (hdr->numSamples != 0) : (hdr->numSamples != 7 || hdr->criterion != 1.5))
                    return 8;
                auto a = download(g0), b = download(g1);
                fwrite(a.data(), 4, a.size(), fo);
                fwrite(b.data(), 4, b.size(), fo);
            }
            // resetting the state while an aggregation is pending is a logic error
            bool threw = false;
            try { agg.AggregateGradients(grads, hdr, true); } catch (const std::logic_error&) { threw = true; }
            if (!threw)
                return 11;
            DistGradHeader::Destroy(hdr);
        }
        else
            return 2;
    }
    catch (const std::exception& e)
    {
        fprintf(stderr, "exception: %s\n", e.what());
        return 10;
    }
    fclose(fi);
    fclose(fo);
    printf("compat ok\n");
    return 0;
}
