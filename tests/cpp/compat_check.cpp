// compat_check.cpp -- drives the C++ mirror of the reference interfaces the way the reference's own callers do and dumps
// the results for tests/test_gpu_compat.py to compare with the CPU oracle.
//   mode "quantizer": the loop of TestRunQuantization (Tests/UnitTests/MathTests/MatrixQuantizerTests.cpp:268-316):
//       MatrixQuantizerImpl::Create, QuantizeAsync(in, residue, CPU QuantizedMatrix, residue), UnquantizeAsync(add = it > 0)
//   mode "quantizer_f64": the same loop with MatrixQuantizerImpl<double> (64-bit packed words)
//   mode "aggregator": AllReduceDistGradAggregator::AggregateGradients on one rank (SGD.cpp:1376), two calls
//   mode "aggregator_async": the same with useAsyncAggregation = true (one-step-stale results, AllReduceDistGradAggregator.h:156-229)
//   mode "schedule": SGD's per-epoch bookkeeping (gradientBits as a per-epoch array re-creating the aggregator, warm start by
//       parallelizationStartEpoch: SGD.cpp:427-432, 553-559, 2336-2359) on one rank
//   mode "multi": one of K processes (one per GPU), tied together by a unique id passed through a file: the V1 aggregator,
//       the V2 aggregator (synchronous and buffered asynchronous), the V2 learner and the unquantized aggregator run a
//       real K-rank exchange, DistGradHeader included; the V2 learner also runs over a momentum-SGD learner with and without
//       the update fused into the exchange
// usage: compat_check <mode> <in.bin> <out.bin> M N bits zeroThr iters [rank K idfile]
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <thread>
#include <vector>

#include "../../cntk_b200/csrc/cntk_compat/AllReduceDistGradAggregator.h"
#include "../../cntk_b200/csrc/cntk_compat/DataParallelSGD.h"
#include "../../cntk_b200/csrc/cntk_compat/SimpleDistGradAggregator.h"
#include "../../cntk_b200/csrc/cntk_compat/QuantizedDataParallelDistributedLearner.h"
#include "../../cntk_b200/csrc/cntk_compat/MomentumSGDLearner.h"
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
        else if (mode == "quantizer_f64")
        {
            // the same loop for ElemType = double (CPUMatrix1BitQuantizeDouble / GPUMatrix1BitQuantizeDouble); the input file holds doubles
            std::unique_ptr<MatrixQuantizerImpl<double>> q(MatrixQuantizerImpl<double>::Create(0, false));
            Matrix<double> inM(M, N, 0), residue(M, N, 0), out(M, N, 0);
            std::vector<double> ind(M * N), hr(M * N), ho(M * N);
            for (int it = 0; it < iters; ++it)
            {
                if (fread(ind.data(), 8, ind.size(), fi) != ind.size())
                    return 4;
                cudaMemcpy(inM.Data(), ind.data(), ind.size() * 8, cudaMemcpyHostToDevice);
                QuantizedMatrix<double> packed(M, N, bits, CPUDEVICE);
                q->QuantizeAsync(inM, residue, packed, residue, zeroThr != 0);
                q->WaitQuantizeAsyncDone();
                q->UnquantizeAsync(packed, out, it > 0);
                q->WaitUnquantizeAsyncDone();
                fwrite(packed.Buffer(), 1, packed.GetSize(), fo);
                cudaMemcpy(hr.data(), residue.Data(), hr.size() * 8, cudaMemcpyDeviceToHost);
                cudaMemcpy(ho.data(), out.Data(), ho.size() * 8, cudaMemcpyDeviceToHost);
                fwrite(hr.data(), 8, hr.size(), fo);
                fwrite(ho.data(), 8, ho.size(), fo);
            }
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
            std::vector<::CNTK::NDArrayViewPtr> noResidues, noStripeResidues;
            comm->QuantizedAggregateInPlace(vals, noResidues, noStripeResidues, comm->Workers());
            if (!noResidues.empty() || !noStripeResidues.empty()) // one worker: the residual vectors come back as they went in
                return 24;
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
        else if (mode == "schedule")
        {
            // SGD's per-epoch aggregator bookkeeping on one rank: gradientBits = 1:1:4:32 (the last value repeats),
            // parallelizationStartEpoch = 2; five epochs of two minibatches.  Epoch 0 must leave the gradients alone, epochs 1
            // and 2 are quantize -> unquantize round trips at 1 and 4 bits from zero residuals, epochs 3 and 4 the
            // unquantized sum over one rank.
            auto mpi = std::make_shared<MPIWrapper>(std::string(), 0, 1, 0);
            DataParallelSGDConfig cfg;
            cfg.gradientBits = {1, 1, 4, 32};
            cfg.parallelizationStartEpoch = 2;
            cfg.useZeroThresholdFor1BitQuantization = zeroThr != 0;
            DataParallelSGD<float> sgd(mpi, cfg, 1, 0);
            Matrix<float> g0(M, N, 0), g1(M, 1, 0);
            std::vector<Matrix<float>*> grads{&g0, &g1};
            sgd.BeginTraining(0);
            for (int epoch = 0; epoch < 5; ++epoch)
            {
                sgd.BeginEpoch((size_t) epoch);
                if (sgd.CurrentNumGradientBits() != (epoch < 2 ? 1 : epoch == 2 ? 4 : 32))
                    return 50;
                for (int mb = 0; mb < 2; ++mb)
                {
                    if (fread(in.data(), 4, in.size(), fi) != in.size())
                        return 4;
                    cudaMemcpy(g0.Data(), in.data(), in.size() * 4, cudaMemcpyHostToDevice);
                    cudaMemcpy(g1.Data(), in.data(), M * 4, cudaMemcpyHostToDevice);
                    sgd.Header().Clear();
                    sgd.Header().numSamples = 9;
                    sgd.Header().criterion = 0.75;
                    if (!sgd.AggregateMinibatch(grads, mb == 0) || sgd.Header().numSamples != 9 || sgd.Header().criterion != 0.75)
                        return 51;
                    auto a = download(g0), b = download(g1);
                    fwrite(a.data(), 4, a.size(), fo);
                    fwrite(b.data(), 4, b.size(), fo);
                }
            }
            if (sgd.TimesInitialized() != 3) // 1 bit at the start, 4 bits before epoch 2, 32 bits before epoch 3
                return 52;
            // the checks of the configuration (SGD.cpp:3318-3319, 3338-3342)
            int refused = 0;
            for (int bad = 0; bad < 3; ++bad)
            {
                DataParallelSGDConfig c;
                if (bad == 0)
                    c.gradientBits = {0};
                else if (bad == 1)
                    c.gradientBits = {1, 33};
                else
                    c.parallelizationStartEpoch = 0;
                try { DataParallelSGD<float> x(mpi, c, 1, 0); } catch (const std::invalid_argument&) { ++refused; }
            }
            if (refused != 3)
                return 53;
            // useV2Aggregator on one worker: the V2 communicator returns at once, gradients stay as they are
            DataParallelSGDConfig v2 = cfg;
            v2.useV2Aggregator = true;
            v2.parallelizationStartEpoch = 1;
            DataParallelSGD<float> sgd2(mpi, v2, 1, 0);
            sgd2.BeginTraining(0);
            sgd2.BeginEpoch(0);
            cudaMemcpy(g0.Data(), in.data(), in.size() * 4, cudaMemcpyHostToDevice);
            sgd2.Header().Clear();
            sgd2.Header().numSamples = 3;
            if (!sgd2.AggregateMinibatch(grads, true))
                return 54;
            auto v = download(g0);
            if (memcmp(v.data(), in.data(), in.size() * 4) != 0)
                return 55;
        }
        else if (mode == "multi")
        {
            if (argc < 12)
                return 2;
            const int rank = atoi(argv[9]), K = atoi(argv[10]);
            const std::string idfile = argv[11];
            std::string id;
            if (rank == 0)
            {
                id = MPIWrapper::NewUniqueId();
                std::ofstream(idfile + ".tmp", std::ios::binary).write(id.data(), (std::streamsize) id.size());
                if (rename((idfile + ".tmp").c_str(), idfile.c_str()) != 0)
                    return 30;
            }
            else
            {
                for (int tries = 0; tries < 600 && id.empty(); ++tries)
                {
                    std::ifstream f(idfile, std::ios::binary);
                    if (f)
                        id.assign((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
                    else
                        std::this_thread::sleep_for(std::chrono::milliseconds(100));
                }
                if (id.size() != QAGG_UNIQUE_ID_BYTES)
                    return 31;
            }
            int ndev = 0;
            cudaGetDeviceCount(&ndev);
            const int dev = rank % (ndev > 0 ? ndev : 1);
            auto mpi = std::make_shared<MPIWrapper>(id, rank, K, dev);
            // inputs: per iteration, per rank: g0 (M x N) then g1 (M x 1); every process reads the whole file
            std::vector<std::vector<float>> mine0(iters), mine1(iters);
            for (int it = 0; it < iters; ++it)
                for (int r = 0; r < K; ++r)
                {
                    std::vector<float> a(M * N), b(M);
                    if (fread(a.data(), 4, a.size(), fi) != a.size() || fread(b.data(), 4, b.size(), fi) != b.size())
                        return 4;
                    if (r == rank)
                    {
                        mine0[it] = a;
                        mine1[it] = b;
                    }
                }
            Matrix<float> g0(M, N, dev), g1(M, 1, dev);
            std::vector<Matrix<float>*> grads{&g0, &g1};
            auto load = [&](int it) {
                cudaMemcpy(g0.Data(), mine0[it].data(), M * N * 4, cudaMemcpyHostToDevice);
                cudaMemcpy(g1.Data(), mine1[it].data(), M * 4, cudaMemcpyHostToDevice);
            };
            auto dump = [&]() {
                auto a = download(g0), b = download(g1);
                fwrite(a.data(), 4, a.size(), fo);
                fwrite(b.data(), 4, b.size(), fo);
            };
            DistGradHeader* hdr = DistGradHeader::Create(1);
            auto fillHeader = [&](DistGradHeader* h) {
                h->Clear();
                h->numSamples = 7 + rank;
                h->numSamplesWithLabel = 5 + rank;
                h->criterion = 1.5 * (rank + 1);
                h->evalErrors[0] = {0.25 * rank, (size_t) (3 + rank)};
            };
            auto headerIsSum = [&](const DistGradHeader* h) {
                size_t ns = 0, nl = 0, ne = 0;
                double cr = 0, ee = 0;
                for (int r = 0; r < K; ++r)
                {
                    ns += 7 + r;
                    nl += 5 + r;
                    cr += 1.5 * (r + 1);
                    ee += 0.25 * r;
                    ne += 3 + r;
                }
                return h->numSamples == ns && h->numSamplesWithLabel == nl && h->criterion == cr && h->evalErrors[0].first == ee &&
                       h->evalErrors[0].second == ne;
            };
            // A. V1 aggregator, synchronous
            {
                AllReduceDistGradAggregator<float> agg(mpi, bits, zeroThr != 0, true, false, 0, 0);
                for (int it = 0; it < iters; ++it)
                {
                    load(it);
                    fillHeader(hdr);
                    if (!agg.AggregateGradients(grads, hdr, it == 0) || !headerIsSum(hdr))
                        return 32;
                    dump();
                }
                agg.WaitAll();
            }
            // B. V2 aggregator over the V2 communicator, synchronous; its residual views, made readable, are dumped at the end
            auto comm = ::CNTK::QuantizedMPICommunicator(mpi, zeroThr != 0, true, (size_t) bits);
            {
                V2AllReduceDistGradAggregator<float> agg(comm, false, 0, 0);
                for (int it = 0; it < iters; ++it)
                {
                    load(it);
                    fillHeader(hdr);
                    if (!agg.AggregateGradients(grads, hdr, it == 0) || !headerIsSum(hdr))
                        return 33;
                    dump();
                }
                if (agg.Residuals().size() != 2 || !agg.Residuals()[0] || agg.StripeResiduals().size() != 2)
                    return 34;
                static_cast<::CNTK::QuantizedMPICommunicatorImpl*>(comm.get())->MaterializeResiduals();
                auto r0 = download(*agg.Residuals()[0]);
                fwrite(r0.data(), 4, r0.size(), fo);
                // resetState zeroes the residuals: the next step equals a first step
                load(0);
                fillHeader(hdr);
                if (!agg.AggregateGradients(grads, hdr, true))
                    return 35;
                dump();
            }
            // C. the same, buffered asynchronous: results are one call stale, zeros after the reset
            {
                auto comm2 = ::CNTK::QuantizedMPICommunicator(mpi, zeroThr != 0, true, (size_t) bits);
                V2AllReduceDistGradAggregator<float> agg(comm2, true, 0, 0);
                for (int it = 0; it <= iters; ++it)
                {
                    hdr->Clear();
                    if (it < iters)
                    {
                        load(it);
                        fillHeader(hdr);
                    }
                    else
                    {
                        g0.SetValue(0);
                        g1.SetValue(0);
                        hdr->numSamples = 1; // keeps the pipeline going for the drain call
                    }
                    if (!agg.AggregateGradients(grads, hdr, it == 0))
                        return 36;
                    if (it == 0 ? (hdr->numSamples != 0) : !headerIsSum(hdr))
                        return 37;
                    dump();
                }
            }
            // D. the V2 learner: aggregation from the first sample on, checkpoint zeroes the residuals
            {
                struct NullLearner : ::CNTK::Learner
                {
                    bool Update(std::vector<::CNTK::NDArrayViewPtr>&, size_t, bool) override { return true; }
                };
                // the factory with the reference's own signature finds the registered process-wide MPIWrapper
                bool threwNoInstance = false;
                try { ::CNTK::QuantizedMPICommunicator(zeroThr != 0, true, (size_t) bits); } catch (const std::runtime_error&) { threwNoInstance = true; }
                if (!threwNoInstance)
                    return 45;
                MPIWrapper::SetInstance(mpi);
                auto comm3 = ::CNTK::QuantizedMPICommunicator(zeroThr != 0, true, (size_t) bits);
                MPIWrapper::DeleteInstance();
                auto dl = ::CNTK::CreateQuantizedDataParallelDistributedLearner(comm3, std::make_shared<NullLearner>(), 0);
                std::vector<::CNTK::NDArrayViewPtr> vals{std::make_shared<Matrix<float>>(M, N, g0.Data(), dev), std::make_shared<Matrix<float>>(M, 1, g1.Data(), dev)};
                for (int it = 0; it < iters; ++it)
                {
                    load(it);
                    ::CNTK::MinibatchInfo info;
                    info.numberOfSamples = 4 + rank;
                    info.trainingLossValue = 2.0 + rank;
                    info.evalCriterionValue = 0.5;
                    if (!dl->Update(vals, info))
                        return 38;
                    size_t ns = 0;
                    double tl = 0;
                    for (int r = 0; r < K; ++r)
                    {
                        ns += 4 + r;
                        tl += 2.0 + r;
                    }
                    if (info.numberOfSamples != ns || info.trainingLossValue != tl || info.evalCriterionValue != 0.5 * K)
                        return 39;
                    dump();
                    if (it == 0)
                        dl->CreateCheckpoint(); // residuals zeroed: the next step starts from scratch again
                }
            }
            // E. the unquantized aggregator (gradientBits = 32), all-reduce path
            {
                SimpleDistGradAggregator<float> agg(mpi, false, dev, 0);
                load(0);
                fillHeader(hdr);
                if (!agg.AggregateGradients(grads, hdr, false) || !headerIsSum(hdr))
                    return 40;
                dump();
            }
            // F. the V2 learner over a momentum-SGD learner, twice: the reference's order (aggregate, then Update) and with the
            //    update fused into the exchange's last kernel.  Same parameters and smoothed gradients bit for bit; the fused
            //    run leaves the gradient views alone.  Parameters start as 1 + 1000 * (this rank's first gradients).
            {
                const float lr = 0.05f, momentum = 0.9f;
                std::vector<float> p0(M * N), p1(M);
                for (size_t i = 0; i < p0.size(); ++i)
                    p0[i] = 1.0f + 1000.0f * mine0[0][i];
                for (size_t i = 0; i < p1.size(); ++i)
                    p1[i] = 1.0f + 1000.0f * mine1[0][i];
                std::vector<::CNTK::NDArrayViewPtr> params[2];
                std::shared_ptr<::CNTK::MomentumSGDLearner> sgd[2];
                ::CNTK::DistributedLearnerPtr dl[2];
                for (int f = 0; f < 2; ++f)
                {
                    params[f] = {std::make_shared<Matrix<float>>(M, N, dev), std::make_shared<Matrix<float>>(M, 1, dev)};
                    cudaMemcpy(params[f][0]->Data(), p0.data(), p0.size() * 4, cudaMemcpyHostToDevice);
                    cudaMemcpy(params[f][1]->Data(), p1.data(), p1.size() * 4, cudaMemcpyHostToDevice);
                    sgd[f] = std::make_shared<::CNTK::MomentumSGDLearner>(params[f], lr, momentum, true);
                    dl[f] = ::CNTK::CreateQuantizedDataParallelDistributedLearner(::CNTK::QuantizedMPICommunicator(mpi, zeroThr != 0, true, (size_t) bits),
                                                                                  sgd[f], 0);
                    dl[f]->SetConsumerFusion(f == 1);
                }
                std::vector<::CNTK::NDArrayViewPtr> vals{std::make_shared<Matrix<float>>(M, N, g0.Data(), dev), std::make_shared<Matrix<float>>(M, 1, g1.Data(), dev)};
                for (int it = 0; it < iters; ++it)
                    for (int f = 0; f < 2; ++f)
                    {
                        load(it);
                        ::CNTK::MinibatchInfo info;
                        info.numberOfSamples = 4 + rank;
                        if (!dl[f]->Update(vals, info))
                            return 41;
                        if (f == 1 && (download(g0) != mine0[it] || download(g1) != mine1[it]))
                            return 42; // the fused step must not touch the gradient views
                    }
                for (int t = 0; t < 2; ++t)
                {
                    const auto a = download(*params[0][t]), b = download(*params[1][t]);
                    const auto sa = download(*sgd[0]->SmoothedGradients()[t]), sb = download(*sgd[1]->SmoothedGradients()[t]);
                    if (memcmp(a.data(), b.data(), a.size() * 4) != 0 || memcmp(sa.data(), sb.data(), sa.size() * 4) != 0)
                        return 43;
                    fwrite(b.data(), 4, b.size(), fo);
                    fwrite(sb.data(), 4, sb.size(), fo);
                }
                if (sgd[1]->TotalNumberOfMinibatchesSeen() != (size_t) iters || sgd[0]->TotalNumberOfSamplesSeen() != sgd[1]->TotalNumberOfSamplesSeen())
                    return 44;
            }
            // G. the V1 aggregator for double gradients (the float inputs widened), synchronous
            {
                AllReduceDistGradAggregator<double> agg(mpi, bits, zeroThr != 0, true, false, 0, 0);
                Matrix<double> d0(M, N, dev), d1(M, 1, dev);
                std::vector<Matrix<double>*> dgrads{&d0, &d1};
                for (int it = 0; it < iters; ++it)
                {
                    std::vector<double> w0(mine0[it].begin(), mine0[it].end()), w1(mine1[it].begin(), mine1[it].end());
                    cudaMemcpy(d0.Data(), w0.data(), w0.size() * 8, cudaMemcpyHostToDevice);
                    cudaMemcpy(d1.Data(), w1.data(), w1.size() * 8, cudaMemcpyHostToDevice);
                    fillHeader(hdr);
                    if (!agg.AggregateGradients(dgrads, hdr, it == 0) || !headerIsSum(hdr))
                        return 46;
                    cudaMemcpy(w0.data(), d0.Data(), w0.size() * 8, cudaMemcpyDeviceToHost);
                    cudaMemcpy(w1.data(), d1.Data(), w1.size() * 8, cudaMemcpyDeviceToHost);
                    fwrite(w0.data(), 8, w0.size(), fo);
                    fwrite(w1.data(), 8, w1.size(), fo);
                }
            }
            mpi->WaitAll();
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
