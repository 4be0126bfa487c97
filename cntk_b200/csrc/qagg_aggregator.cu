// qagg_aggregator.cu -- communicator and striped aggregator behind include/qagg.h.
//
// One aggregation step on rank r of K (AllReduceDistGradAggregator.h:237-566 restated for device buffers):
//   K1  one launch quantizes every gradient against its residual and writes each packed column straight into
//       the region of the send buffer that belongs to the column's owner (own columns go to the receive slot);
//   X1  grouped ncclSend/ncclRecv: region p -> rank p, one message per peer covering all tensors;
//   K2  one launch per step: for every owned stripe, unpack the K stripes, add them in rank order (own first),
//       add the stripe residual, requantize into this rank's slot of the gather buffer;
//   X2  ncclAllGather of the (equal-sized, padded) slots;
//   K3  one launch unpacks every tensor from the gather buffer into the gradient.
// All buffers live for the lifetime of the aggregator; nothing is allocated per step.
#include "../../include/qagg.h"
#include "qagg_comm.h"
#include "qagg_internal.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <vector>

using namespace qagg;

namespace {

inline int64_t align_up(int64_t v, int64_t a)
{
    return (v + a - 1) / a * a;
}

int check_nccl(ncclResult_t r, const char* what)
{
    if (r == ncclSuccess)
        return QAGG_OK;
    return fail(QAGG_ENCCL, std::string(what) + ": " + ncclGetErrorString(r));
}

struct DevBuf
{
    void* p = nullptr;
    size_t bytes = 0;
    ~DevBuf()
    {
        if (p)
            cudaFree(p);
    }
    int alloc(size_t bytes, bool zero)
    {
        if (bytes == 0)
            bytes = 16;
        this->bytes = bytes;
        int rc = check_cuda(cudaMalloc(&p, bytes), "cudaMalloc");
        if (rc)
            return rc;
        if (zero)
            return check_cuda(cudaMemset(p, 0, bytes), "cudaMemset");
        return QAGG_OK;
    }
};

} // namespace

// Wire layout of one rank's view of the exchange; pure host arithmetic (no device needed).
//   region p  = the packed stripes owned by rank p, tensor after tensor (each block 16-byte aligned): the message
//               this rank sends to p in the scatter, and what rank p contributes to the all-gather;
//   gather slot = the largest region, padded, so that the all-gather moves equal counts.
struct qagg_plan
{
    int rank = 0, K = 1, T = 0, bits = 1;
    std::vector<int64_t> M, N, colBytes;
    std::vector<int64_t> parentN, col0; // tensor i is columns [col0, col0 + N) of a matrix of parentN columns (whole: 0, N)
    std::vector<std::vector<int64_t>> sStart, sN, tOff; // [p][i]; sStart is relative to the tensor's first column
    std::vector<int64_t> regionBytes;
    int64_t gatherSlot = 0;

    int build(int rank_, int K_, int T_, const int64_t* M_, const int64_t* N_, int bits_, const int64_t* parentN_ = nullptr,
              const int64_t* col0_ = nullptr)
    {
        if (K_ < 1 || K_ > QAGG_MAXK || rank_ < 0 || rank_ >= K_ || T_ < 0 || (T_ > 0 && (!M_ || !N_)))
            return fail(QAGG_EINVAL, "plan: bad arguments");
        if (!bits_ok(bits_))
            return fail(QAGG_EINVAL, "bits must be a power of two in 1..32");
        rank = rank_;
        K = K_;
        T = T_;
        bits = bits_;
        M.assign(M_, M_ + T);
        N.assign(N_, N_ + T);
        parentN = N;
        col0.assign(T, 0);
        if (parentN_ && col0_)
        {
            parentN.assign(parentN_, parentN_ + T);
            col0.assign(col0_, col0_ + T);
        }
        colBytes.resize(T);
        for (int i = 0; i < T; ++i)
        {
            if (M[i] < 0 || N[i] < 0 || M[i] > 0x3fffffffLL || N[i] > 0x7fffffffLL || col0[i] < 0 || col0[i] + N[i] > parentN[i] ||
                parentN[i] > 0x7fffffffLL)
                return fail(QAGG_EINVAL, "plan: bad tensor shape");
            colBytes[i] = 8 + 4 * ((M[i] * bits + 31) / 32);
        }
        sStart.assign(K, std::vector<int64_t>(T));
        sN.assign(K, std::vector<int64_t>(T));
        tOff.assign(K, std::vector<int64_t>(T));
        regionBytes.assign(K, 0);
        gatherSlot = 0;
        for (int p = 0; p < K; ++p)
        {
            int64_t off = 0;
            for (int i = 0; i < T; ++i)
            {
                // the owner's stripe of the whole matrix, cut to this tensor's columns
                int64_t ps = 0, pn = 0;
                qagg_stripe(parentN[i], p, K, &ps, &pn);
                const int64_t lo = std::max(ps, col0[i]), hi = std::min(ps + pn, col0[i] + N[i]);
                sStart[p][i] = (hi > lo ? lo : col0[i]) - col0[i];
                sN[p][i] = hi > lo ? hi - lo : 0;
                tOff[p][i] = off;
                off += align_up(sN[p][i] * colBytes[i], 16);
            }
            regionBytes[p] = off;
            gatherSlot = std::max(gatherSlot, align_up(off, 256));
        }
        return QAGG_OK;
    }
};

struct qagg_aggregator
{
    qagg_comm* comm = nullptr;
    int T = 0;
    int bits = 1;
    int flags = 0;
    int mode = 0;
    std::vector<int64_t> M, N, colBytes, parentN, col0;
    // stripe geometry: [p][i]
    std::vector<std::vector<int64_t>> sStart, sN, tOff;
    std::vector<int64_t> regionBytes; // packed bytes of rank p's stripes over all tensors (16-byte aligned blocks)
    std::vector<int64_t> sendOff;     // offset of region p in the send buffer
    int64_t slotBytes = 0;            // regionBytes[rank], padded: size of one receive slot
    int64_t gatherSlot = 0;           // max region, padded: size of one gather slot
    // "window": [flags][receive slots][gather slots] in ONE allocation, so that a single IPC handle exposes to the
    // peers everything they write into this rank's memory
    DevBuf sendbuf, window, resAll, sresAll, tables, hostStage;
    // scatter flags [0, K), gather flags [64, 64 + K), status word at [127]; then one header slot (QAGG_HEADER_MAX doubles) per rank
    static const int64_t kHeaderOff = 512;
    static const int64_t kFlagBytes = kHeaderOff + (int64_t) QAGG_MAXK * QAGG_HEADER_MAX * 8;
    // header exchange: pinned, device-mapped host buffer: [0, MAX) this rank's header of the step, [MAX, 2 MAX) the sum
    double* hdrHost = nullptr;
    double* hdrDev = nullptr; // NCCL path only: device staging
    int hdrN = 0;             // doubles in the step's header (0: the step carries none)
    unsigned char* recvbuf = nullptr;
    unsigned char* gatherbuf = nullptr;
    // peer-memory exchange (off until qagg_agg_enable_peer): packed columns are stored straight into the peers' windows
    bool peer = false;
    unsigned char* peerWin[QAGG_MAXK] = {};
    bool peerOpened[QAGG_MAXK] = {};
    unsigned stepNo = 0;
    long long waitPolls = 20000000; // bounded device-side waits (about two seconds of polling)
    // peer mode, all-gather half: true = the requantize kernel writes locally and a small copy kernel pushes the finished
    // region to the peers; false = the requantize kernel itself stores every packed word K times
    bool pushGather = false;
    std::vector<float*> res, sres;
    bool externalRes = false; // the residual buffers belong to the caller (qagg_agg_bind_residuals)
    // 1 bit with threshold 0: the quantize kernel (and optionally the owner's reduce-requantize kernel) is the streaming
    // kernel, which keeps its residual set in deferred form: the buffer above holds the quantized values v, and lv (slv)
    // each column's two reconstruction values (see qagg_internal.h)
    bool deferred = false;      // quantize kernel: residuals `res`
    bool deferredOwner = false; // owner kernels (form + walk): stripe residuals `sres`
    DevBuf tmaps;                        // tensor maps of the streaming quantize descriptors (QAGG_STREAM_MAP_BYTES each)
    std::vector<unsigned char> hostMaps; // their host mirror
    DevBuf ownMaps, ownStats;            // owner kernels: one tensor map per owned stripe; two counters per owned column
    long long k2Units = 0;               // work units of the owner's form kernel
    // owner kernels, tall matrices apart: their table entries, form units and walk items come first (see launch_owner)
    OwnerSplit k2Split = {};
    bool k2SplitOn = false;
    // Quantize kernel, very tall matrices apart (1 bit, threshold 0, whole tensors only): a column of tens of thousands of
    // rows is one long chain of dependent adds, which the streaming kernel walks a chunk at a time with a fixed cost per
    // chunk.  Such matrices go through the owner's form + walk kernel pair instead (one table entry per owner's stripe, the
    // raw gradient as the only source), the walk beside the streaming kernel of the other matrices.
    std::vector<QTensor> hK1t;
    std::vector<int> k1tTensor;          // tensor index of each entry
    std::vector<long long> k1tCol;       // first column (of the tensor) of each entry
    std::vector<QItem> iK1t;
    long long k1tUnits = 0;
    QTensor* dK1t = nullptr;
    QItem* dI1t = nullptr;
    DevBuf k1tMaps, k1tStats, k1tCounters;
    cudaStream_t k1Side = nullptr;
    cudaEvent_t k1Fork = nullptr, k1Join = nullptr;
    // the stream the last step was enqueued on: calls that rewrite what that step reads (tables, tensor maps, residual
    // state) from another stream wait for it first
    cudaStream_t lastStream = nullptr;
    bool stepped = false;
    DevBuf lvAll, slvAll;
    std::vector<float*> lv, slv;
    // device tables and their host mirrors
    std::vector<QTensor> hK1, hK2, hK3;
    std::vector<QItem> iK1, iK2;
    long long k3Units = 0; // work units of the unquantize launch
    int k3SmemWords = 0;   // shared-memory words per warp the unquantize launch needs
    QTensor *dK1 = nullptr, *dK2 = nullptr, *dK3 = nullptr;
    QItem *dI1 = nullptr, *dI2 = nullptr;
    // consumer fusion: a copy of the unquantize table whose destinations are the caller's parameter and smoothed-gradient
    // matrices, and the rule the unquantize launch applies when `updating`
    DevBuf updTable;
    bool updBound = false, updating = false;
    UpdateRule updRule = {};
    DevBuf queue; // three pairs of work-queue counters (one pair per kernel), zero when no kernel is running
    std::vector<int> k2Tensor; // tensor index of each K2 table entry
    // The device tables (and tensor maps) hold the gradient pointers.  Two sets are kept, each bound to one array of
    // gradient pointers, so that a caller that alternates between two gradient buffer sets (double-buffered aggregation)
    // pays for the table upload only twice.
    struct Binding
    {
        std::vector<float*> grads;
        QTensor *dK1 = nullptr, *dK2 = nullptr, *dK3 = nullptr, *dK1t = nullptr;
        QItem *dI1 = nullptr, *dI2 = nullptr, *dI1t = nullptr;
    };
    Binding bindings[2];
    int curBinding = 0;
    size_t tableBytes = 0; // size of one set of tables
    LaunchCfg cfg;
    int64_t totalValues = 0;
    bool identity = false;
    // optional per-phase timing
    static const int kProfSlots = 64;
    bool profiling = false;
    cudaEvent_t ev[kProfSlots][6] = {};
    long long profSteps = 0; // profiled steps recorded since profiling was switched on or last read
    // host-path staging
    DevBuf devGrads;
    std::vector<float*> devGradPtr;

    ~qagg_aggregator()
    {
        if (hdrHost)
            cudaFreeHost(hdrHost);
        if (hdrDev)
            cudaFree(hdrDev);
        for (int p = 0; p < QAGG_MAXK; ++p)
            if (peerOpened[p])
                cudaIpcCloseMemHandle(peerWin[p]);
        for (auto& slot : ev)
            for (auto& e : slot)
                if (e)
                    cudaEventDestroy(e);
        if (k1Fork)
            cudaEventDestroy(k1Fork);
        if (k1Join)
            cudaEventDestroy(k1Join);
        if (k1Side)
            cudaStreamDestroy(k1Side);
        if (k2Split.fork)
            cudaEventDestroy(k2Split.fork);
        if (k2Split.join)
            cudaEventDestroy(k2Split.join);
        if (k2Split.side)
            cudaStreamDestroy(k2Split.side);
    }
    int mark(int i, cudaStream_t st)
    {
        if (!profiling)
            return QAGG_OK;
        return check_cuda(cudaEventRecord(ev[profSteps % kProfSlots][i], st), "cudaEventRecord");
    }
    unsigned char* send_region(int p) const { return static_cast<unsigned char*>(sendbuf.p) + sendOff[p]; }
    unsigned char* recv_slot(int src) const { return recvbuf + (int64_t) src * slotBytes; }
    unsigned char* gather_slot(int p) const { return gatherbuf + (int64_t) p * gatherSlot; }
    unsigned* flag_words() const { return static_cast<unsigned*>(window.p); }
    unsigned* status_word() const { return static_cast<unsigned*>(window.p) + 127; }
    // the same places inside peer p's window (its receive slots have ITS region size)
    int64_t peer_slot_bytes(int p) const { return align_up(regionBytes[p], 256); }
    unsigned char* peer_recv_slot(int p, int src) const { return peerWin[p] + kFlagBytes + (int64_t) src * peer_slot_bytes(p); }
    unsigned char* peer_gather_slot(int p, int slot) const
    {
        return peerWin[p] + kFlagBytes + peer_slot_bytes(p) * comm->K + (int64_t) slot * gatherSlot;
    }
    unsigned* peer_flags(int p) const { return reinterpret_cast<unsigned*>(peerWin[p]); }
    double* header_slot(unsigned char* win, int src) const { return reinterpret_cast<double*>(win + kHeaderOff) + (int64_t) src * QAGG_HEADER_MAX; }
};

namespace {

void make_items(std::vector<QItem>& items, int tensor, int64_t M, int64_t N, int c)
{
    for (int64_t col0 = 0; col0 < N; col0 += c)
        items.push_back(QItem{tensor, (int) col0, (int) std::min<int64_t>(c, N - col0)});
}

// Columns per work item for each matrix of one launch.  Start from as many as shared memory holds; while the launch
// would not even fill the resident CTA slots once, halve the item of the matrix whose items are the most expensive
// (rows x columns): a tall column's ordered walk is a fixed latency, so fewer columns per item shortens the launch
// when there are CTA slots to spare.
std::vector<int> choose_cols(const std::vector<std::pair<int64_t, int64_t>>& shapes, const LaunchCfg& cfg, int bits = 1, int packedSources = 0)
{
    std::vector<int> c(shapes.size(), 1);
    auto items = [&](size_t i) { return shapes[i].second > 0 ? (shapes[i].second + c[i] - 1) / c[i] : 0; };
    int64_t total = 0;
    for (size_t i = 0; i < shapes.size(); ++i)
    {
        const int colWords = 2 + (int) ((shapes[i].first * bits + 31) / 32);
        c[i] = cols_per_item(shapes[i].first, shapes[i].second, cfg.smemFloats, nullptr, packedSources * colWords);
        total += items(i);
    }
    const int64_t slots = (int64_t) cfg.numSMs * cfg.ctasPerSM;
    while (total < slots)
    {
        int best = -1;
        int64_t bestCost = 0;
        for (size_t i = 0; i < shapes.size(); ++i)
        {
            const int64_t cost = shapes[i].first * c[i];
            if (c[i] > 1 && shapes[i].second > 0 && cost > bestCost)
            {
                bestCost = cost;
                best = (int) i;
            }
        }
        if (best < 0)
            break;
        total -= items(best);
        c[best] = (c[best] + 1) / 2;
        total += items(best);
    }
    return c;
}

int build_tables(qagg_aggregator* a)
{
    const int K = a->comm->K, r = a->comm->rank, T = a->T;
    a->hK1.assign(T, QTensor{});
    a->hK3.assign(T, QTensor{});
    a->k3Units = 0;
    a->k3SmemWords = 0;
    for (int i = 0; i < T; ++i)
    {
        // every entry, empty matrices included, carries the running unit count (the kernel searches this column)
        a->hK3[i].unit0 = a->k3Units;
        a->k3Units += unq_units(a->M[i], a->N[i], a->bits);
        if (a->N[i] > 0)
            a->k3SmemWords = std::max(a->k3SmemWords, unq_smem_words(a->M[i], a->bits));
    }
    a->hK2.clear();
    a->k2Tensor.clear();
    a->iK1.clear();
    a->iK2.clear();
    a->k2Units = 0;
    std::vector<std::pair<int64_t, QItem>> cost1, cost2;
    std::vector<std::pair<int64_t, int64_t>> shapes1, shapes2;
    for (int i = 0; i < T; ++i)
    {
        const bool live = a->M[i] > 0 && a->N[i] > 0;
        shapes1.push_back({a->M[i], live ? a->N[i] : 0});
        shapes2.push_back({a->M[i], (live && K > 1) ? a->sN[r][i] : 0});
    }
    const std::vector<int> c1 = choose_cols(shapes1, a->cfg), c2 = choose_cols(shapes2, a->cfg);
    std::vector<std::pair<long long, long long>> k2Shapes; // streaming kernels: (rows, columns) per entry of the owner table
    for (int i = 0; i < T; ++i)
    {
        const int64_t M = a->M[i], N = a->N[i];
        if (M == 0 || N == 0)
            continue;
        QTensor& q1 = a->hK1[i];
        fill_layout(&q1, M, N, a->bits);
        q1.res_in = a->res[i];
        q1.res_out = a->res[i];
        q1.lv = a->deferred ? a->lv[i] : nullptr;
        q1.K = K;
        q1.per = a->parentN[i] / K;
        q1.rem = a->parentN[i] % K;
        q1.col0 = a->col0[i];
        QTensor& q3 = a->hK3[i];
        const long long unit0 = q3.unit0;
        q3 = q1;
        q3.unit0 = unit0;
        q3.res_in = nullptr;
        q3.res_out = nullptr;
        q3.lv = nullptr;
        for (int p = 0; p < K; ++p)
        {
            if (K == 1)
                q1.pk[p] = a->gather_slot(0) + a->tOff[0][i];
            else if (p == r)
                q1.pk[p] = a->recv_slot(r) + a->tOff[p][i];
            else if (a->peer)
                q1.pk[p] = a->peer_recv_slot(p, r) + a->tOff[p][i]; // straight into the owner's receive slot over NVLink
            else
                q1.pk[p] = a->send_region(p) + a->tOff[p][i];
            q3.pk[p] = a->gather_slot(p) + a->tOff[p][i];
        }
        {
            std::vector<QItem> tmp;
            make_items(tmp, i, M, N, c1[i]);
            for (auto& it : tmp)
                cost1.push_back({M * it.ncols, it});
        }
    }
    // The owner's table.  With the two-kernel owner, matrices much taller than the rest come first: their walk is the longest
    // dependent chain and gets a launch of its own (launch_owner).  "Tall": more than half the rows of the tallest owned matrix.
    std::vector<int> k2Order;
    {
        int64_t tallest = 0;
        for (int i = 0; i < T; ++i)
            if (K > 1 && a->M[i] > 0 && a->N[i] > 0 && a->sN[r][i] > 0)
                tallest = std::max(tallest, a->M[i]);
        for (int pass = 0; pass < 2; ++pass)
            for (int i = 0; i < T; ++i)
            {
                if (!(K > 1 && a->M[i] > 0 && a->N[i] > 0 && a->sN[r][i] > 0))
                    continue;
                const bool tall = a->deferredOwner && 2 * a->M[i] > tallest;
                if (tall == (pass == 0))
                    k2Order.push_back(i);
            }
        a->k2Split.tallUnits = 0;
        a->k2Split.tallItems = 0;
        for (int i : k2Order)
            if (a->deferredOwner && 2 * a->M[i] > tallest)
            {
                a->k2Split.tallUnits += owner_form_units(a->M[i], a->sN[r][i]);
                a->k2Split.tallItems += (int) ((a->sN[r][i] + 31) / 32);
            }
    }
    for (int i : k2Order)
    {
        const int64_t M = a->M[i];
        if (K > 1 && a->sN[r][i] > 0)
        {
            QTensor q2 = {};
            fill_layout(&q2, M, a->sN[r][i], a->bits);
            q2.res_in = a->sres[i];
            q2.res_out = a->sres[i];
            q2.lv = a->deferredOwner ? a->slv[i] : nullptr;
            if (a->deferredOwner)
            {
                // columns of the earlier tensors' stripes come first in the per-column arrays (slv is laid out the same way)
                q2.stats = static_cast<unsigned*>(a->ownStats.p) + (a->slv[i] - static_cast<float*>(a->slvAll.p));
                q2.unit0 = a->k2Units;
                a->k2Units += owner_form_units(M, q2.N);
            }
            q2.selfRaw = (a->flags & QAGG_SELF_QUANTIZED) ? 0 : 1;
            q2.nsrc = K;
            q2.src[0] = a->recv_slot(r) + a->tOff[r][i];
            int s = 1;
            for (int src = 0; src < K; ++src)
                if (src != r)
                    q2.src[s++] = a->recv_slot(src) + a->tOff[r][i];
            q2.pk[0] = a->gather_slot(r) + a->tOff[r][i];
            q2.bcast = (a->peer && !a->pushGather) ? 1 : 0; // also into slot r of every peer's gather buffer
            q2.bcastOff = a->tOff[r][i];
            const int e = (int) a->hK2.size();
            a->hK2.push_back(q2);
            k2Shapes.push_back({M, q2.N});
            a->k2Tensor.push_back(i);
            std::vector<QItem> tmp;
            make_items(tmp, e, M, q2.N, c2[i]);
            for (auto& it : tmp)
                cost2.push_back({M * it.ncols, it});
        }
    }
    // tallest work first: the ordered walk of a column takes time proportional to its height
    auto byCost = [](const std::pair<int64_t, QItem>& x, const std::pair<int64_t, QItem>& y) { return x.first > y.first; };
    std::stable_sort(cost1.begin(), cost1.end(), byCost);
    std::stable_sort(cost2.begin(), cost2.end(), byCost);
    for (auto& c : cost1)
        a->iK1.push_back(c.second);
    for (auto& c : cost2)
        a->iK2.push_back(c.second);
    if (a->deferred)
    {
        // the streaming kernels size and order their own work items
        std::vector<std::pair<long long, long long>> k1Shapes;
        for (int i = 0; i < T; ++i)
            k1Shapes.push_back({a->M[i], (a->M[i] > 0 && a->N[i] > 0) ? a->N[i] : 0});
        // very tall matrices leave the streaming kernel (tuning knob, results never change: QAGG_TALL_ROWS=<rows>, 0 = never)
        long long tallRows = 16384;
        if (const char* e = std::getenv("QAGG_TALL_ROWS"))
            tallRows = std::atoll(e);
        a->hK1t.clear();
        a->k1tTensor.clear();
        a->k1tCol.clear();
        a->iK1t.clear();
        a->k1tUnits = 0;
        std::vector<std::pair<long long, long long>> tallShapes;
        long long tallCols = 0;
        for (int i = 0; i < T; ++i)
        {
            const bool whole = a->col0[i] == 0 && a->parentN[i] == a->N[i];
            if (!(tallRows > 0 && a->M[i] >= tallRows && a->N[i] > 0 && (a->M[i] & 3) == 0 && whole && a->bits == 1))
                continue;
            k1Shapes[i].second = 0; // no streaming work items for this matrix
            for (int p = 0; p < K; ++p)
            {
                const long long s0 = (K == 1) ? 0 : a->sStart[p][i], n = (K == 1) ? a->N[i] : a->sN[p][i];
                if (n <= 0)
                    continue;
                QTensor e = {};
                fill_layout(&e, a->M[i], n, a->bits);
                e.res_in = e.res_out = a->res[i] + s0 * a->M[i];
                e.lv = a->lv[i] + 2 * s0;
                e.nsrc = 1;
                e.selfRaw = 1;
                e.pk[0] = a->hK1[i].pk[p]; // owner p's block of this matrix: its first column is that owner's stripe start
                e.unit0 = a->k1tUnits;
                a->k1tUnits += owner_form_units(a->M[i], n);
                a->hK1t.push_back(e);
                a->k1tTensor.push_back(i);
                a->k1tCol.push_back(s0);
                tallShapes.push_back({a->M[i], n});
                tallCols += n;
            }
        }
        if (!a->hK1t.empty())
        {
            int rc;
            if (!a->k1tStats.p || a->k1tStats.bytes < (size_t) tallCols * 8)
            {
                if (a->k1tStats.p)
                    cudaFree(a->k1tStats.p);
                a->k1tStats.p = nullptr;
                if ((rc = a->k1tStats.alloc((size_t) tallCols * 8, true)))
                    return rc;
            }
            if (!a->k1tMaps.p || a->k1tMaps.bytes < a->hK1t.size() * 128)
            {
                if (a->k1tMaps.p)
                    cudaFree(a->k1tMaps.p);
                a->k1tMaps.p = nullptr;
                if ((rc = a->k1tMaps.alloc(a->hK1t.size() * 128, true)))
                    return rc;
            }
            if (!a->k1tCounters.p && (rc = a->k1tCounters.alloc(QAGG_COUNTER_UINTS * sizeof(unsigned), true)))
                return rc;
            long long col = 0;
            std::vector<unsigned char> maps(a->hK1t.size() * 128);
            bool mapsOk = true;
            for (size_t e = 0; e < a->hK1t.size(); ++e)
            {
                a->hK1t[e].stats = static_cast<unsigned*>(a->k1tStats.p) + 2 * col;
                col += a->hK1t[e].N;
                mapsOk = owner_set_map(&a->hK1t[e], maps.data() + e * 128, static_cast<unsigned char*>(a->k1tMaps.p) + e * 128) && mapsOk;
            }
            (void) mapsOk; // an entry without a map is walked from global memory by the walk kernel
            if ((rc = check_cuda(cudaMemcpy(a->k1tMaps.p, maps.data(), maps.size(), cudaMemcpyHostToDevice), "tensor map upload")))
                return rc;
            owner_make_items(tallShapes, a->iK1t);
            if (!a->k1Side)
            {
                if ((rc = check_cuda(cudaStreamCreateWithFlags(&a->k1Side, cudaStreamNonBlocking), "cudaStreamCreate")) ||
                    (rc = check_cuda(cudaEventCreateWithFlags(&a->k1Fork, cudaEventDisableTiming), "cudaEventCreate")) ||
                    (rc = check_cuda(cudaEventCreateWithFlags(&a->k1Join, cudaEventDisableTiming), "cudaEventCreate")))
                    return rc;
            }
        }
        std::vector<std::pair<int, int>> box;
        stream_make_items(k1Shapes, a->cfg.numSMs, a->bits, a->iK1, box);
        for (int i = 0; i < T; ++i)
        {
            a->hK1[i].boxCols[0] = box[i].first;
            a->hK1[i].boxCols[1] = box[i].second;
        }
        a->hostMaps.assign(a->hK1.size() * (size_t) QAGG_STREAM_MAP_BYTES, 0);
    }
    if (a->deferredOwner && !a->hK2.empty())
    {
        // the owner kernels: walk items, and one tensor map per owned stripe (it covers the stripe residual, whose address
        // does not depend on the bound gradients, so it is made and uploaded here)
        owner_make_items(k2Shapes, a->iK2);
        std::vector<unsigned char> maps(a->hK2.size() * 128);
        for (size_t e = 0; e < a->hK2.size(); ++e)
            owner_set_map(&a->hK2[e], maps.data() + e * 128, static_cast<unsigned char*>(a->ownMaps.p) + e * 128);
        int rc = check_cuda(cudaMemcpy(a->ownMaps.p, maps.data(), maps.size(), cudaMemcpyHostToDevice), "tensor map upload");
        if (rc)
            return rc;
        // the tall matrices' walk on a stream of its own (tuning knob, results never change: QAGG_OWNER_SPLIT=0 keeps one
        // form and one walk launch)
        bool wantSplit = a->k2Split.tallItems > 0 && a->k2Split.tallItems < (int) a->iK2.size() &&
                         8 * std::min(a->k2Split.tallItems, a->cfg.numSMs) <= a->cfg.numSMs; // launch_owner's own condition
        if (const char* e = std::getenv("QAGG_OWNER_SPLIT"))
            if (e[0] == '0')
                wantSplit = false;
        if (wantSplit && !a->k2Split.side)
        {
            if ((rc = check_cuda(cudaStreamCreateWithFlags(&a->k2Split.side, cudaStreamNonBlocking), "cudaStreamCreate")) ||
                (rc = check_cuda(cudaEventCreateWithFlags(&a->k2Split.fork, cudaEventDisableTiming), "cudaEventCreate")) ||
                (rc = check_cuda(cudaEventCreateWithFlags(&a->k2Split.join, cudaEventDisableTiming), "cudaEventCreate")))
                return rc;
        }
        a->k2SplitOn = wantSplit;
    }
    return QAGG_OK;
}

size_t table_bytes(const qagg_aggregator* a)
{
    return (a->hK1.size() + a->hK2.size() + a->hK3.size() + a->hK1t.size()) * sizeof(QTensor) +
           (a->iK1.size() + a->iK2.size() + a->iK1t.size()) * sizeof(QItem) + 256;
}

// copies the host tables to table set `slot` on the device (synchronously: only when a new array of gradient pointers is bound)
int upload_tables(qagg_aggregator* a, int slot)
{
    unsigned char* base = static_cast<unsigned char*>(a->tables.p) + (size_t) slot * a->tableBytes;
    size_t off = 0;
    auto put = [&](const void* src, size_t bytes, void** devp) -> int {
        *devp = base + off;
        if (bytes)
        {
            int rc = check_cuda(cudaMemcpy(base + off, src, bytes, cudaMemcpyHostToDevice), "table upload");
            if (rc)
                return rc;
        }
        off += align_up((int64_t) bytes, 16);
        return QAGG_OK;
    };
    int rc;
    if ((rc = put(a->hK1.data(), a->hK1.size() * sizeof(QTensor), (void**) &a->dK1)))
        return rc;
    if ((rc = put(a->hK2.data(), a->hK2.size() * sizeof(QTensor), (void**) &a->dK2)))
        return rc;
    if ((rc = put(a->hK3.data(), a->hK3.size() * sizeof(QTensor), (void**) &a->dK3)))
        return rc;
    if ((rc = put(a->iK1.data(), a->iK1.size() * sizeof(QItem), (void**) &a->dI1)))
        return rc;
    if ((rc = put(a->iK2.data(), a->iK2.size() * sizeof(QItem), (void**) &a->dI2)))
        return rc;
    if ((rc = put(a->hK1t.data(), a->hK1t.size() * sizeof(QTensor), (void**) &a->dK1t)))
        return rc;
    if ((rc = put(a->iK1t.data(), a->iK1t.size() * sizeof(QItem), (void**) &a->dI1t)))
        return rc;
    return QAGG_OK;
}

int bind_grads(qagg_aggregator* a, float* const* grads, cudaStream_t st)
{
    for (int s = 0; s < 2; ++s)
    {
        const qagg_aggregator::Binding& b = a->bindings[s];
        bool same = (b.grads.size() == (size_t) a->T) && b.dK3 != nullptr;
        for (int i = 0; same && i < a->T; ++i)
            same = (b.grads[i] == grads[i]);
        if (same)
        {
            a->curBinding = s;
            a->dK1 = b.dK1;
            a->dK2 = b.dK2;
            a->dK3 = b.dK3;
            a->dI1 = b.dI1;
            a->dI2 = b.dI2;
            a->dK1t = b.dK1t;
            a->dI1t = b.dI1t;
            return QAGG_OK;
        }
    }
    // not bound yet: take the set that is not the current one (the first call takes set 0)
    const int slot = a->bindings[a->curBinding].dK3 ? (a->curBinding ^ 1) : a->curBinding;
    for (int i = 0; i < a->T; ++i)
    {
        if (!grads[i] && a->M[i] * a->N[i] > 0)
            return fail(QAGG_EINVAL, "qagg_agg_step: null gradient pointer");
        a->hK1[i].grad = grads[i];
        a->hK3[i].out = grads[i];
    }
    const int r = a->comm->rank;
    for (size_t e = 0; e < a->hK2.size(); ++e)
    {
        const int i = a->k2Tensor[e];
        a->hK2[e].grad = grads[i] + a->sStart[r][i] * a->M[i];
    }
    for (size_t e = 0; e < a->hK1t.size(); ++e)
        a->hK1t[e].grad = grads[a->k1tTensor[e]] + a->k1tCol[e] * a->M[a->k1tTensor[e]];
    // an earlier step may still be reading the tables of that set -- on this stream or on the one it was enqueued on
    int rc = check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize");
    if (rc)
        return rc;
    if (a->stepped && a->lastStream != st && (rc = check_cuda(cudaStreamSynchronize(a->lastStream), "cudaStreamSynchronize")))
        return rc;
    if (a->deferred)
    {
        // the streaming kernels fetch gradient and residual tiles through tensor maps, which hold the base addresses
        unsigned char* dev = static_cast<unsigned char*>(a->tmaps.p) + (size_t) slot * align_up((int64_t) a->hostMaps.size(), 128);
        for (size_t i = 0; i < a->hK1.size(); ++i)
            stream_set_maps(&a->hK1[i], a->hostMaps.data() + i * QAGG_STREAM_MAP_BYTES, dev + i * QAGG_STREAM_MAP_BYTES);
        if (!a->hostMaps.empty())
            if ((rc = check_cuda(cudaMemcpy(dev, a->hostMaps.data(), a->hostMaps.size(), cudaMemcpyHostToDevice), "tensor map upload")))
                return rc;
    }
    rc = upload_tables(a, slot);
    if (rc)
        return rc;
    qagg_aggregator::Binding& b = a->bindings[slot];
    b.grads.assign(grads, grads + a->T);
    b.dK1 = a->dK1;
    b.dK2 = a->dK2;
    b.dK3 = a->dK3;
    b.dI1 = a->dI1;
    b.dI2 = a->dI2;
    b.dK1t = a->dK1t;
    b.dI1t = a->dI1t;
    a->curBinding = slot;
    return QAGG_OK;
}

// peer mode, process group, streaming quantize kernel: the header values are pushed by that kernel's first CTA and summed by
// the flag wait that follows, instead of by two small kernels of their own
bool header_rides_with_k1(const qagg_aggregator* a)
{
    return a->hdrN > 0 && a->comm->K > 1 && a->peer && !a->comm->local && a->deferred && !a->iK1.empty();
}

// peer mode: which flag words (one per peer, indexed by this rank) the kernel releases when it is done
Signal make_signal(const qagg_aggregator* a, bool gatherPhase)
{
    Signal sg = {};
    if (!a->peer)
        return sg;
    const int K = a->comm->K, r = a->comm->rank;
    for (int p = 0; p < K; ++p)
    {
        if (p == r)
            continue;
        sg.flag[sg.n++] = a->peer_flags(p) + (gatherPhase ? 64 : 0) + r;
        if (gatherPhase)
            sg.bcastBase[sg.nbcast++] = a->peer_gather_slot(p, r);
    }
    sg.value = a->stepNo;
    if (!gatherPhase && header_rides_with_k1(a))
    {
        sg.hdrIn = a->hdrHost;
        sg.hdrN = a->hdrN;
        for (int p = 0; p < K; ++p)
            sg.hdrDst[sg.hdrDstN++] = a->header_slot(a->peerWin[p], r);
    }
    return sg;
}
int launch_k1(qagg_aggregator* a, cudaStream_t st)
{
    const Signal sg = make_signal(a, false);
    if (a->deferred && !a->hK1t.empty())
    {
        // Very tall matrices: formed first, then walked on this stream while the streaming kernel takes the other matrices on
        // a second stream (it is made to wait for the form launch only so that the walk, a same-stream successor, gets its
        // SMs first: one walk CTA fills an SM's shared memory).  The flags are released by a kernel of their own once both
        // are done; the header values still ride with the streaming kernel.
        Signal quiet = sg;
        quiet.n = 0;
        int rc = check_cuda(launch_owner(st, a->dK1t, (int) a->hK1t.size(), a->k1tUnits, a->dI1t, (int) a->iK1t.size(), a->cfg,
                                         static_cast<unsigned*>(a->k1tCounters.p), nullptr, a->status_word(), nullptr, a->k1Fork), "quantize launch (tall matrices)");
        if (rc)
            return rc;
        if ((rc = check_cuda(cudaStreamWaitEvent(a->k1Side, a->k1Fork, 0), "cudaStreamWaitEvent")))
            return rc;
        if (!a->iK1.empty() &&
            (rc = check_cuda(launch_stream1(a->k1Side, a->dK1, a->dI1, (int) a->iK1.size(), a->cfg, static_cast<unsigned*>(a->queue.p), &quiet, a->status_word()),
                             "quantize launch")))
            return rc;
        if ((rc = check_cuda(cudaEventRecord(a->k1Join, a->k1Side), "cudaEventRecord")) ||
            (rc = check_cuda(cudaStreamWaitEvent(st, a->k1Join, 0), "cudaStreamWaitEvent")))
            return rc;
        return sg.n > 0 ? check_cuda(launch_signal_only(st, sg), "flag release launch") : QAGG_OK;
    }
    if (a->deferred)
        return check_cuda(launch_stream1(st, a->dK1, a->dI1, (int) a->iK1.size(), a->cfg, static_cast<unsigned*>(a->queue.p), &sg, a->status_word()),
                          "quantize launch");
    return check_cuda(launch_colquant(st, false, a->mode, nullptr, a->dK1, a->dI1, (int) a->iK1.size(), 0, a->cfg,
                                      static_cast<unsigned*>(a->queue.p), &sg), "quantize launch");
}
int launch_k2(qagg_aggregator* a, cudaStream_t st)
{
    const Signal sg = make_signal(a, true);
    unsigned* q2 = static_cast<unsigned*>(a->queue.p) + QAGG_COUNTER_UINTS;
    if (a->peer && a->pushGather)
    {
        int rc = check_cuda(a->deferredOwner ? launch_owner(st, a->dK2, (int) a->hK2.size(), a->k2Units, a->dI2, (int) a->iK2.size(), a->cfg, q2, nullptr,
                                                            a->status_word(), a->k2SplitOn ? &a->k2Split : nullptr)
                                             : launch_colquant(st, true, a->mode, nullptr, a->dK2, a->dI2, (int) a->iK2.size(), 0, a->cfg, q2, nullptr),
                            "reduce-requantize launch");
        if (rc)
            return rc;
        const int r = a->comm->rank;
        return check_cuda(launch_push(st, a->gather_slot(r), (size_t) a->regionBytes[r], sg, static_cast<unsigned*>(a->queue.p) + 3 * QAGG_COUNTER_UINTS,
                                      a->cfg.numSMs), "gather push launch");
    }
    if (a->deferredOwner)
        return check_cuda(launch_owner(st, a->dK2, (int) a->hK2.size(), a->k2Units, a->dI2, (int) a->iK2.size(), a->cfg, q2, &sg, a->status_word(),
                                       a->k2SplitOn ? &a->k2Split : nullptr),
                          "reduce-requantize launch");
    return check_cuda(launch_colquant(st, true, a->mode, nullptr, a->dK2, a->dI2, (int) a->iK2.size(), 0, a->cfg, q2, &sg),
                      "reduce-requantize launch");
}
int wait_peers(qagg_aggregator* a, bool gatherPhase, cudaStream_t st)
{
    if (!gatherPhase && a->hdrN > 0 && a->comm->K > 1 && !a->comm->local)
    {
        // the scatter wait also sums the header values that the ranks stored before releasing their flags
        HeaderPtrs src = {};
        for (int p = 0; p < a->comm->K; ++p)
            src.p[src.n++] = a->header_slot(static_cast<unsigned char*>(a->window.p), p);
        return check_cuda(launch_wait_flags(st, a->flag_words(), a->comm->K, a->comm->rank, a->stepNo, a->waitPolls, a->status_word(), &src, a->hdrN,
                                            a->hdrHost + QAGG_HEADER_MAX), "flag wait launch");
    }
    return check_cuda(launch_wait_flags(st, a->flag_words() + (gatherPhase ? 64 : 0), a->comm->K, a->comm->rank, a->stepNo, a->waitPolls,
                                        a->status_word()), "flag wait launch");
}
int launch_k3(qagg_aggregator* a, cudaStream_t st)
{
    if (a->updating)
        return check_cuda(launch_unquantize(st, UNQ_UPDATE, a->bits, nullptr, static_cast<const QTensor*>(a->updTable.p), (int) a->hK3.size(), a->k3Units,
                                            a->k3SmemWords, a->cfg, &a->updRule), "unquantize-update launch");
    return check_cuda(launch_unquantize(st, UNQ_STORE, a->bits, nullptr, a->dK3, (int) a->hK3.size(), a->k3Units, a->k3SmemWords, a->cfg), "unquantize launch");
}

// Creation-time handshake (process groups only): every rank must describe the same exchange -- tensor count, shapes, column
// slices, bit width, flags -- or the stripes one rank sends would not be what its peers expect, which no later check would
// catch.  Each rank hashes its description (FNV-1a), cuts the hash into four 16-bit pieces p and all-reduces (p, p * p):
// the pieces agree on all K ranks exactly when K * sum(p^2) == (sum p)^2, every quantity exact in a double.  All ranks see
// the same sums, so all of them fail together.  The reference has no such check (a mismatch there shows as an MPI
// truncation error or a hang); its nearest relative is the dimension check of ResetState
// (Source/1BitSGD/AllReduceDistGradAggregator.h:69-71).
int handshake(qagg_comm* comm, int T, const int64_t* M, const int64_t* N, const int64_t* wholeN, const int64_t* firstCol, int bits, int flags)
{
    if (comm->K == 1 || comm->local)
        return QAGG_OK;
    unsigned long long h = 1469598103934665603ull;
    auto mix = [&h](long long v) {
        for (int b = 0; b < 8; ++b)
        {
            h ^= (unsigned long long) ((v >> (8 * b)) & 0xff);
            h *= 1099511628211ull;
        }
    };
    mix(T);
    mix(bits);
    mix(flags);
    mix(comm->K);
    for (int i = 0; i < T; ++i)
    {
        mix(M[i]);
        mix(N[i]);
        mix(wholeN ? wholeN[i] : N[i]);
        mix(firstCol ? firstCol[i] : 0);
    }
    double v[8];
    for (int j = 0; j < 4; ++j)
    {
        v[j] = (double) ((h >> (16 * j)) & 0xffffull);
        v[4 + j] = v[j] * v[j];
    }
    int rc = qagg_comm_allreduce_f64(comm, v, 8, nullptr);
    if (rc)
        return rc;
    for (int j = 0; j < 4; ++j)
        if ((double) comm->K * v[4 + j] != v[j] * v[j])
            return fail(QAGG_ESTATE, "qagg_agg_create: the ranks do not describe the same exchange (tensor count, shapes, slices, bits or flags differ)");
    return QAGG_OK;
}

} // namespace

extern "C" {

int qagg_plan_create(int rank, int num_ranks, int num_tensors, const int64_t* M, const int64_t* N, int bits, qagg_plan** out)
{
    if (!out)
        return fail(QAGG_EINVAL, "qagg_plan_create: null output");
    std::unique_ptr<qagg_plan> p(new qagg_plan);
    int rc = p->build(rank, num_ranks, num_tensors, M, N, bits);
    if (rc)
        return rc;
    *out = p.release();
    return QAGG_OK;
}

int64_t qagg_plan_region_bytes(const qagg_plan* p, int peer)
{
    if (!p || peer < 0 || peer >= p->K)
        return fail(QAGG_EINVAL, "qagg_plan_region_bytes: bad arguments");
    return p->regionBytes[peer];
}

int64_t qagg_plan_tensor_offset(const qagg_plan* p, int peer, int tensor)
{
    if (!p || peer < 0 || peer >= p->K || tensor < 0 || tensor >= p->T)
        return fail(QAGG_EINVAL, "qagg_plan_tensor_offset: bad arguments");
    return p->tOff[peer][tensor];
}

int64_t qagg_plan_gather_slot_bytes(const qagg_plan* p)
{
    if (!p)
        return fail(QAGG_EINVAL, "null plan");
    return p->gatherSlot;
}

int qagg_plan_destroy(qagg_plan* p)
{
    delete p;
    return QAGG_OK;
}

int64_t qagg_plan_stream_items(int num_tensors, const int64_t* M, const int64_t* N, int bits, int num_sms, int32_t* items, int64_t capacity)
{
    if (num_tensors < 0 || (num_tensors > 0 && (!M || !N)) || !bits_ok(bits) || num_sms < 1 || capacity < 0 || (capacity > 0 && !items))
        return fail(QAGG_EINVAL, "qagg_plan_stream_items: bad arguments");
    std::vector<std::pair<long long, long long>> shapes;
    for (int i = 0; i < num_tensors; ++i)
    {
        if (M[i] < 0 || N[i] < 0 || M[i] > 0x3fffffffLL || N[i] > 0x7fffffffLL)
            return fail(QAGG_EINVAL, "qagg_plan_stream_items: bad tensor shape");
        const long long Q = (M[i] * bits + 31) / 32;
        if (M[i] > 0 && N[i] > 0 && stream_max_cols(Q) < 1)
            return fail(QAGG_EINVAL, "qagg_plan_stream_items: a column is too tall for the streaming kernel");
        shapes.push_back({M[i], (M[i] > 0 && N[i] > 0) ? N[i] : 0});
    }
    std::vector<QItem> out;
    std::vector<std::pair<int, int>> box;
    stream_make_items(shapes, num_sms, bits, out, box);
    for (size_t k = 0; k < out.size() && (int64_t) k < capacity; ++k)
    {
        items[3 * k] = out[k].tensor;
        items[3 * k + 1] = out[k].col0;
        items[3 * k + 2] = out[k].ncols;
    }
    return (int64_t) out.size();
}

int qagg_unique_id(void* out)
{
    if (!out)
        return fail(QAGG_EINVAL, "qagg_unique_id: null pointer");
    static_assert(sizeof(ncclUniqueId) <= QAGG_UNIQUE_ID_BYTES, "unique id does not fit");
    ncclUniqueId id;
    int rc = check_nccl(ncclGetUniqueId(&id), "ncclGetUniqueId");
    if (rc)
        return rc;
    std::memset(out, 0, QAGG_UNIQUE_ID_BYTES);
    std::memcpy(out, &id, sizeof(id));
    return QAGG_OK;
}

int qagg_comm_create(const void* unique_id, int rank, int num_ranks, int device, qagg_comm** out)
{
    if (!out || num_ranks < 1 || num_ranks > QAGG_MAXK || rank < 0 || rank >= num_ranks)
        return fail(QAGG_EINVAL, "qagg_comm_create: bad arguments");
    int rc = check_cuda(cudaSetDevice(device), "cudaSetDevice");
    if (rc)
        return rc;
    std::unique_ptr<qagg_comm> c(new qagg_comm);
    c->rank = rank;
    c->K = num_ranks;
    c->device = device;
    if (num_ranks > 1)
    {
        if (!unique_id)
            return fail(QAGG_EINVAL, "qagg_comm_create: unique id required for more than one rank");
        ncclUniqueId id;
        std::memcpy(&id, unique_id, sizeof(id));
        rc = check_nccl(ncclCommInitRank(&c->nccl, num_ranks, id, rank), "ncclCommInitRank");
        if (rc)
            return rc;
    }
    *out = c.release();
    return QAGG_OK;
}

int qagg_comm_create_local_group(int num_ranks, int device, qagg_comm** out)
{
    if (!out || num_ranks < 1 || num_ranks > QAGG_MAXK)
        return fail(QAGG_EINVAL, "qagg_comm_create_local_group: bad arguments");
    int rc = check_cuda(cudaSetDevice(device), "cudaSetDevice");
    if (rc)
        return rc;
    for (int r = 0; r < num_ranks; ++r)
    {
        qagg_comm* c = new qagg_comm;
        c->rank = r;
        c->K = num_ranks;
        c->device = device;
        c->local = true;
        out[r] = c;
    }
    return QAGG_OK;
}

int qagg_comm_rank(const qagg_comm* c)
{
    return c ? c->rank : fail(QAGG_EINVAL, "null communicator");
}

int qagg_comm_size(const qagg_comm* c)
{
    return c ? c->K : fail(QAGG_EINVAL, "null communicator");
}

int qagg_comm_allreduce_f64(qagg_comm* c, double* host_values, int n, void* stream)
{
    if (!c || !host_values || n < 0 || n > qagg_comm::kMaxScalars)
        return fail(QAGG_EINVAL, "qagg_comm_allreduce_f64: bad arguments (at most 512 values)");
    if (c->K == 1 || n == 0)
        return QAGG_OK;
    if (c->local)
        return fail(QAGG_ESTATE, "qagg_comm_allreduce_f64: not available on an in-process group");
    cudaStream_t st = (cudaStream_t) stream;
    int rc = check_cuda(cudaSetDevice(c->device), "cudaSetDevice");
    if (rc)
        return rc;
    if (!c->scalars && (rc = check_cuda(cudaMalloc(reinterpret_cast<void**>(&c->scalars), qagg_comm::kMaxScalars * sizeof(double)), "cudaMalloc")))
        return rc;
    if ((rc = check_cuda(cudaMemcpyAsync(c->scalars, host_values, n * sizeof(double), cudaMemcpyHostToDevice, st), "header upload")))
        return rc;
    if ((rc = check_nccl(ncclAllReduce(c->scalars, c->scalars, (size_t) n, ncclDouble, ncclSum, c->nccl, st), "ncclAllReduce")))
        return rc;
    if ((rc = check_cuda(cudaMemcpyAsync(host_values, c->scalars, n * sizeof(double), cudaMemcpyDeviceToHost, st), "header download")))
        return rc;
    return check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize");
}

int qagg_comm_barrier(qagg_comm* c, void* stream)
{
    double one = 1.0;
    if (c && c->local)
        return QAGG_OK;
    return qagg_comm_allreduce_f64(c, &one, 1, stream);
}

int qagg_comm_destroy(qagg_comm* c)
{
    if (!c)
        return QAGG_OK;
    int rc = QAGG_OK;
    if (c->scalars)
        cudaFree(c->scalars);
    if (c->nccl)
        rc = check_nccl(ncclCommDestroy(c->nccl), "ncclCommDestroy");
    delete c;
    return rc;
}

int qagg_agg_create(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, int bits, int flags, qagg_aggregator** out)
{
    return qagg_agg_create_slices(comm, num_tensors, M, N, nullptr, nullptr, bits, flags, out);
}

int qagg_agg_create_slices(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, const int64_t* whole_N, const int64_t* first_col,
                           int bits, int flags, qagg_aggregator** out)
{
    if (!comm || !out || num_tensors < 0 || (num_tensors > 0 && (!M || !N)) || ((whole_N == nullptr) != (first_col == nullptr)))
        return fail(QAGG_EINVAL, "qagg_agg_create: bad arguments");
    if (!bits_ok(bits))
        return fail(QAGG_EINVAL, "bits must be a power of two in 1..32");
    for (int i = 0; i < num_tensors; ++i)
        if (M[i] < 0 || N[i] < 0 || M[i] > 0x3fffffffLL || N[i] > 0x7fffffffLL)
            return fail(QAGG_EINVAL, "qagg_agg_create: bad tensor shape");
    int rc = check_cuda(cudaSetDevice(comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    if ((rc = handshake(comm, num_tensors, M, N, whole_N, first_col, bits, flags)))
        return rc;
    std::unique_ptr<qagg_aggregator> a(new qagg_aggregator);
    a->comm = comm;
    a->T = num_tensors;
    a->bits = bits;
    a->flags = flags;
    a->mode = mode_of(bits, flags & QAGG_ZERO_THRESHOLD);
    const int K = comm->K, r = comm->rank;
    a->identity = (K == 1) && (flags & QAGG_V2_IDENTITY_K1);
    if (const char* e = std::getenv("QAGG_PUSH_GATHER")) // tuning knob: 0 = requantize kernel stores to the peers itself
        a->pushGather = (e[0] != '0');
    // 1 bit, threshold 0: the quantize kernel streams with a deferred residual, unless a column is too tall for that.
    // The owner's reduce-requantize is then the form + walk kernel pair, which keeps the stripe residuals deferred too.
    // Tuning knobs (results never change): QAGG_STREAM=0 resident-column kernels only; QAGG_OWNER=0 resident-column kernel
    // for the owner only.
    a->deferred = (a->mode == MODE_ONEBIT_ZERO);
    for (int i = 0; i < num_tensors; ++i)
        if (M[i] > 0 && N[i] > 0 && stream_max_cols((M[i] * bits + 31) / 32) < 1)
            a->deferred = false;
    if (const char* e = std::getenv("QAGG_STREAM"))
        if (e[0] == '0')
            a->deferred = false;
    a->deferredOwner = a->deferred && K > 1;
    if (const char* e = std::getenv("QAGG_OWNER"))
        if (e[0] == '0')
            a->deferredOwner = false;
    rc = check_cuda(get_launch_cfg(comm->device, &a->cfg), "cudaGetDeviceProperties");
    if (rc)
        return rc;
    qagg_plan plan;
    if ((rc = plan.build(r, K, num_tensors, M, N, bits, whole_N, first_col)))
        return rc;
    a->M = plan.M;
    a->N = plan.N;
    a->parentN = plan.parentN;
    a->col0 = plan.col0;
    a->colBytes = plan.colBytes;
    a->sStart = plan.sStart;
    a->sN = plan.sN;
    a->tOff = plan.tOff;
    a->regionBytes = plan.regionBytes;
    a->gatherSlot = plan.gatherSlot;
    int64_t resFloats = 0, sresFloats = 0;
    for (int i = 0; i < num_tensors; ++i)
    {
        a->totalValues += M[i] * N[i];
        resFloats += align_up(M[i] * N[i], 4);
    }
    a->sendOff.assign(K, 0);
    int64_t sendTotal = 0;
    for (int p = 0; p < K; ++p)
    {
        a->sendOff[p] = sendTotal;
        sendTotal += align_up(a->regionBytes[p], 256);
    }
    a->slotBytes = align_up(a->regionBytes[r], 256);
    for (int i = 0; i < num_tensors; ++i)
        sresFloats += align_up(M[i] * a->sN[r][i], 4);

    if ((rc = a->sendbuf.alloc((size_t) sendTotal, true)))
        return rc;
    if ((rc = a->window.alloc((size_t) (qagg_aggregator::kFlagBytes + a->slotBytes * K + a->gatherSlot * K), true)))
        return rc;
    a->recvbuf = static_cast<unsigned char*>(a->window.p) + qagg_aggregator::kFlagBytes;
    a->gatherbuf = a->recvbuf + a->slotBytes * K;
    if ((rc = a->resAll.alloc((size_t) resFloats * 4, true)))
        return rc;
    if ((rc = a->sresAll.alloc((size_t) sresFloats * 4, true)))
        return rc;
    a->res.resize(num_tensors);
    a->sres.resize(num_tensors);
    a->lv.assign(num_tensors, nullptr);
    a->slv.assign(num_tensors, nullptr);
    if (a->deferred)
    {
        int64_t cols = 0, scols = 0;
        for (int i = 0; i < num_tensors; ++i)
        {
            cols += N[i];
            scols += a->sN[r][i];
        }
        if ((rc = a->lvAll.alloc((size_t) cols * 8, true)))
            return rc;
        if ((rc = a->slvAll.alloc((size_t) scols * 8, true)))
            return rc;
        if ((rc = a->ownStats.alloc((size_t) scols * 8, true)))
            return rc;
        if ((rc = a->ownMaps.alloc((size_t) std::max(num_tensors, 1) * 128, true)))
            return rc;
    }
    int64_t ro = 0, so = 0, lo = 0, slo = 0;
    for (int i = 0; i < num_tensors; ++i)
    {
        a->res[i] = static_cast<float*>(a->resAll.p) + ro;
        ro += align_up(M[i] * N[i], 4);
        a->sres[i] = (a->sN[r][i] > 0 && K > 1) ? static_cast<float*>(a->sresAll.p) + so : nullptr;
        so += align_up(M[i] * a->sN[r][i], 4);
        if (a->deferred)
        {
            a->lv[i] = static_cast<float*>(a->lvAll.p) + lo;
            a->slv[i] = static_cast<float*>(a->slvAll.p) + slo;
            lo += 2 * N[i];
            slo += 2 * a->sN[r][i];
        }
    }
    if ((rc = build_tables(a.get())))
        return rc;
    a->tableBytes = (size_t) align_up((int64_t) table_bytes(a.get()), 256);
    if ((rc = a->tables.alloc(2 * a->tableBytes, true)))
        return rc;
    if (a->deferred)
        if ((rc = a->tmaps.alloc(2 * (size_t) align_up((int64_t) a->hostMaps.size(), 128) + 128, true)))
            return rc;
    if ((rc = a->queue.alloc(4 * QAGG_COUNTER_UINTS * sizeof(unsigned), true)))
        return rc;
    *out = a.release();
    return QAGG_OK;
}

static int exchange_scatter(qagg_aggregator* a, cudaStream_t st)
{
    const int K = a->comm->K, r = a->comm->rank;
    int rc = check_nccl(ncclGroupStart(), "ncclGroupStart");
    if (rc)
        return rc;
    for (int p = 0; p < K; ++p)
    {
        if (p == r)
            continue;
        if (a->regionBytes[p] > 0)
            if ((rc = check_nccl(ncclSend(a->send_region(p), (size_t) a->regionBytes[p], ncclChar, p, a->comm->nccl, st), "ncclSend")))
                return rc;
        if (a->regionBytes[r] > 0)
            if ((rc = check_nccl(ncclRecv(a->recv_slot(p), (size_t) a->regionBytes[r], ncclChar, p, a->comm->nccl, st), "ncclRecv")))
                return rc;
    }
    return check_nccl(ncclGroupEnd(), "ncclGroupEnd");
}

static int exchange_gather(qagg_aggregator* a, cudaStream_t st)
{
    const int r = a->comm->rank;
    return check_nccl(ncclAllGather(a->gather_slot(r), a->gatherbuf, (size_t) a->gatherSlot, ncclChar, a->comm->nccl, st), "ncclAllGather");
}

namespace {

// the step's header goes into the pinned buffer (and, with one rank, straight to the result)
int stage_header(qagg_aggregator* a, const double* header, int n)
{
    if (n < 0 || n > QAGG_HEADER_MAX || (n > 0 && !header))
        return fail(QAGG_EINVAL, "header: at most 64 doubles");
    a->hdrN = n;
    if (n == 0)
        return QAGG_OK;
    if (!a->hdrHost)
    {
        int rc = check_cuda(cudaHostAlloc(reinterpret_cast<void**>(&a->hdrHost), 2 * QAGG_HEADER_MAX * sizeof(double), cudaHostAllocMapped | cudaHostAllocPortable),
                            "cudaHostAlloc");
        if (rc)
            return rc;
        std::memset(a->hdrHost, 0, 2 * QAGG_HEADER_MAX * sizeof(double));
    }
    std::memcpy(a->hdrHost, header, (size_t) n * sizeof(double));
    if (a->comm->K == 1)
        std::memcpy(a->hdrHost + QAGG_HEADER_MAX, header, (size_t) n * sizeof(double));
    return QAGG_OK;
}

// peer mode, before the quantize kernel: this rank's header into slot `rank` of every rank's window (its own included); the
// quantize kernel's flag release, which follows on the stream, publishes it together with the packed stripes
int push_header(qagg_aggregator* a, cudaStream_t st)
{
    if (a->hdrN == 0 || a->comm->K == 1 || !a->peer || header_rides_with_k1(a))
        return QAGG_OK;
    HeaderPtrs dst = {};
    for (int p = 0; p < a->comm->K; ++p)
        dst.p[dst.n++] = a->header_slot(a->peerWin[p], a->comm->rank);
    return check_cuda(launch_header_push(st, a->hdrHost, a->hdrN, dst), "header push launch");
}

// after the scatter (flag wait or send/recv): the sum over ranks into the pinned result
int sum_header(qagg_aggregator* a, cudaStream_t st)
{
    if (a->hdrN == 0 || a->comm->K == 1)
        return QAGG_OK;
    double* out = a->hdrHost + QAGG_HEADER_MAX;
    if (a->peer && !a->comm->local)
        return QAGG_OK; // summed by the scatter wait (wait_peers)
    if (a->peer)
    {
        HeaderPtrs src = {};
        for (int p = 0; p < a->comm->K; ++p)
            src.p[src.n++] = a->header_slot(static_cast<unsigned char*>(a->window.p), p);
        return check_cuda(launch_header_sum(st, src, a->hdrN, out), "header sum launch");
    }
    int rc;
    if (!a->hdrDev && (rc = check_cuda(cudaMalloc(reinterpret_cast<void**>(&a->hdrDev), QAGG_HEADER_MAX * sizeof(double)), "cudaMalloc")))
        return rc;
    if ((rc = check_cuda(cudaMemcpyAsync(a->hdrDev, a->hdrHost, (size_t) a->hdrN * sizeof(double), cudaMemcpyHostToDevice, st), "header upload")))
        return rc;
    if ((rc = check_nccl(ncclAllReduce(a->hdrDev, a->hdrDev, (size_t) a->hdrN, ncclDouble, ncclSum, a->comm->nccl, st), "ncclAllReduce")))
        return rc;
    return check_cuda(cudaMemcpyAsync(out, a->hdrDev, (size_t) a->hdrN * sizeof(double), cudaMemcpyDeviceToHost, st), "header download");
}

} // namespace

extern "C" int qagg_agg_step_header(qagg_aggregator* a, float* const* grads, const double* header, int n, void* stream);

int qagg_agg_step(qagg_aggregator* a, float* const* grads, void* stream)
{
    return qagg_agg_step_header(a, grads, nullptr, 0, stream);
}

int qagg_agg_step_header(qagg_aggregator* a, float* const* grads, const double* header, int n, void* stream)
{
    if (!a || (a->T > 0 && !grads))
        return fail(QAGG_EINVAL, "qagg_agg_step: bad arguments");
    if (a->comm->local && a->comm->K > 1)
        return fail(QAGG_ESTATE, "aggregators of a local group must be stepped with qagg_agg_step_group");
    {
        int hrc = stage_header(a, header, n);
        if (hrc)
            return hrc;
    }
    if (a->identity || a->totalValues == 0)
    {
        // nothing to aggregate, but the header is still summed over the ranks
        if (a->hdrN > 0 && a->comm->K > 1)
        {
            if (a->comm->local)
                return fail(QAGG_ESTATE, "header exchange of a local group needs qagg_agg_step_group_header");
            std::memcpy(a->hdrHost + QAGG_HEADER_MAX, a->hdrHost, (size_t) a->hdrN * sizeof(double));
            return qagg_comm_allreduce_f64(a->comm, a->hdrHost + QAGG_HEADER_MAX, a->hdrN, stream);
        }
        return QAGG_OK;
    }
    cudaStream_t st = (cudaStream_t) stream;
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    if ((rc = bind_grads(a, grads, st)))
        return rc;
    a->lastStream = st;
    a->stepped = true;
    a->stepNo++;
    if ((rc = a->mark(0, st)))
        return rc;
    if ((rc = push_header(a, st)))
        return rc;
    if ((rc = launch_k1(a, st)))
        return rc;
    if ((rc = a->mark(1, st)))
        return rc;
    if (a->comm->K > 1)
    {
        if ((rc = a->peer ? wait_peers(a, false, st) : exchange_scatter(a, st)))
            return rc;
        if ((rc = sum_header(a, st)))
            return rc;
        if ((rc = a->mark(2, st)))
            return rc;
        if ((rc = launch_k2(a, st)))
            return rc;
        if ((rc = a->mark(3, st)))
            return rc;
        if ((rc = a->peer ? wait_peers(a, true, st) : exchange_gather(a, st)))
            return rc;
    }
    else
    {
        if ((rc = a->mark(2, st)) || (rc = a->mark(3, st)))
            return rc;
    }
    if ((rc = a->mark(4, st)))
        return rc;
    if ((rc = launch_k3(a, st)))
        return rc;
    if ((rc = a->mark(5, st)))
        return rc;
    if (a->profiling)
        a->profSteps++;
    return QAGG_OK;
}

int qagg_agg_header_result(qagg_aggregator* a, double* out, int n, void* stream)
{
    if (!a || n < 0 || n > QAGG_HEADER_MAX || (n > 0 && !out))
        return fail(QAGG_EINVAL, "qagg_agg_header_result: bad arguments");
    if (n != a->hdrN)
        return fail(QAGG_ESTATE, "qagg_agg_header_result: the last step carried a header of a different length");
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    if ((rc = check_cuda(cudaStreamSynchronize((cudaStream_t) stream), "cudaStreamSynchronize")))
        return rc;
    if (n > 0)
        std::memcpy(out, a->hdrHost + QAGG_HEADER_MAX, (size_t) n * sizeof(double));
    return QAGG_OK;
}

int qagg_agg_set_profiling(qagg_aggregator* a, int enabled)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    if (enabled)
    {
        int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
        if (rc)
            return rc;
        for (auto& slot : a->ev)
            for (auto& e : slot)
                if (!e && (rc = check_cuda(cudaEventCreate(&e), "cudaEventCreate")))
                    return rc;
    }
    a->profiling = enabled != 0;
    a->profSteps = 0;
    return QAGG_OK;
}

int qagg_agg_phase_ms(qagg_aggregator* a, float* out5)
{
    if (!a || !out5)
        return fail(QAGG_EINVAL, "qagg_agg_phase_ms: bad arguments");
    if (a->profSteps == 0)
        return fail(QAGG_ESTATE, "qagg_agg_phase_ms: no profiled step has been recorded");
    const long long n = std::min<long long>(a->profSteps, qagg_aggregator::kProfSlots);
    double sum[5] = {0, 0, 0, 0, 0};
    for (long long k = 0; k < n; ++k)
    {
        const int slot = (int) ((a->profSteps - 1 - k) % qagg_aggregator::kProfSlots);
        int rc = check_cuda(cudaEventSynchronize(a->ev[slot][5]), "cudaEventSynchronize");
        if (rc)
            return rc;
        for (int i = 0; i < 5; ++i)
        {
            float ms = 0.f;
            if ((rc = check_cuda(cudaEventElapsedTime(&ms, a->ev[slot][i], a->ev[slot][i + 1]), "cudaEventElapsedTime")))
                return rc;
            sum[i] += ms;
        }
    }
    for (int i = 0; i < 5; ++i)
        out5[i] = (float) (sum[i] / (double) n);
    a->profSteps = 0;
    return QAGG_OK;
}

int qagg_agg_step_group(qagg_aggregator* const* aggs, int num_ranks, float* const* const* grads, void* stream)
{
    return qagg_agg_step_group_header(aggs, num_ranks, grads, nullptr, 0, stream);
}

int qagg_agg_step_group_header(qagg_aggregator* const* aggs, int num_ranks, float* const* const* grads, const double* const* headers, int n,
                               void* stream)
{
    if (!aggs || !grads || num_ranks < 1 || (n > 0 && !headers))
        return fail(QAGG_EINVAL, "qagg_agg_step_group: bad arguments");
    cudaStream_t st = (cudaStream_t) stream;
    const int K = num_ranks;
    for (int r = 0; r < K; ++r)
    {
        if (!aggs[r] || aggs[r]->comm->K != K || aggs[r]->comm->rank != r || !aggs[r]->comm->local)
            return fail(QAGG_ESTATE, "qagg_agg_step_group: aggregators are not ranks 0..K-1 of one local group");
        if (aggs[r]->T != aggs[0]->T || aggs[r]->bits != aggs[0]->bits || aggs[r]->M != aggs[0]->M || aggs[r]->N != aggs[0]->N)
            return fail(QAGG_ESTATE, "qagg_agg_step_group: aggregators disagree on tensor shapes or bits");
    }
    int rc = check_cuda(cudaSetDevice(aggs[0]->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    // the header: every rank's values are in its pinned buffer; one small kernel per rank adds them in rank order (the ranks
    // share this process, so no exchange is needed)
    for (int r = 0; r < K; ++r)
        if ((rc = stage_header(aggs[r], n > 0 ? headers[r] : nullptr, n)))
            return rc;
    if (n > 0 && K > 1)
    {
        HeaderPtrs src = {};
        for (int r = 0; r < K; ++r)
            src.p[src.n++] = aggs[r]->hdrHost;
        for (int r = 0; r < K; ++r)
            if ((rc = check_cuda(launch_header_sum(st, src, n, aggs[r]->hdrHost + QAGG_HEADER_MAX), "header sum launch")))
                return rc;
    }
    if (aggs[0]->identity || aggs[0]->totalValues == 0)
        return QAGG_OK;
    const bool peer = aggs[0]->peer;
    for (int r = 0; r < K; ++r)
        if (aggs[r]->peer != peer)
            return fail(QAGG_ESTATE, "qagg_agg_step_group: peer mode must be enabled on all ranks or on none");
    // Per-phase timing (qagg_agg_set_profiling) on a local group: the events bracket each rank's own three kernels, so
    // phases 0, 2 and 4 (quantize, reduce-requantize, unquantize) are that rank's kernel times; phases 1 and 3 then span
    // the other ranks' kernels and mean nothing here.
    for (int r = 0; r < K; ++r)
    {
        if ((rc = bind_grads(aggs[r], grads[r], st)))
            return rc;
        aggs[r]->lastStream = st;
        aggs[r]->stepped = true;
        aggs[r]->stepNo++;
        if ((rc = aggs[r]->mark(0, st)) || (rc = launch_k1(aggs[r], st)) || (rc = aggs[r]->mark(1, st)))
            return rc;
    }
    if (K > 1 && peer)
    {
        // every rank's kernels run one after the other on this one stream, so each flag is already set when its
        // waiter starts: the waits check the protocol, they never actually spin here
        for (int r = 0; r < K; ++r)
            if ((rc = wait_peers(aggs[r], false, st)))
                return rc;
        for (int r = 0; r < K; ++r)
            if ((rc = aggs[r]->mark(2, st)) || (rc = launch_k2(aggs[r], st)) || (rc = aggs[r]->mark(3, st)))
                return rc;
        for (int r = 0; r < K; ++r)
            if ((rc = wait_peers(aggs[r], true, st)))
                return rc;
    }
    else if (K > 1)
    {
        // scatter: region p of rank r's send buffer -> receive slot r of rank p
        for (int r = 0; r < K; ++r)
            for (int p = 0; p < K; ++p)
                if (p != r && aggs[r]->regionBytes[p] > 0)
                    if ((rc = check_cuda(cudaMemcpyAsync(aggs[p]->recv_slot(r), aggs[r]->send_region(p), (size_t) aggs[r]->regionBytes[p],
                                                         cudaMemcpyDeviceToDevice, st), "stripe copy")))
                        return rc;
        for (int r = 0; r < K; ++r)
            if ((rc = aggs[r]->mark(2, st)) || (rc = launch_k2(aggs[r], st)) || (rc = aggs[r]->mark(3, st)))
                return rc;
        // all-gather: gather slot r of rank r -> gather slot r of every other rank
        for (int r = 0; r < K; ++r)
            for (int p = 0; p < K; ++p)
                if (p != r && aggs[r]->regionBytes[r] > 0)
                    if ((rc = check_cuda(cudaMemcpyAsync(aggs[p]->gather_slot(r), aggs[r]->gather_slot(r), (size_t) aggs[r]->regionBytes[r],
                                                         cudaMemcpyDeviceToDevice, st), "aggregated stripe copy")))
                        return rc;
    }
    for (int r = 0; r < K; ++r)
    {
        if (K == 1 && ((rc = aggs[r]->mark(2, st)) || (rc = aggs[r]->mark(3, st))))
            return rc;
        if ((rc = aggs[r]->mark(4, st)) || (rc = launch_k3(aggs[r], st)) || (rc = aggs[r]->mark(5, st)))
            return rc;
        if (aggs[r]->profiling)
            aggs[r]->profSteps++;
    }
    return QAGG_OK;
}

int qagg_agg_peer_handle(qagg_aggregator* a, void* out)
{
    if (!a || !out)
        return fail(QAGG_EINVAL, "qagg_agg_peer_handle: bad arguments");
    static_assert(sizeof(cudaIpcMemHandle_t) <= QAGG_PEER_HANDLE_BYTES, "IPC handle does not fit");
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    std::memset(out, 0, QAGG_PEER_HANDLE_BYTES);
    if (a->comm->local)
    {
        // ranks of an in-process group share an address space: the "handle" is the window's address
        std::memcpy(out, &a->window.p, sizeof(void*));
        return QAGG_OK;
    }
    cudaIpcMemHandle_t h;
    if ((rc = check_cuda(cudaIpcGetMemHandle(&h, a->window.p), "cudaIpcGetMemHandle")))
        return rc;
    std::memcpy(out, &h, sizeof(h));
    return QAGG_OK;
}

int qagg_agg_enable_peer(qagg_aggregator* a, const void* handles)
{
    if (!a || !handles)
        return fail(QAGG_EINVAL, "qagg_agg_enable_peer: bad arguments");
    if (a->peer)
        return fail(QAGG_ESTATE, "qagg_agg_enable_peer: already enabled");
    const int K = a->comm->K, r = a->comm->rank;
    if (K == 1)
        return QAGG_OK;
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    const unsigned char* hb = static_cast<const unsigned char*>(handles);
    for (int p = 0; p < K; ++p)
    {
        if (p == r)
        {
            a->peerWin[p] = static_cast<unsigned char*>(a->window.p);
            continue;
        }
        if (a->comm->local)
        {
            void* q = nullptr;
            std::memcpy(&q, hb + (size_t) p * QAGG_PEER_HANDLE_BYTES, sizeof(void*));
            a->peerWin[p] = static_cast<unsigned char*>(q);
        }
        else
        {
            cudaIpcMemHandle_t h;
            std::memcpy(&h, hb + (size_t) p * QAGG_PEER_HANDLE_BYTES, sizeof(h));
            void* q = nullptr;
            if ((rc = check_cuda(cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")))
                return rc;
            a->peerWin[p] = static_cast<unsigned char*>(q);
            a->peerOpened[p] = true;
        }
        if (!a->peerWin[p])
            return fail(QAGG_EINVAL, "qagg_agg_enable_peer: null peer window");
    }
    a->peer = true;
    // the routing of the packed columns changes: rebuild and re-upload the tables on the next step
    if ((rc = build_tables(a)))
        return rc;
    for (auto& b : a->bindings)
        b = qagg_aggregator::Binding();
    a->curBinding = 0;
    return QAGG_OK;
}

int qagg_agg_set_wait_limit(qagg_aggregator* a, long long max_polls)
{
    if (!a || max_polls < 1)
        return fail(QAGG_EINVAL, "qagg_agg_set_wait_limit: bad arguments");
    a->waitPolls = max_polls;
    return QAGG_OK;
}

int qagg_agg_check(qagg_aggregator* a, void* stream)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    unsigned st = 0;
    if ((rc = check_cuda(cudaMemcpyAsync(&st, a->status_word(), sizeof(st), cudaMemcpyDeviceToHost, (cudaStream_t) stream), "status read")))
        return rc;
    if ((rc = check_cuda(cudaStreamSynchronize((cudaStream_t) stream), "cudaStreamSynchronize")))
        return rc;
    if (st & 1u)
        return fail(QAGG_ETIMEOUT, "a device-side wait for a peer's flag ran out: a peer did not reach the step (results of that step are invalid)");
    if (st & 2u)
        return fail(QAGG_ETIMEOUT, "a device-side wait for a copy into shared memory ran out (results of that step are invalid)");
    // an asynchronous NCCL error (a peer process died, a link went down) does not show in a launch's return value
    if (a->comm->nccl)
    {
        ncclResult_t asyncErr = ncclSuccess;
        if ((rc = check_nccl(ncclCommGetAsyncError(a->comm->nccl, &asyncErr), "ncclCommGetAsyncError")))
            return rc;
        if (asyncErr != ncclSuccess && asyncErr != ncclInProgress)
            return check_nccl(asyncErr, "asynchronous NCCL error");
    }
    return QAGG_OK;
}

int qagg_agg_clear_status(qagg_aggregator* a, void* stream)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    if ((rc = check_cuda(cudaMemsetAsync(a->status_word(), 0, sizeof(unsigned), (cudaStream_t) stream), "status clear")))
        return rc;
    return check_cuda(cudaStreamSynchronize((cudaStream_t) stream), "cudaStreamSynchronize");
}

int qagg_stream_wait_selftest(void* stream, int max_tries, unsigned* status_dev, long long* cycles_dev)
{
    if (!status_dev || max_tries < 1 || max_tries > (1 << 22))
        return fail(QAGG_EINVAL, "qagg_stream_wait_selftest: bad arguments");
    return check_cuda(launch_stream_wait_selftest((cudaStream_t) stream, max_tries, status_dev, cycles_dev), "wait self-test launch");
}

int qagg_wait_flags(void* stream, const unsigned* flags_dev, int n, int skip, unsigned value, long long max_polls, unsigned* status_dev)
{
    if (!flags_dev || !status_dev || n < 1 || n > 32 || max_polls < 1)
        return fail(QAGG_EINVAL, "qagg_wait_flags: bad arguments");
    return check_cuda(launch_wait_flags((cudaStream_t) stream, flags_dev, n, skip, value, max_polls, status_dev), "flag wait launch");
}

int qagg_agg_step_host(qagg_aggregator* a, float* const* host_grads, void* stream)
{
    if (!a || (a->T > 0 && !host_grads))
        return fail(QAGG_EINVAL, "qagg_agg_step_host: bad arguments");
    cudaStream_t st = (cudaStream_t) stream;
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    if (!a->devGrads.p)
    {
        int64_t floats = 0;
        for (int i = 0; i < a->T; ++i)
            floats += align_up(a->M[i] * a->N[i], 4);
        if ((rc = a->devGrads.alloc((size_t) floats * 4, false)))
            return rc;
        a->devGradPtr.resize(a->T);
        int64_t o = 0;
        for (int i = 0; i < a->T; ++i)
        {
            a->devGradPtr[i] = static_cast<float*>(a->devGrads.p) + o;
            o += align_up(a->M[i] * a->N[i], 4);
        }
    }
    for (int i = 0; i < a->T; ++i)
    {
        const size_t bytes = (size_t) (a->M[i] * a->N[i]) * 4;
        if (bytes && (rc = check_cuda(cudaMemcpyAsync(a->devGradPtr[i], host_grads[i], bytes, cudaMemcpyHostToDevice, st), "gradient upload")))
            return rc;
    }
    if ((rc = qagg_agg_step(a, a->devGradPtr.data(), stream)))
        return rc;
    for (int i = 0; i < a->T; ++i)
    {
        const size_t bytes = (size_t) (a->M[i] * a->N[i]) * 4;
        if (bytes && (rc = check_cuda(cudaMemcpyAsync(host_grads[i], a->devGradPtr[i], bytes, cudaMemcpyDeviceToHost, st), "gradient download")))
            return rc;
    }
    return check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize");
}

// =====================================================================================================================
// Host-buffer aggregator: the same step for callers whose gradients live in host memory.  A tensor's aggregate depends
// on that tensor only, so the gradient set is cut into chunks of consecutive tensors, each with its own aggregator, and
// the chunks are software-pipelined over a few streams: while chunk c computes, chunk c+1 uploads and chunk c-1
// downloads (PCIe is full duplex).  With more than one rank the chunks overlap only in peer mode (each chunk has its
// own window and flags); on the NCCL path they run one after the other on a single stream, because one communicator
// must see its collectives in one order.
// =====================================================================================================================
struct qagg_host_aggregator
{
    qagg_comm* comm = nullptr;
    int T = 0;
    std::vector<int64_t> rows; // rows per tensor
    // A chunk is a list of column slices (tensor, first column, columns) with about the same number of values as every other
    // chunk: small tensors are grouped, large ones cut by COLUMNS.  Columns are independent of each other, and every slice
    // keeps the stripe ownership of its whole tensor (GetStripeForNode on the whole matrix), so the results are
    // bit-identical to aggregating the whole set at once.
    struct Slice
    {
        int tensor;
        int64_t col0, ncols;
    };
    std::vector<std::vector<Slice>> chunks;
    std::vector<qagg_aggregator*> kids;
    // a three-stage pipeline: all uploads on one stream, all kernels on a second, all downloads on a third, so that the
    // upload engine never waits behind a download; chunk c's kernels wait for uploaded[c], its download for computed[c]
    cudaStream_t sIn = nullptr, sCompute = nullptr, sOut = nullptr;
    std::vector<cudaEvent_t> uploaded, computed;
    std::vector<DevBuf> dev;  // one device gradient buffer per chunk
    std::vector<std::vector<float*>> devPtr;
    bool peer = false;
    ~qagg_host_aggregator()
    {
        for (auto* k : kids)
            qagg_agg_destroy(k);
        for (auto e : uploaded)
            cudaEventDestroy(e);
        for (auto e : computed)
            cudaEventDestroy(e);
        for (auto st : {sIn, sCompute, sOut})
            if (st)
                cudaStreamDestroy(st);
    }
};

int qagg_hagg_create(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, int bits, int flags, int num_chunks,
                     qagg_host_aggregator** out)
{
    if (!comm || !out || num_tensors < 1 || !M || !N || num_chunks < 1)
        return fail(QAGG_EINVAL, "qagg_hagg_create: bad arguments");
    int rc = check_cuda(cudaSetDevice(comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    std::unique_ptr<qagg_host_aggregator> h(new qagg_host_aggregator);
    h->comm = comm;
    h->T = num_tensors;
    int64_t total = 0;
    for (int i = 0; i < num_tensors; ++i)
    {
        if (M[i] < 0 || N[i] < 0)
            return fail(QAGG_EINVAL, "qagg_hagg_create: bad tensor shape");
        h->rows.push_back(M[i]);
        total += M[i] * N[i];
    }
    // equal-value chunks of column slices, in tensor order (first and last chunk at half size, so that less of the copies
    // at both ends goes without overlap, measured the same within the noise of the host link: not kept)
    const int64_t target = std::max<int64_t>(1, (total + num_chunks - 1) / num_chunks);
    h->chunks.emplace_back();
    int64_t room = target;
    for (int i = 0; i < num_tensors; ++i)
    {
        int64_t c0 = 0;
        while (c0 < N[i] && M[i] > 0)
        {
            if (room <= 0 && (int) h->chunks.size() < num_chunks)
            {
                h->chunks.emplace_back();
                room = target;
            }
            int64_t take = (int) h->chunks.size() < num_chunks ? std::max<int64_t>(1, room / M[i]) : N[i] - c0;
            take = std::min(take, N[i] - c0);
            h->chunks.back().push_back({i, c0, take});
            room -= take * M[i];
            c0 += take;
        }
    }
    if (h->chunks.back().empty())
        h->chunks.pop_back();
    if (h->chunks.empty())
        h->chunks.emplace_back();
    const int chunks = (int) h->chunks.size();
    h->dev.resize(chunks);
    h->devPtr.resize(chunks);
    for (int c = 0; c < chunks; ++c)
    {
        std::vector<int64_t> cm, cn, pn, pc;
        int64_t floats = 0;
        for (auto& sl : h->chunks[c])
        {
            cm.push_back(M[sl.tensor]);
            cn.push_back(sl.ncols);
            pn.push_back(N[sl.tensor]);
            pc.push_back(sl.col0);
            floats += align_up(M[sl.tensor] * sl.ncols, 4);
        }
        qagg_aggregator* kid = nullptr;
        if ((rc = qagg_agg_create_slices(comm, (int) cm.size(), cm.data(), cn.data(), pn.data(), pc.data(), bits, flags, &kid)))
            return rc;
        h->kids.push_back(kid);
        if ((rc = h->dev[c].alloc((size_t) floats * 4, false)))
            return rc;
        int64_t o = 0;
        for (auto& sl : h->chunks[c])
        {
            h->devPtr[c].push_back(static_cast<float*>(h->dev[c].p) + o);
            o += align_up(M[sl.tensor] * sl.ncols, 4);
        }
    }
    for (cudaStream_t* st : {&h->sIn, &h->sCompute, &h->sOut})
        if ((rc = check_cuda(cudaStreamCreateWithFlags(st, cudaStreamNonBlocking), "cudaStreamCreate")))
            return rc;
    h->uploaded.resize(chunks);
    h->computed.resize(chunks);
    for (int c = 0; c < chunks; ++c)
        if ((rc = check_cuda(cudaEventCreateWithFlags(&h->uploaded[c], cudaEventDisableTiming), "cudaEventCreate")) ||
            (rc = check_cuda(cudaEventCreateWithFlags(&h->computed[c], cudaEventDisableTiming), "cudaEventCreate")))
            return rc;
    *out = h.release();
    return QAGG_OK;
}

int qagg_hagg_chunks(const qagg_host_aggregator* h)
{
    return h ? (int) h->kids.size() : fail(QAGG_EINVAL, "null host aggregator");
}

int qagg_hagg_peer_handles(qagg_host_aggregator* h, void* out)
{
    if (!h || !out)
        return fail(QAGG_EINVAL, "qagg_hagg_peer_handles: bad arguments");
    for (size_t c = 0; c < h->kids.size(); ++c)
    {
        int rc = qagg_agg_peer_handle(h->kids[c], static_cast<unsigned char*>(out) + c * QAGG_PEER_HANDLE_BYTES);
        if (rc)
            return rc;
    }
    return QAGG_OK;
}

int qagg_hagg_enable_peer(qagg_host_aggregator* h, const void* handles)
{
    if (!h || !handles)
        return fail(QAGG_EINVAL, "qagg_hagg_enable_peer: bad arguments");
    const int K = h->comm->K;
    const size_t chunks = h->kids.size();
    std::vector<unsigned char> one((size_t) K * QAGG_PEER_HANDLE_BYTES);
    for (size_t c = 0; c < chunks; ++c)
    {
        for (int p = 0; p < K; ++p) // rank-major input: rank p's handles for chunks 0..chunks-1
            std::memcpy(one.data() + (size_t) p * QAGG_PEER_HANDLE_BYTES,
                        static_cast<const unsigned char*>(handles) + ((size_t) p * chunks + c) * QAGG_PEER_HANDLE_BYTES, QAGG_PEER_HANDLE_BYTES);
        int rc = qagg_agg_enable_peer(h->kids[c], one.data());
        if (rc)
            return rc;
    }
    h->peer = true;
    return QAGG_OK;
}

static int hagg_run(qagg_host_aggregator* h, float* const* host_grads, bool aggregate)
{
    if (!h || !host_grads)
        return fail(QAGG_EINVAL, "qagg_hagg_step: bad arguments");
    int rc = check_cuda(cudaSetDevice(h->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    // Every rank issues the chunks in the same order on its one compute stream, so a flag wait of chunk c only ever waits
    // for kernels that its peers enqueued before their own waits of chunk c.
    const size_t chunks = h->kids.size();
    for (size_t c = 0; c < chunks; ++c)
    {
        const auto& slices = h->chunks[c];
        for (size_t k = 0; k < slices.size(); ++k)
        {
            const int64_t M = h->rows[slices[k].tensor], bytes = M * slices[k].ncols * 4;
            if (bytes && (rc = check_cuda(cudaMemcpyAsync(h->devPtr[c][k], host_grads[slices[k].tensor] + slices[k].col0 * M, (size_t) bytes,
                                                          cudaMemcpyHostToDevice, h->sIn), "gradient upload")))
                return rc;
        }
        if ((rc = check_cuda(cudaEventRecord(h->uploaded[c], h->sIn), "cudaEventRecord")) ||
            (rc = check_cuda(cudaStreamWaitEvent(h->sCompute, h->uploaded[c], 0), "cudaStreamWaitEvent")))
            return rc;
        if (aggregate && (rc = qagg_agg_step(h->kids[c], h->devPtr[c].data(), h->sCompute)))
            return rc;
        if ((rc = check_cuda(cudaEventRecord(h->computed[c], h->sCompute), "cudaEventRecord")) ||
            (rc = check_cuda(cudaStreamWaitEvent(h->sOut, h->computed[c], 0), "cudaStreamWaitEvent")))
            return rc;
        for (size_t k = 0; k < slices.size(); ++k)
        {
            const int64_t M = h->rows[slices[k].tensor], bytes = M * slices[k].ncols * 4;
            if (bytes && (rc = check_cuda(cudaMemcpyAsync(host_grads[slices[k].tensor] + slices[k].col0 * M, h->devPtr[c][k], (size_t) bytes,
                                                          cudaMemcpyDeviceToHost, h->sOut), "gradient download")))
                return rc;
        }
    }
    for (auto st : {h->sIn, h->sCompute, h->sOut})
        if ((rc = check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize")))
            return rc;
    return QAGG_OK;
}

int qagg_hagg_step(qagg_host_aggregator* h, float* const* host_grads)
{
    return hagg_run(h, host_grads, true);
}

int qagg_hagg_copy_only(qagg_host_aggregator* h, float* const* host_grads)
{
    return hagg_run(h, host_grads, false);
}

int qagg_hagg_check(qagg_host_aggregator* h)
{
    if (!h)
        return fail(QAGG_EINVAL, "null host aggregator");
    for (auto* k : h->kids)
    {
        int rc = qagg_agg_check(k, nullptr);
        if (rc)
            return rc;
    }
    return QAGG_OK;
}

int qagg_hagg_destroy(qagg_host_aggregator* h)
{
    delete h;
    return QAGG_OK;
}

int qagg_agg_bind_update(qagg_aggregator* a, float* const* params, float* const* smoothed)
{
    if (!a)
        return fail(QAGG_EINVAL, "qagg_agg_bind_update: null aggregator");
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    if (!params && !smoothed)
    {
        a->updBound = a->updating = false;
        return QAGG_OK;
    }
    if (!params || !smoothed)
        return fail(QAGG_EINVAL, "qagg_agg_bind_update: parameters and smoothed gradients come together");
    if (a->identity)
        return fail(QAGG_ESTATE, "qagg_agg_bind_update: this aggregator leaves the gradients as they are (one worker, identity semantics)");
    std::vector<QTensor> tab(a->hK3);
    for (int i = 0; i < a->T; ++i)
    {
        if (a->M[i] * a->N[i] > 0 && (!params[i] || !smoothed[i]))
            return fail(QAGG_EINVAL, "qagg_agg_bind_update: null matrix pointer");
        if (((uintptr_t) params[i] | (uintptr_t) smoothed[i]) & 3)
            return fail(QAGG_EINVAL, "qagg_agg_bind_update: matrices must be 4-byte aligned");
        tab[i].out = params[i];
        tab[i].res_out = smoothed[i];
    }
    // an earlier step may still be reading the table
    if ((rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize")))
        return rc;
    if (!a->updTable.p && (rc = a->updTable.alloc(tab.size() * sizeof(QTensor), false)))
        return rc;
    if (!tab.empty() && (rc = check_cuda(cudaMemcpy(a->updTable.p, tab.data(), tab.size() * sizeof(QTensor), cudaMemcpyHostToDevice), "table upload")))
        return rc;
    a->updBound = true;
    return QAGG_OK;
}

int qagg_agg_set_update(qagg_aggregator* a, int enabled, float learn_rate_per_sample, float momentum, float unit_gain_factor)
{
    if (!a)
        return fail(QAGG_EINVAL, "qagg_agg_set_update: null aggregator");
    if (!enabled)
    {
        a->updating = false;
        return QAGG_OK;
    }
    if (!a->updBound)
        return fail(QAGG_ESTATE, "qagg_agg_set_update: no parameter matrices bound (qagg_agg_bind_update)");
    if (!(momentum >= 0.0f && momentum <= 1.0f))
        return fail(QAGG_EINVAL, "qagg_agg_set_update: momentum must lie in [0, 1]");
    a->updRule = make_update_rule(learn_rate_per_sample, momentum, unit_gain_factor);
    a->updating = true;
    return QAGG_OK;
}

int qagg_agg_bind_residuals(qagg_aggregator* a, float* const* value_residuals, float* const* stripe_residuals, int keep_plain)
{
    if (!a || (a->T > 0 && (!value_residuals || !stripe_residuals)))
        return fail(QAGG_EINVAL, "qagg_agg_bind_residuals: bad arguments");
    const int r = a->comm->rank, K = a->comm->K;
    for (int i = 0; i < a->T; ++i)
    {
        if (a->M[i] * a->N[i] > 0 && !value_residuals[i])
            return fail(QAGG_EINVAL, "qagg_agg_bind_residuals: null residual buffer");
        if (K > 1 && a->M[i] * a->sN[r][i] > 0 && !stripe_residuals[i])
            return fail(QAGG_EINVAL, "qagg_agg_bind_residuals: null stripe residual buffer for a tensor whose stripe this rank owns");
        if ((reinterpret_cast<uintptr_t>(value_residuals[i]) & 3) || (reinterpret_cast<uintptr_t>(stripe_residuals[i]) & 3))
            return fail(QAGG_EINVAL, "qagg_agg_bind_residuals: buffers must be 4-byte aligned");
    }
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    // no step may still be using the old buffers or tables
    if ((rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize")))
        return rc;
    for (int i = 0; i < a->T; ++i)
    {
        a->res[i] = value_residuals[i];
        a->sres[i] = (K > 1 && a->sN[r][i] > 0) ? stripe_residuals[i] : nullptr;
    }
    a->externalRes = true;
    if (keep_plain)
    {
        a->deferred = false;
        a->deferredOwner = false;
    }
    // the buffers hold plain residuals now: with zero reconstruction values the deferred form means exactly that
    if (a->lvAll.p && (rc = check_cuda(cudaMemset(a->lvAll.p, 0, a->lvAll.bytes), "cudaMemset")))
        return rc;
    if (a->slvAll.p && (rc = check_cuda(cudaMemset(a->slvAll.p, 0, a->slvAll.bytes), "cudaMemset")))
        return rc;
    if ((rc = build_tables(a)))
        return rc;
    a->tableBytes = std::max(a->tableBytes, (size_t) align_up((int64_t) table_bytes(a), 256));
    if (a->tables.bytes < 2 * a->tableBytes)
    {
        cudaFree(a->tables.p);
        a->tables.p = nullptr;
        if ((rc = a->tables.alloc(2 * a->tableBytes, true)))
            return rc;
    }
    for (auto& b : a->bindings)
        b = qagg_aggregator::Binding();
    a->curBinding = 0;
    return QAGG_OK;
}

int qagg_agg_materialize_residuals(qagg_aggregator* a, void* stream)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    cudaStream_t st = (cudaStream_t) stream;
    const int r = a->comm->rank;
    int rc = check_cuda(cudaSetDevice(a->comm->device), "cudaSetDevice");
    if (rc)
        return rc;
    for (int i = 0; i < a->T; ++i)
    {
        if (a->deferred && a->M[i] * a->N[i] > 0)
        {
            if ((rc = check_cuda(launch_materialize(st, a->res[i], a->lv[i], a->res[i], a->M[i], a->N[i], a->cfg.numSMs), "residual export")) ||
                (rc = check_cuda(cudaMemsetAsync(a->lv[i], 0, (size_t) a->N[i] * 8, st), "cudaMemsetAsync")))
                return rc;
        }
        if (a->deferredOwner && a->sres[i] && a->M[i] * a->sN[r][i] > 0)
        {
            if ((rc = check_cuda(launch_materialize(st, a->sres[i], a->slv[i], a->sres[i], a->M[i], a->sN[r][i], a->cfg.numSMs), "residual export")) ||
                (rc = check_cuda(cudaMemsetAsync(a->slv[i], 0, (size_t) a->sN[r][i] * 8, st), "cudaMemsetAsync")))
                return rc;
        }
    }
    return QAGG_OK;
}

int qagg_agg_reset_residuals(qagg_aggregator* a, void* stream)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    cudaStream_t st = (cudaStream_t) stream;
    if (a->externalRes)
    {
        // the caller's buffers, one by one
        const int rr = a->comm->rank;
        int rc = QAGG_OK;
        for (int i = 0; i < a->T && !rc; ++i)
        {
            if (a->M[i] * a->N[i] > 0)
                rc = check_cuda(cudaMemsetAsync(a->res[i], 0, (size_t) (a->M[i] * a->N[i]) * 4, st), "cudaMemsetAsync");
            if (!rc && a->sres[i] && a->M[i] * a->sN[rr][i] > 0)
                rc = check_cuda(cudaMemsetAsync(a->sres[i], 0, (size_t) (a->M[i] * a->sN[rr][i]) * 4, st), "cudaMemsetAsync");
        }
        if (!rc && a->lvAll.p)
            rc = check_cuda(cudaMemsetAsync(a->lvAll.p, 0, a->lvAll.bytes, st), "cudaMemsetAsync");
        if (!rc && a->slvAll.p)
            rc = check_cuda(cudaMemsetAsync(a->slvAll.p, 0, a->slvAll.bytes, st), "cudaMemsetAsync");
        return rc;
    }
    int64_t resFloats = 0, sresFloats = 0;
    const int r = a->comm->rank;
    for (int i = 0; i < a->T; ++i)
    {
        resFloats += align_up(a->M[i] * a->N[i], 4);
        sresFloats += align_up(a->M[i] * a->sN[r][i], 4);
    }
    int rc = check_cuda(cudaMemsetAsync(a->resAll.p, 0, (size_t) std::max<int64_t>(resFloats, 1) * 4, st), "cudaMemsetAsync");
    if (rc)
        return rc;
    if (a->deferred)
    {
        // an all-zero deferred state is a zero residual
        if ((rc = check_cuda(cudaMemsetAsync(a->lvAll.p, 0, a->lvAll.bytes, st), "cudaMemsetAsync")))
            return rc;
        if ((rc = check_cuda(cudaMemsetAsync(a->slvAll.p, 0, a->slvAll.bytes, st), "cudaMemsetAsync")))
            return rc;
    }
    return check_cuda(cudaMemsetAsync(a->sresAll.p, 0, (size_t) std::max<int64_t>(sresFloats, 1) * 4, st), "cudaMemsetAsync");
}

int qagg_agg_residuals(qagg_aggregator* a, int tensor, float** residual, float** stripe_residual)
{
    if (!a || tensor < 0 || tensor >= a->T)
        return fail(QAGG_EINVAL, "qagg_agg_residuals: bad arguments");
    if (a->deferred)
    {
        // turn this tensor's deferred state into plain residuals in place (with zero reconstruction values the state means
        // the same), so that the caller sees residuals; runs on the default stream and waits (first for the last step, which
        // may have been enqueued on a stream that the default stream does not order itself after)
        const int r = a->comm->rank;
        if (a->stepped && a->lastStream != nullptr)
        {
            const int src = check_cuda(cudaStreamSynchronize(a->lastStream), "cudaStreamSynchronize");
            if (src)
                return src;
        }
        int rc = check_cuda(launch_materialize(nullptr, a->res[tensor], a->lv[tensor], a->res[tensor], a->M[tensor], a->N[tensor], a->cfg.numSMs),
                            "residual export");
        if (!rc && a->N[tensor] > 0)
            rc = check_cuda(cudaMemsetAsync(a->lv[tensor], 0, (size_t) a->N[tensor] * 8, nullptr), "cudaMemsetAsync");
        if (!rc && a->sres[tensor] && a->deferredOwner)
        {
            rc = check_cuda(launch_materialize(nullptr, a->sres[tensor], a->slv[tensor], a->sres[tensor], a->M[tensor], a->sN[r][tensor], a->cfg.numSMs),
                            "residual export");
            if (!rc)
                rc = check_cuda(cudaMemsetAsync(a->slv[tensor], 0, (size_t) a->sN[r][tensor] * 8, nullptr), "cudaMemsetAsync");
        }
        if (!rc)
            rc = check_cuda(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
        if (rc)
            return rc;
    }
    if (residual)
        *residual = a->res[tensor];
    if (stripe_residual)
        *stripe_residual = a->sres[tensor];
    return QAGG_OK;
}

int qagg_agg_copy_residual(qagg_aggregator* a, int tensor, int which, float* dst_dev, void* stream)
{
    if (!a || tensor < 0 || tensor >= a->T || !dst_dev || which < 0 || which > 1)
        return fail(QAGG_EINVAL, "qagg_agg_copy_residual: bad arguments");
    const int r = a->comm->rank;
    const float* src = which ? a->sres[tensor] : a->res[tensor];
    const int64_t n = a->M[tensor] * (which ? a->sN[r][tensor] : a->N[tensor]);
    if (n == 0 || !src)
        return QAGG_OK;
    if (which ? a->deferredOwner : a->deferred)
        return check_cuda(launch_materialize((cudaStream_t) stream, src, which ? a->slv[tensor] : a->lv[tensor], dst_dev, a->M[tensor],
                                             which ? a->sN[r][tensor] : a->N[tensor], a->cfg.numSMs), "residual export");
    return check_cuda(cudaMemcpyAsync(dst_dev, src, (size_t) n * 4, cudaMemcpyDeviceToDevice, (cudaStream_t) stream), "residual copy");
}

int qagg_agg_copy_packed(qagg_aggregator* a, int tensor, void* dst_dev, void* stream)
{
    if (!a || tensor < 0 || tensor >= a->T || !dst_dev)
        return fail(QAGG_EINVAL, "qagg_agg_copy_packed: bad arguments");
    const int K = a->comm->K;
    for (int p = 0; p < K; ++p)
    {
        const int64_t bytes = a->sN[p][tensor] * a->colBytes[tensor];
        if (bytes == 0)
            continue;
        int rc = check_cuda(cudaMemcpyAsync(static_cast<unsigned char*>(dst_dev) + a->sStart[p][tensor] * a->colBytes[tensor],
                                            a->gather_slot(p) + a->tOff[p][tensor], (size_t) bytes, cudaMemcpyDeviceToDevice, (cudaStream_t) stream),
                            "packed copy");
        if (rc)
            return rc;
    }
    return QAGG_OK;
}

int64_t qagg_agg_wire_bytes(const qagg_aggregator* a)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    const int K = a->comm->K, r = a->comm->rank;
    int64_t b = 0;
    for (int p = 0; p < K; ++p)
        if (p != r)
            b += a->regionBytes[p] + a->regionBytes[r];
    return b;
}

int qagg_agg_launches_per_step(const qagg_aggregator* a)
{
    if (!a)
        return fail(QAGG_EINVAL, "null aggregator");
    if (a->identity || a->totalValues == 0)
        return 0;
    if (a->comm->K == 1)
        return 2;
    // quantize, owner (one kernel, or form + walk, or both twice when the tall matrices go apart), unquantize; + two flag waits
    // (+ the gather push) (+ a header push when the last step carried a header that the quantize kernel did not take along)
    // in peer mode
    const int tall = a->hK1t.empty() ? 0 : 2 + (a->peer ? 1 : 0) - (a->iK1.empty() ? 1 : 0); // form, walk, flag release; no streaming launch
    return 3 + tall + (a->deferredOwner ? (a->k2SplitOn ? 3 : 1) : 0) +
           (a->peer ? 2 + (a->pushGather ? 1 : 0) + ((a->hdrN > 0 && !header_rides_with_k1(a)) ? 1 : 0) : 0);
}

int qagg_agg_destroy(qagg_aggregator* a)
{
    delete a;
    return QAGG_OK;
}

} // extern "C"
