// qagg_internal.h -- structures shared by the kernels, the single-matrix C entry points and the aggregator.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <utility>
#include <vector>

#define QAGG_MAXK 16 // most ranks in one group (one 8-GPU box needs 8)
#define QAGG_COUNTER_UINTS 272

namespace qagg {

// Everything the column kernels need to know about one matrix.  Used for
//   - the pre-aggregation quantize   (source = grad + residual, all N columns, packed column j routed to its owner),
//   - the owner's reduce-requantize  (source = sum of `nsrc` packed stripes (+ raw own stripe) + stripe residual),
//   - the final unquantize           (packed column j fetched from its owner's gather slot).
struct QTensor
{
    const float* grad;   // quantize: gradient, M x N.  reduce: raw own stripe (M x N) or nullptr.  unquantize: unused
    const float* res_in; // residual read
    float* res_out;      // residual written (may equal res_in)
    float* out;          // unquantize: destination, M x N
    long long M, N;      // rows, columns handled by this descriptor
    int Q;               // 32-bit words per packed column = ceil(M * bits / 32)
    int colBytes;        // 8 + 4 * Q
    int bits;
    int K;               // owners the packed columns are routed over (1 = one contiguous packed matrix)
    long long per, rem;  // (columns of the whole matrix) / K and % K: owner p holds columns [p*per + min(p, rem), ...)
                         // (GetStripeForNode)
    long long col0;      // this descriptor covers columns [col0, col0 + N) of the whole matrix (0 unless it is a column slice)
    unsigned char* pk[QAGG_MAXK]; // packed base for owner p; its first column is that owner's stripe start
    int nsrc;                           // reduce: number of packed sources
    int selfRaw;                        // reduce: 1 = start from `grad` instead of src[0]
    const unsigned char* src[QAGG_MAXK]; // reduce: packed sources, M x N each, summed in index order
    int bcast;                           // 1 = every packed column is also written to the launch's broadcast bases
    int pad_;
    long long bcastOff;                  // offset of this matrix's block from a broadcast base (K == 1 routing only)
    float* lv;                           // streaming kernel only: the two reconstruction values of each column's previous
                                         // quantization (2 floats per column), read at the start and rewritten at the end
    // streaming kernel only: tensor maps (device addresses of 128-byte CUtensorMap objects) through which the chunk tiles of
    // `grad` ([g][0]) and `res_in` ([g][1]) are fetched, for two tile geometries: items of up to boxCols[0] columns and
    // items of up to boxCols[1] < boxCols[0] columns (0: no such items).  All null: the matrix is fetched with plain loads.
    const void* tm[2][2];
    int boxCols[2];
    long long unit0; // unquantize and owner-form kernels: number of work units of the table entries before this one
    unsigned* stats; // owner kernels only: two words per column (rows with a set bit, NaN seen), zero between steps
};

// What the unquantize kernel does with a value it has expanded.
constexpr int UNQ_STORE = 0;  // out = value
constexpr int UNQ_ADD = 1;    // out += value
constexpr int UNQ_UPDATE = 2; // momentum-SGD step on (parameter, smoothed gradient) with the value as the gradient

// The momentum-SGD update of Matrix<ElemType>::MomentumSGDUpdate (Source/Math/Matrix.cpp:1681-1698): the smoothed gradient
// becomes ScaleAndAdd(alpha, gradient, momentum, smoothed) with alpha = unitGainFactor * learnRatePerSample, then the
// parameter loses the smoothed gradient.  ScaleAndAdd with a weight on the destination (Matrix.cpp:5415-5429) has three
// forms, chosen on the host:
//   kind 0 (momentum == 1): smoothed += alpha * g                       a = alpha
//   kind 1 (momentum == 0): smoothed  = alpha * g                       a = alpha
//   kind 2 (otherwise)    : smoothed  = (smoothed + (alpha / momentum) * g) * momentum     a = alpha / momentum
// The reference hands the multiply-add to a BLAS axpy; it is taken as ONE fused multiply-add here (what cuBLAS and the
// vector units of current CPUs do), and the scaling as one multiplication.
struct UpdateRule
{
    float a;
    float beta;
    int kind;
};
UpdateRule make_update_rule(float learnRatePerSample, float momentum, float unitGainFactor);
// plain update kernel over n values (qagg_update.cu): the same arithmetic from a gradient held in memory
cudaError_t launch_sgd_update(cudaStream_t st, float* params, const float* grads, float* smoothed, long long n, const UpdateRule& rule, int numSMs);

// Flags that the last CTA of a kernel writes (release, system scope) after all of the kernel's stores: one word in each
// peer's memory, set to `value`.  n == 0: no signalling.
struct Signal
{
    unsigned* flag[QAGG_MAXK];
    int n;
    unsigned value;
    unsigned char* bcastBase[QAGG_MAXK]; // broadcast copies (peer gather slots) for matrices with bcast == 1
    int nbcast;
    // header values that ride with the kernel (streaming quantize kernel only): its first CTA copies hdrN doubles from hdrIn
    // (pinned host memory) into every hdrDst[p] (this rank's header slot in each rank's window) before the flags are released
    const double* hdrIn;
    double* hdrDst[QAGG_MAXK];
    int hdrN, hdrDstN;
};

// header exchange: up to QAGG_HEADER_MAX doubles per rank (DistGradHeader needs 3 + 2 per evaluation node)
#define QAGG_HEADER_MAX 64
struct HeaderPtrs
{
    double* p[QAGG_MAXK];
    int n;
};

struct QItem
{
    int tensor;
    int col0;
    int ncols;
};

enum QuantMode
{
    MODE_ONEBIT_ZERO = 0, // 1 bit, threshold 0, separate level means
    MODE_ONEBIT_MEAN = 1, // 1 bit, threshold = column mean
    MODE_MULTIBIT = 2     // 2..32 bits, range = +-4 sigma
};

// shared-memory row stride (in floats) of one staged column: >= M, multiple of 4, == 4 mod 32 so that
// 128-bit reads of the same rows of neighbouring columns fall into distinct banks
__host__ __device__ inline int smem_stride(long long M)
{
    long long s = (M + 3) & ~3LL;
    s += (36 - (s & 31)) & 31;
    return (int) s;
}

struct LaunchCfg
{
    int numSMs = 0;
    int smemFloats = 0;  // dynamic shared memory per CTA, in floats
    int ctasPerSM = 0;
};

// cols per work item for a matrix of M rows under a given shared-memory budget; *resident tells whether whole
// columns fit (else the kernel streams the column through shared memory in chunks and reads its inputs twice)
// extraFloatsPerCol: further shared memory a column needs (the reduce kernel stages its K packed source columns:
// K * colBytes / 4)
int cols_per_item(long long M, long long N, int smemFloats, bool* resident, int extraFloatsPerCol = 0);

// launchers (qagg_kernels.cu).  `single` != nullptr: one matrix described by value, items derived from the block index.
// otherwise `tensors`/`items` are device tables.
// `counters` (optional, QAGG_COUNTER_UINTS zero-initialised uints in device memory, private to one kernel in flight)
// switches the kernel from static striding over the items to a shared work queue: [0] next item, [1] CTAs finished
// (both re-zeroed by the kernel before it ends), [8 + smid] per-SM tickets that spread the walking warps.
cudaError_t launch_colquant(cudaStream_t st, bool stripes, int mode, const QTensor* single, const QTensor* tensors,
                            const QItem* items, int nItems, int colsPerItem, const LaunchCfg& cfg, unsigned* counters = nullptr,
                            const Signal* signal = nullptr);
// copies `bytes` (rounded up to 16) from local `src` to the same offset of every signal.bcastBase[], then releases signal.flag[]
cudaError_t launch_push(cudaStream_t st, const void* src, size_t bytes, const Signal& signal, unsigned* counters, int numSMs);
// one warp polls flags[i] (i < n, i != skip) until each is >= value (wrap-safe) or maxPolls polls have passed; on
// give-up it ORs 1 into *status and returns: the context stays usable and the host reads the status later
// hdrSrc (optional): once the flags are in, the hdrN doubles behind each hdrSrc->p[] are added in index order into hdrOut
cudaError_t launch_wait_flags(cudaStream_t st, const unsigned* flags, int n, int skip, unsigned value, long long maxPolls, unsigned* status,
                              const HeaderPtrs* hdrSrc = nullptr, int hdrN = 0, double* hdrOut = nullptr);
// unquantize (qagg_unquantize.cu): `single` != nullptr: one matrix described by value; otherwise `tensors` is a device table
// of nTensors entries (all of `bits` bits) whose unit0 fields are the running sums of unq_units() (entry order = unit order)
// smemWordsPerWarp: the largest unq_smem_words() over the matrices of the launch (0: none of them takes the row-major form)
// mode: UNQ_STORE, UNQ_ADD, or UNQ_UPDATE (needs `rule`; each entry's `out` is then the parameter matrix and `res_out` the
// smoothed gradient, both M x N)
cudaError_t launch_unquantize(cudaStream_t st, int mode, int bits, const QTensor* single, const QTensor* tensors, int nTensors,
                              long long totalUnits, int smemWordsPerWarp, const LaunchCfg& cfg, const UpdateRule* rule = nullptr);
long long unq_units(long long M, long long N, int bits); // work units of an M x N matrix in the unquantize kernel
int unq_smem_words(long long M, int bits);               // shared-memory words per warp an M-row matrix needs there
// header exchange kernels (qagg_kernels.cu): in[0..n) -> dst.p[*][0..n);  out[i] = src.p[0][i] + src.p[1][i] + ... in that order
cudaError_t launch_header_push(cudaStream_t st, const double* in, int n, const HeaderPtrs& dst);
cudaError_t launch_header_sum(cudaStream_t st, const HeaderPtrs& src, int n, double* out);
cudaError_t get_launch_cfg(int device, LaunchCfg* cfg);
// releases the flags of `signal` from a one-thread kernel (a rank with nothing to compute still has to tell its peers)
cudaError_t launch_signal_only(cudaStream_t st, const Signal& signal);

// ---- streaming kernel for 1 bit with threshold 0 (qagg_stream.cu) --------------------------------------------------
// It keeps the error-feedback state of a matrix in DEFERRED form: the buffer holds v (the value that was quantized:
// gradient + residual) and `lv` holds each column's two reconstruction values; the residual proper,
// v - (v >= 0 ? lv[1] : lv[0]), is formed with the same single subtraction when the state is next read.  All-zero
// buffers are a zero residual.  Columns stream through shared memory in row chunks, so column height is limited only
// by the shared-memory copy of a work item's packed words: nc * Q <= QAGG_STREAM_PKWORDS.
#define QAGG_STREAM_PKWORDS 2560
#define QAGG_STREAM_CMAX 32
// most columns per work item for columns of Q packed words (0: the column is too tall for this kernel)
inline int stream_max_cols(long long Q)
{
    if (Q <= 0)
        return QAGG_STREAM_CMAX;
    const long long c = QAGG_STREAM_PKWORDS / Q;
    return (int) (c > QAGG_STREAM_CMAX ? QAGG_STREAM_CMAX : c);
}
// Work items of one launch of the streaming kernel, in queue order.  shapes[t] = (rows, columns) of table entry t.
// Items are sized for about (all values) / (2 x resident CTAs) values each, ordered longest first; the items in the last
// quarter of the queue are cut into three, so that the launch ends with short items and all CTAs finish together.
// boxCols[t] = {columns of a full item, columns of a cut item or 0} for matrix t.
void stream_make_items(const std::vector<std::pair<long long, long long>>& shapes, int numSMs, int bits, std::vector<QItem>& out,
                       std::vector<std::pair<int, int>>& boxCols);
// Encodes the tensor maps of one streaming descriptor whose grad / res_in / res_out / M / N / selfRaw / boxCols are set:
// writes up to four maps to hostMaps (512 bytes, to be copied to devMaps, 128-byte aligned) and sets t->tm[][] to their
// device addresses -- or to null if the matrix cannot be fetched through tensor maps (rows not a multiple of 4, or
// buffers not 16-byte aligned), in which case the kernel uses plain loads for it.
void stream_set_maps(QTensor* t, unsigned char* hostMaps, unsigned char* devMaps);
// 128-byte tensor map of a column-major M x N fp32 matrix with a box of boxRows rows x boxCols columns (each <= 256), looked
// up through the runtime's driver entry point; false if it cannot be encoded (rows not a multiple of 4, base not 16-byte
// aligned, driver too old)
bool encode_map_2d(void* out128, const float* base, long long M, long long N, int boxRows, int boxCols);
#define QAGG_STREAM_MAP_BYTES 512
// always table-driven with a work queue (`counters` as for launch_colquant, required).  The kernel's waits for copies in
// flight are bounded: if one runs out, bit 1 of *status is set and the kernel ends normally (results invalid)
cudaError_t launch_stream1(cudaStream_t st, const QTensor* tensors, const QItem* items, int nItems, const LaunchCfg& cfg, unsigned* counters,
                           const Signal* signal = nullptr, unsigned* status = nullptr);

// ---- the owner's reduce-requantize for 1 bit with threshold 0, two kernels (qagg_owner.cu) -------------------------------
// Table entries describe the owned stripes: src[] / nsrc / selfRaw / grad (raw own stripe), res_in == res_out (stripe
// residual in deferred form), lv, stats, pk[0] (this rank's gather slot), bcast / bcastOff, unit0 = running sum of
// owner_form_units(), tm[0][1] = tensor map of res_out made by owner_set_map (null: plain loads).
long long owner_form_units(long long M, long long n);
// walk items (32 adjacent columns of one entry), tallest columns first; shapes[e] = (rows, owned columns) of entry e
void owner_make_items(const std::vector<std::pair<long long, long long>>& shapes, std::vector<QItem>& out);
bool owner_set_map(QTensor* t, unsigned char* hostMap, unsigned char* devMap);
// form kernel, then walk kernel; the walk kernel's last CTA releases signal.flag[] (`counters` as for launch_colquant; only
// [1] is used).  Its waits for tiles in flight are bounded like the streaming kernel's (bit 1 of *status).
// `split` (optional): the table's first entries are "tall" matrices -- tallUnits form units, tallItems walk items -- whose
// walk runs on the stream `side` (ordered by the events `fork` and `join`) while the other matrices are formed and walked on
// `st`; on return `st` is ordered after everything.  counters[1..3] are used.
struct OwnerSplit
{
    long long tallUnits;
    int tallItems;
    cudaStream_t side;
    cudaEvent_t fork, join;
};
cudaError_t launch_owner(cudaStream_t st, const QTensor* tensors, int nTensors, long long formUnits, const QItem* items, int nItems,
                         const LaunchCfg& cfg, unsigned* counters, const Signal* signal = nullptr, unsigned* status = nullptr,
                         const OwnerSplit* split = nullptr, cudaEvent_t afterForm = nullptr);
// (afterForm: recorded on `st` between the form and the walk launch of the unsplit sequence)
// runs the streaming kernel's bounded mbarrier wait on a barrier that nothing completes (see qagg_stream_wait_selftest)
cudaError_t launch_stream_wait_selftest(cudaStream_t st, int maxTries, unsigned* status, long long* cycles);
// dst[i, j] = buf[i, j] - (buf[i, j] >= 0 ? lv[2j + 1] : lv[2j]): the residual proper of a deferred state (dst may be buf)
cudaError_t launch_materialize(cudaStream_t st, const float* buf, const float* lv, float* dst, long long M, long long N, int numSMs);

// error plumbing (qagg_capi.cu)
int fail(int code, const std::string& msg);
int check_cuda(cudaError_t e, const char* what);
bool bits_ok(int bits);
int mode_of(int bits, int zeroThr);
void fill_layout(QTensor* t, long long M, long long N, int bits);
int launch_cfg_for_current_device(LaunchCfg* cfg); // per-device launch configuration, looked up once
int check_dims(long long M, long long N, int bits); // shape and bit-width limits of the single-matrix entry points

} // namespace qagg
