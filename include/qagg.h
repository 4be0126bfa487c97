/*
 * qagg.h -- C ABI of libqagg: B200 (sm_100a) implementation of CNTK's quantized data-parallel
 * gradient aggregation (1-bit SGD): the 1/2/4/8/16/32-bit column quantizer with error-feedback
 * residual, the packed QuantizedMatrix wire layout, and the striped exchange.
 *
 * Conventions
 *   - Every entry point returns 0 on success and a negative QAGG_E* code on failure; nothing
 *     throws, aborts or exits.  qagg_last_error() returns the calling thread's last message.
 *   - fp32 matrices are column-major, M rows x N columns, element (i, j) at j*M + i, as CNTK's
 *     Matrix<float> (Source/Math/ColumnQuantizer.h:10).
 *   - A packed matrix is N columns of qagg_packed_col_bytes(M, bits) bytes each:
 *         float lower; float upper; uint32 words[Q];   Q = ceil(M*bits/32)
 *     word w holds rows w, w+Q, w+2Q, ...; the k-th of them at bit k*bits
 *     (Source/Math/QuantizedMatrix.h:27-48, Source/Math/ColumnQuantizer.h:50-65).  A column range
 *     [start, start+n) of a packed matrix is the byte range [start*C, (start+n)*C): that is a stripe,
 *     and the wire message.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  Device entry
 *     points only enqueue work; they do not synchronise unless stated.
 *   - Results are bit-identical to the reference CPU quantizer (MatrixQuantizerCPU): per-column sums
 *     are accumulated in row order in fp32 without fused multiply-add.
 *   - There is no CPU fallback: without a CUDA device every compute entry point fails with
 *     QAGG_ECUDA.
 */
#ifndef QAGG_H_
#define QAGG_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QAGG_OK 0
#define QAGG_EINVAL (-1)   /* bad argument (bits not a power of two in 1..32, negative size, null pointer ...) */
#define QAGG_ECUDA (-2)    /* a CUDA runtime call or kernel launch failed */
#define QAGG_ENCCL (-3)    /* an NCCL call failed */
#define QAGG_ESTATE (-4)   /* object used in the wrong state (e.g. mismatched group) */
#define QAGG_ETIMEOUT (-5) /* a bounded device-side wait ran out */

/* flags of qagg_agg_create (defaults of the reference: both set, Source/SGDLib/SGD.cpp:2323-2327,
 * bindings/python/cntk/train/distributed.py:135-140) */
#define QAGG_ZERO_THRESHOLD 1  /* 1-bit: threshold at 0 instead of the column mean (zeroThresholdFor1Bit) */
#define QAGG_SELF_QUANTIZED 2  /* owner starts its aggregate from its own QUANTIZED stripe (useQuantizationForSelfStripe) */
#define QAGG_V2_IDENTITY_K1 4  /* one worker: leave inputs untouched (QuantizedDistributedCommunicator.h:75-81)
                                  instead of V1's quantize -> unquantize round trip */

typedef struct qagg_comm qagg_comm;
typedef struct qagg_aggregator qagg_aggregator;
typedef struct qagg_plan qagg_plan;
typedef struct qagg_host_aggregator qagg_host_aggregator;
typedef struct qagg_dense_aggregator qagg_dense_aggregator;

/* Last error message of the calling thread ("" if none). */
const char* qagg_last_error(void);
/* ABI version of this header (bumped on incompatible change). */
int qagg_abi_version(void);

/* ---- layout helpers ------------------------------------------------------------------------ */

/* QuantizedColumn<float>::QuantizedColumnSize (Source/Math/QuantizedMatrix.h:42-47). <0 on bad args. */
int64_t qagg_packed_col_bytes(int64_t M, int bits);
/* QuantizedMatrix<float>::GetSize (Source/Math/QuantizedMatrix.cpp): N * column size. */
int64_t qagg_packed_bytes(int64_t M, int64_t N, int bits);
/* GetStripeForNode (Source/1BitSGD/AllReduceDistGradAggregator.h:56-65). */
int qagg_stripe(int64_t num_cols, int rank, int num_ranks, int64_t* start_col, int64_t* num_cols_in_stripe);

/* ---- single-matrix quantizer (device buffers) ------------------------------------------------- */

/* MatrixQuantizerImpl<float>::QuantizeAsync (Source/Math/MatrixQuantizerImpl.h:31;
 * GPU body Source/Math/MatrixQuantizerGPU.cu:226-269, kernels Source/Math/MatrixQuantizer_kernel.cu:132-179):
 * per column, range statistics of grad+res_in, quantize, pack, res_out = (grad+res_in) - unquantized.
 * res_in may equal res_out.  All pointers are device pointers; `packed` receives qagg_packed_bytes(). */
int qagg_quantize(void* stream, const float* grad, const float* res_in, float* res_out, void* packed,
                  int64_t M, int64_t N, int bits, int zero_threshold);

/* MatrixQuantizerImpl<float>::UnquantizeAsync (Source/Math/MatrixQuantizerImpl.h:34;
 * Source/Math/MatrixQuantizerGPU.cu:286-334, kernel Source/Math/MatrixQuantizer_kernel.cu:181-202):
 * out = (add ? out : 0) + unquantized(packed). */
int qagg_unquantize(void* stream, const void* packed, float* out, int64_t M, int64_t N, int bits, int add);

/* The stripe owner's work in one pass (Source/1BitSGD/AllReduceDistGradAggregator.h:366-375, 405-435):
 *   agg = self_raw ? self_raw : unquantized(stripes[0]);  agg += unquantized(stripes[s]) for s = 1..K-1 in order;
 *   then quantize agg against the stripe residual into packed_out (same rules as qagg_quantize).
 * `stripes` is a HOST array of K device pointers to packed M x n matrices (stripes[0] may be NULL when
 * self_raw is given).  The fp32 aggregate is never written to memory. */
int qagg_reduce_requantize(void* stream, const void* const* stripes, int K, const float* self_raw,
                           const float* sres_in, float* sres_out, void* packed_out,
                           int64_t M, int64_t n, int bits, int zero_threshold);

/* The same three for ElemType = double (MatrixQuantizerImpl<double>; QWord = unsigned long long, Source/Math/ValueQuantizer.h:48-55):
 * a packed column is `double lower; double upper; uint64 words[Q]`, Q = ceil(M*bits/64), 64 one-bit values per word, bits a
 * power of two in 1..64 (64 = bit-cast pass-through).  Bit-identical to the reference CPU quantizer instantiated for double
 * (what its own 1-bit end-to-end tests run, precision=double).  Buffers must be 8-byte aligned.  The striped aggregator is
 * float only. */
int64_t qagg_packed_col_bytes_f64(int64_t M, int bits);
int64_t qagg_packed_bytes_f64(int64_t M, int64_t N, int bits);
int qagg_quantize_f64(void* stream, const double* grad, const double* res_in, double* res_out, void* packed,
                      int64_t M, int64_t N, int bits, int zero_threshold);
int qagg_unquantize_f64(void* stream, const void* packed, double* out, int64_t M, int64_t N, int bits, int add);

/* The striped aggregation for double gradients: AllReduceDistGradAggregator<double> (Source/1BitSGD/AllReduceDistGradAggregator.h:237-566;
 * the reference's 1-bit end-to-end tests run precision=double), composed from qagg_quantize_f64 / qagg_unquantize_f64 one
 * matrix at a time exactly as the reference composes it from its quantizer; stripes travel by NCCL send/recv (process
 * groups) or device copies (in-process groups, qagg_agg_f64_step_group).  Flags as for qagg_agg_create.  Bit-identical to
 * the CPU checker; one launch per matrix and phase, so it is the functional double path, not a tuned one.  Residuals are
 * plain (never deferred); qagg_agg_f64_residuals hands out the device pointers (stripe pointer for the columns this rank
 * owns, NULL with one rank). */
typedef struct qagg_aggregator_f64 qagg_aggregator_f64;
int qagg_agg_f64_create(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, int bits, int flags, qagg_aggregator_f64** out);
int qagg_agg_f64_step(qagg_aggregator_f64* a, double* const* grads, void* stream);
int qagg_agg_f64_step_group(qagg_aggregator_f64* const* aggs, int num_ranks, double* const* const* grads, void* stream);
int qagg_agg_f64_reset_residuals(qagg_aggregator_f64* a, void* stream);
int qagg_agg_f64_residuals(qagg_aggregator_f64* a, int tensor, double** residual, double** stripe_residual);
/* which: 0 = residual (M x N), 1 = stripe residual (M x owned columns) -> dst (device) */
int qagg_agg_f64_copy_residual(qagg_aggregator_f64* a, int tensor, int which, double* dst, void* stream);
int qagg_agg_f64_destroy(qagg_aggregator_f64* a);

/* Batched qagg_quantize that allocates nothing.  It has no counterpart in the reference.
 * For callers that must not allocate device memory at call time -- a plugin whose host framework owns the rest of the
 * card, a step that cannot afford the device-wide stall of cudaMalloc, a component with a memory budget fixed at start-up.
 * One launch quantizes `num_matrices` matrices (same rules and results as qagg_quantize on each; all arrays are HOST
 * arrays of device pointers / sizes).  The kernel's descriptor tables and work-queue counters live in a fixed 64 KB array
 * inside the library image (every GPU that loads the library holds it until the process exits), hence the limits:
 * at most QAGG_NOALLOC_MAX_MATRICES matrices and QAGG_NOALLOC_MAX_ITEMS work items (groups of adjacent columns; a
 * 2048-row matrix uses one item per 9 columns) per call -- beyond that the call fails with QAGG_EINVAL and launches nothing.
 * The first call on each device also looks up the array's address and clears its counters: make that call before any
 * stream capture.  Every call reuses the same array, so two calls whose kernels may overlap on the GPU race; calls on one
 * stream are ordered and safe.  Calls no cudaMalloc / cudaFree.  The call builds its tables in about 62 KB of the calling
 * thread's stack (mind small thread stacks) and uploads them from there; for that reason a call on a stream that is
 * being captured is refused with QAGG_ESTATE. */
#define QAGG_NOALLOC_MAX_MATRICES 32
#define QAGG_NOALLOC_MAX_ITEMS 4096
int qagg_quantize_batch_noalloc(void* stream, int num_matrices, const float* const* grads, const float* const* res_in,
                                float* const* res_out, void* const* packed, const int64_t* M, const int64_t* N, int bits,
                                int zero_threshold);

/* ---- single-matrix quantizer, packed buffer on the HOST ---------------------------------------- */

/* As the reference's GPU quantizer is driven (packed QuantizedMatrix on the CPU, Source/Math/MatrixQuantizerGPU.cu:243,
 * 260-268, 300-325): device gradient/residual, packed words delivered to / taken from host memory.  `dev_scratch`
 * is a device buffer of qagg_packed_bytes() the caller owns.  Both calls return after the copy has completed. */
int qagg_quantize_to_host(void* stream, const float* grad, const float* res_in, float* res_out, void* dev_scratch,
                          void* host_packed, int64_t M, int64_t N, int bits, int zero_threshold);
int qagg_unquantize_from_host(void* stream, const void* host_packed, void* dev_scratch, float* out,
                              int64_t M, int64_t N, int bits, int add);

/* ---- wire layout (host arithmetic only; needs no device) ------------------------------------------------
 * How one rank of K lays the packed stripes out for the exchange.  "Region p" is the concatenation, tensor after
 * tensor (each block padded to 16 bytes), of the packed stripes that rank p owns: the one message this rank sends to p
 * where the reference posts one MPI_Isend per tensor and peer (Source/1BitSGD/AllReduceDistGradAggregator.h:336-365),
 * and rank p's contribution to the all-gather (:486-502).  The stripe of tensor i inside region p starts at
 * qagg_plan_tensor_offset(p, i) and holds columns GetStripeForNode(N[i], p, K) in the packed column format. */
int qagg_plan_create(int rank, int num_ranks, int num_tensors, const int64_t* M, const int64_t* N, int bits, qagg_plan** out);
int64_t qagg_plan_region_bytes(const qagg_plan* p, int peer);
int64_t qagg_plan_tensor_offset(const qagg_plan* p, int peer, int tensor);
int64_t qagg_plan_gather_slot_bytes(const qagg_plan* p); /* size of one (padded, equal-sized) all-gather slot */
int qagg_plan_destroy(qagg_plan* p);
/* Work items of the streaming quantize kernel (1 bit, threshold 0) for a tensor set, exactly as qagg_agg_create cuts them
 * for a device with `num_sms` SMs; host arithmetic only.  An item is `columns` adjacent columns of one tensor, starting at
 * `first column`; items are listed in queue order (most row chunks first, the last quarter cut into thirds).  Writes
 * min(count, capacity) triples (tensor, first column, columns) to `items` and returns count, or a negative QAGG_E* code.
 * No reference counterpart: the reference launches one kernel per matrix (Source/Math/MatrixQuantizerGPU.cu:226-341). */
int64_t qagg_plan_stream_items(int num_tensors, const int64_t* M, const int64_t* N, int bits, int num_sms, int32_t* items, int64_t capacity);

/* ---- communicator ---------------------------------------------------------------------------------
 * Replaces the MPI point-to-point traffic of the reference (Source/1BitSGD/AllReduceDistGradAggregator.h:303-365,
 * 459-502; Source/Common/Include/MPIWrapper.h:74-177) by NCCL send/recv and all-gather of packed stripes between
 * device buffers; bootstrap as Source/Math/NcclComm.cpp:96-111 (a unique id made on rank 0, distributed by the caller). */

#define QAGG_UNIQUE_ID_BYTES 128
/* Fill `out` (QAGG_UNIQUE_ID_BYTES) with a fresh NCCL unique id; call on one rank, distribute by any means. */
int qagg_unique_id(void* out);
/* One rank of a K-rank group on CUDA device `device`.  K == 1 needs no id (may be NULL) and never touches NCCL. */
int qagg_comm_create(const void* unique_id, int rank, int num_ranks, int device, qagg_comm** out);
/* K ranks living in THIS process on ONE device, exchanging by device-to-device copies: how the reference's own
 * multi-rank GPU tests run (all ranks on GPU 0; Tests/EndToEndTests/Speech/DNN/Parallel1BitQuantization/baseline.gpu.txt).
 * Fills out[0..K-1].  Aggregators built on these must be stepped with qagg_agg_step_group. */
int qagg_comm_create_local_group(int num_ranks, int device, qagg_comm** out);
/* Sum `n` (<= 512) doubles in HOST memory over all ranks, in place, and wait for the result: the DistGradHeader / loss
 * scalars of a step (the reference gathers headers on rank 0 and sends the sum back, AllReduceDistGradAggregator.h:324-333,
 * 380-383, 440-457, 504-514; the V2 path all-reduces them, V2AllReduceDistGradAggregator.h:222-248). */
int qagg_comm_allreduce_f64(qagg_comm* c, double* host_values, int n, void* stream);
/* IDistGradAggregator::WaitAll / DistributedCommunicator::Barrier. */
int qagg_comm_barrier(qagg_comm* c, void* stream);
int qagg_comm_rank(const qagg_comm* c);
int qagg_comm_size(const qagg_comm* c);
int qagg_comm_destroy(qagg_comm* c);

/* ---- aggregator -------------------------------------------------------------------------------------
 * AllReduceDistGradAggregator<float> (Source/1BitSGD/AllReduceDistGradAggregator.h:40-147, 237-566) and
 * QuantizedMPICommunicatorImpl::QuantizedAggregateInPlace (Source/1BitSGD/QuantizedDistributedCommunicator.h:51-61,
 * 285-539).  Owns the residuals (zeroed at creation), the packed send/receive/gather buffers and the stripe
 * residuals for its lifetime; tensor shapes are fixed at creation. */
int qagg_agg_create(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, int bits, int flags,
                    qagg_aggregator** out);
/* The same for tensors that are column slices: tensor i is columns [first_col[i], first_col[i] + N[i]) of a matrix with
 * whole_N[i] columns, and its columns keep the owners GetStripeForNode gives them in the WHOLE matrix -- so aggregating
 * the slices of a matrix separately gives bit-identical results to aggregating it whole (a column's aggregate depends on
 * its owner through the order of the owner's sum).  Both arrays null: whole matrices.  No reference counterpart. */
int qagg_agg_create_slices(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, const int64_t* whole_N, const int64_t* first_col,
                           int bits, int flags, qagg_aggregator** out);
/* One AggregateGradients call: grads[i] (device, M[i] x N[i]) is replaced in place by the aggregate over all ranks.
 * Enqueues on `stream`; returns without waiting.  `grads` is a host array. */
int qagg_agg_step(qagg_aggregator* a, float* const* grads, void* stream);
/* The same for all K aggregators of a local group, in lock step: grads[r][i]. */
int qagg_agg_step_group(qagg_aggregator* const* aggs, int num_ranks, float* const* const* grads, void* stream);
/* One AggregateGradients call INCLUDING its DistGradHeader: besides the gradients, `header` (n <= 64 doubles in host memory:
 * criterion, sample counts, evaluation pairs -- what Source/SGDLib/DistGradHeader.h:5-95 carries, what the V2 path packs into
 * a double vector, Source/1BitSGD/V2AllReduceDistGradAggregator.h:222-248) is summed over all ranks as part of the same
 * enqueued step.  Where the reference gathers headers on rank 0 and sends the sum back with four more MPI messages per rank
 * (AllReduceDistGradAggregator.h:324-333, 380-383, 440-457, 504-514), the peer-memory path stores the header into every
 * peer's window ahead of the quantize kernel, whose flag release publishes it with the packed stripes; after the first flag
 * wait a one-block kernel adds the K headers in rank order (the same order on every rank).  The NCCL path all-reduces it.
 * The call copies `header` before it returns.  qagg_agg_header_result waits for `stream` and returns the sum. */
int qagg_agg_step_header(qagg_aggregator* a, float* const* grads, const double* header, int n, void* stream);
int qagg_agg_step_group_header(qagg_aggregator* const* aggs, int num_ranks, float* const* const* grads, const double* const* headers, int n,
                               void* stream);
int qagg_agg_header_result(qagg_aggregator* a, double* out, int n, void* stream);
/* The same through HOST gradient buffers (pinned memory recommended): copies host_grads[i] to the device, aggregates,
 * copies the result back into host_grads[i], and waits for completion. */
int qagg_agg_step_host(qagg_aggregator* a, float* const* host_grads, void* stream);
/* ResetResidue on both quantizer sets (AllReduceDistGradAggregator.h:121-136; also what V2's CreateCheckpoint does,
 * Source/1BitSGD/QuantizedDataParallelDistributedLearner.h:73-91). */
int qagg_agg_reset_residuals(qagg_aggregator* a, void* stream);
/* Caller-owned residuals, as the V2 interface has them (valueQuantizationResidues / stripeQuantizationResidues of
 * QuantizedDistributedCommunicator::QuantizedAggregate, Source/CNTKv2LibraryDll/API/CNTKLibrary.h:6246-6259; the reference
 * creates them on first use, Source/1BitSGD/QuantizedDistributedCommunicator.h:246-261, and the learner owns and zeroes them,
 * Source/1BitSGD/QuantizedDataParallelDistributedLearner.h:56-60, 73-91).  value_residuals[i] is an M[i] x N[i] device
 * buffer, stripe_residuals[i] an M[i] x n buffer for the n columns of tensor i that this rank owns (ignored, may be NULL,
 * where n == 0 or with one rank).  From this call on the aggregator keeps its error-feedback state in these buffers
 * instead of its own; their CONTENT AT THE TIME OF THE CALL is taken as plain residuals.
 *   keep_plain != 0: the buffers hold plain residuals after every step (resident-column kernels; slower).
 *   keep_plain == 0: for 1 bit with threshold 0 the buffers hold the DEFERRED form between steps (the value that was
 *     quantized; the column's two reconstruction values stay inside the aggregator, see qagg_agg_residuals).  Before reading
 *     them call qagg_agg_materialize_residuals (turns them into plain residuals in place, on `stream`); after writing them
 *     from outside (e.g. zeroing them for a checkpoint) call qagg_agg_bind_residuals again, or use
 *     qagg_agg_reset_residuals, which zeroes bound buffers too.
 * Synchronises the device.  No reference counterpart as a function: the reference passes the buffers on every call. */
int qagg_agg_bind_residuals(qagg_aggregator* a, float* const* value_residuals, float* const* stripe_residuals, int keep_plain);
int qagg_agg_materialize_residuals(qagg_aggregator* a, void* stream);
/* ---- consumer fusion: the learner's momentum-SGD step taken straight from the packed aggregate ---------------------------
 * The training loops update the parameters right after aggregation (V1: SGD<ElemType>::UpdateWeights,
 * Source/SGDLib/SGD.cpp:1405-1457, 2509-2527; V2: m_learner->Update in
 * Source/1BitSGD/QuantizedDataParallelDistributedLearner.h:69 -> LearnerMomentumSGD::Update,
 * Source/CNTKv2LibraryDll/Learner.cpp:610-645).  Both end in Matrix<ElemType>::MomentumSGDUpdate
 * (Source/Math/Matrix.cpp:1681-1698):
 *     smoothed = ScaleAndAdd(unit_gain_factor * learn_rate_per_sample, gradient, momentum, smoothed);  param -= smoothed
 * with ScaleAndAdd's three forms for momentum == 1, == 0 and otherwise (Matrix.cpp:5415-5429; the last one is
 * (smoothed + (alpha / momentum) * gradient) * momentum).  The multiply-add, a BLAS axpy in the reference, is ONE fused
 * multiply-add here.  Not covered: clipping, L1/L2 regularisation, update noise, Nesterov, AdaGrad and its relatives.
 *
 * qagg_sgd_update: that step over n values of a gradient held in device memory.
 * qagg_unquantize_sgd: the same with the gradient taken from a packed matrix as it is expanded (never written).
 * qagg_agg_bind_update + qagg_agg_set_update: make the aggregator's last kernel do it.  params[i] and smoothed[i] are
 *   M[i] x N[i] device matrices.  While enabled, every qagg_agg_step* variant ends by updating them with the aggregated
 *   gradient INSTEAD of writing it: the gradient buffers keep what the caller put there.  The three scalars are those of the
 *   step that follows; a caller whose momentum depends on the aggregated sample count of the very same step (the header sum)
 *   must know that count beforehand (fixed minibatch size) or use the unfused calls for that step.  bind_update
 *   synchronises the device; passing two NULLs unbinds.  Refused (QAGG_ESTATE) for an aggregator created with
 *   QAGG_V2_IDENTITY_K1 on one rank, which leaves gradients untouched. */
int qagg_sgd_update(void* stream, float* params, const float* grads, float* smoothed, int64_t n, float learn_rate_per_sample, float momentum,
                    float unit_gain_factor);
int qagg_unquantize_sgd(void* stream, const void* packed, float* params, float* smoothed, int64_t M, int64_t N, int bits, float learn_rate_per_sample,
                        float momentum, float unit_gain_factor);
int qagg_agg_bind_update(qagg_aggregator* a, float* const* params, float* const* smoothed);
int qagg_agg_set_update(qagg_aggregator* a, int enabled, float learn_rate_per_sample, float momentum, float unit_gain_factor);
/* Device pointers to internal state, for inspection: the M x N residual and the M x n stripe residual of tensor i
 * (stripe pointer NULL when this rank owns no column of it).  For 1 bit with threshold 0 the aggregator keeps the
 * residual in a deferred form (the quantized value plus the column's two reconstruction values; the subtraction is done
 * when the state is next read -- the same arithmetic as the reference's, later); this call first turns tensor i's state
 * into plain residuals in place, on the default stream, and waits for that. */
int qagg_agg_residuals(qagg_aggregator* a, int tensor, float** residual, float** stripe_residual);
/* Copy the residual (which = 0, M x N floats) or the stripe residual (which = 1, M x n floats) of tensor i into a
 * device buffer, on `stream`: always plain residuals, bit-identical to the reference's GetResidualMatrix. */
int qagg_agg_copy_residual(qagg_aggregator* a, int tensor, int which, float* dst_dev, void* stream);
/* Copy the gathered packed matrix of tensor i (what every rank unquantized from in the last step) into a device
 * buffer of qagg_packed_bytes(M[i], N[i], bits), in the reference's contiguous layout. */
int qagg_agg_copy_packed(qagg_aggregator* a, int tensor, void* dst_dev, void* stream);
/* ---- aggregation from host buffers, software-pipelined ---------------------------------------------------------------
 * For gradients that live in (pinned) host memory -- the situation of the reference's CPU-device runs and of its GPU runs'
 * packed buffers, which always cross PCIe (Source/Math/MatrixQuantizerGPU.cu:126-142, 313-324).  The gradient set is cut
 * into `num_chunks` chunks of about equal bytes -- small tensors grouped, large ones cut by columns, every column keeping
 * the owner it has in its whole tensor (qagg_agg_create_slices) -- and the chunks go through a three-stage pipeline (an
 * upload stream, a compute stream, a download stream, linked by events), so that the upload of one chunk, the kernels of
 * another and the download of a third overlap and the upload engine never waits behind a download.
 * qagg_hagg_step returns when all results are back in host_grads.  Residuals live inside the object.
 * Peer mode: qagg_hagg_peer_handles writes chunks * QAGG_PEER_HANDLE_BYTES bytes; qagg_hagg_enable_peer takes the
 * handles of all ranks, rank-major (K * chunks * QAGG_PEER_HANDLE_BYTES bytes).  Every rank runs the chunks' kernels in
 * the same order on one stream (which is also what one NCCL communicator needs without peer mode). */
int qagg_hagg_create(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, int bits, int flags, int num_chunks,
                     qagg_host_aggregator** out);
int qagg_hagg_chunks(const qagg_host_aggregator* h);
int qagg_hagg_peer_handles(qagg_host_aggregator* h, void* out);
int qagg_hagg_enable_peer(qagg_host_aggregator* h, const void* handles);
int qagg_hagg_step(qagg_host_aggregator* h, float* const* host_grads);
/* The uploads and downloads of qagg_hagg_step without the kernels between them: the copy floor of this machine for the
 * same chunking (measurement aid; host_grads come back unchanged). */
int qagg_hagg_copy_only(qagg_host_aggregator* h, float* const* host_grads);
int qagg_hagg_check(qagg_host_aggregator* h);
int qagg_hagg_destroy(qagg_host_aggregator* h);

/* ---- unquantized aggregation (gradientBits = 32) ---------------------------------------------------------------------
 * SimpleDistGradAggregator (Source/SGDLib/SimpleDistGradAggregator.h:262-485) / MPICommunicatorImpl::AggregateImpl
 * (Source/CNTKv2LibraryDll/DistributedCommunicator.cpp:311-492): grads[i] is replaced in place by the fp32 sum over all
 * ranks.  Where the reference packs the tensors below its threshold into one buffer (:327-361) and all-reduces buffers and
 * large tensors with MPI or NCCL, all tensors are laid end to end here, cut into K equal slices, and moved by three kernels
 * over peer-mapped windows (scatter to the slice's owner, sum at the owner IN RANK ORDER, gather from the owner): the
 * result is the same on every rank and every run.  qagg_dense_peer_handle / _enable_peer work like the quantized
 * aggregator's; without them more than one rank falls back to one ncclAllReduce of the flat buffer (summation order:
 * NCCL's).  The reference's optional fp16 wire format (useFP16AllReduce, :411-429) is not built.  One rank: no-op. */
int qagg_dense_create(qagg_comm* comm, int num_tensors, const int64_t* M, const int64_t* N, qagg_dense_aggregator** out);
int qagg_dense_step(qagg_dense_aggregator* a, float* const* grads, void* stream);
int qagg_dense_step_group(qagg_dense_aggregator* const* aggs, int num_ranks, float* const* const* grads, void* stream);
int qagg_dense_peer_handle(qagg_dense_aggregator* a, void* out);
int qagg_dense_enable_peer(qagg_dense_aggregator* a, const void* handles);
/* useFP16AllReduce (Source/CNTKv2LibraryDll/DistributedCommunicator.cpp:411-429; SGD.cpp:3327-3329): the gradients are cast
 * to half (round to nearest), exchanged and summed as halves, and cast back -- half the wire bytes.  On the peer-memory path
 * the sum runs in ascending rank order, each addition taken in fp32 and rounded to half; on the NCCL path the order and the
 * intermediate precision are NCCL's.  Takes effect from the next step. */
int qagg_dense_set_fp16(qagg_dense_aggregator* a, int enabled);
int qagg_dense_check(qagg_dense_aggregator* a, void* stream);
int64_t qagg_dense_wire_bytes(const qagg_dense_aggregator* a);
int qagg_dense_destroy(qagg_dense_aggregator* a);

/* ---- peer-memory exchange (optional; replaces the two NCCL collectives of a step) ------------------------------------
 * Where the reference moves every stripe GPU -> pinned host -> MPI -> pinned host -> GPU (Source/Math/MatrixQuantizerGPU.cu:126-142,
 * 313-324; Source/1BitSGD/AllReduceDistGradAggregator.h:303-365, 459-502), the quantize kernel here stores each packed
 * column straight into its owner's receive slot and the owner's requantize kernel stores its result straight into every
 * rank's gather slot, over NVLink peer mappings; a step's two "collectives" shrink to two flag hand-shakes.
 *   1. every rank calls qagg_agg_peer_handle (QAGG_PEER_HANDLE_BYTES bytes out) and the caller all-gathers the handles;
 *   2. every rank calls qagg_agg_enable_peer with the K handles in rank order (cudaIpcOpenMemHandle on the others').
 * From then on qagg_agg_step uses the peer path.  Device-side waits are bounded (qagg_agg_set_wait_limit polls, default
 * about two seconds): a peer that never arrives makes the wait give up and set a status word instead of hanging;
 * qagg_agg_check synchronises the stream and returns QAGG_ETIMEOUT if that happened since creation -- or if a bounded
 * wait inside the streaming quantize kernel (for a copy into shared memory) ever ran out. */
#define QAGG_PEER_HANDLE_BYTES 64
int qagg_agg_peer_handle(qagg_aggregator* a, void* out);
int qagg_agg_enable_peer(qagg_aggregator* a, const void* handles);
int qagg_agg_set_wait_limit(qagg_aggregator* a, long long max_polls);
int qagg_agg_check(qagg_aggregator* a, void* stream);
/* The time-out report is sticky: once set, every later qagg_agg_check repeats it.  After the cause has been dealt with
 * (the missing peer is back and every rank agrees to go on) this call clears it; waits for `stream`.  The results of the
 * step that timed out stay invalid, and so does the residual state it wrote: reset the residuals as well.
 * Streams: an aggregator's steps may be enqueued on any stream, one step at a time; calls that rewrite what an enqueued
 * step reads (a step with new gradient pointers, qagg_agg_residuals) wait for the stream of the last step themselves. */
int qagg_agg_clear_status(qagg_aggregator* a, void* stream);
/* Failure detection of the streaming quantize kernel, exercised without a fault: one warp runs the kernel's own bounded
 * wait on an mbarrier phase that nothing will ever complete.  After `max_tries` polls the wait gives up, ORs 2 into
 * *status_dev and the kernel ends normally; a second wait in the same kernel returns at once.  cycles_dev (2 x int64,
 * may be NULL) receives the clock cycles each wait took.  No reference counterpart. */
int qagg_stream_wait_selftest(void* stream, int max_tries, unsigned* status_dev, long long* cycles_dev);
/* The bounded wait on its own: one warp polls flags_dev[i] (i < n <= 32, i != skip) until each is >= value or max_polls
 * polls have passed; on give-up it ORs 1 into *status_dev.  Never hangs. */
int qagg_wait_flags(void* stream, const unsigned* flags_dev, int n, int skip, unsigned value, long long max_polls, unsigned* status_dev);

/* Per-phase device timing of the steps that follow (no reference counterpart; the reference only has the wall-clock
 * "Actual gradient aggregation time" trace, AllReduceDistGradAggregator.h:241-246, 560-565).  When enabled, each step records
 * CUDA events on its stream around its five phases.  qagg_agg_phase_ms waits for the recorded steps and returns the mean
 * milliseconds per step, over the (at most 64) most recent steps since the last read, for
 * {quantize, scatter, reduce-requantize, all-gather, unquantize} (about 0 for phases a 1-rank step skips). */
int qagg_agg_set_profiling(qagg_aggregator* a, int enabled);
int qagg_agg_phase_ms(qagg_aggregator* a, float* out5);
/* Bytes one step sends over the wire from this rank (scatter + gather), and kernels it launches. */
int64_t qagg_agg_wire_bytes(const qagg_aggregator* a);
int qagg_agg_launches_per_step(const qagg_aggregator* a);
int qagg_agg_destroy(qagg_aggregator* a);

#ifdef __cplusplus
}
#endif
#endif /* QAGG_H_ */
