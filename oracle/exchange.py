"""CPU restatement of CNTK's striped quantized gradient exchange (TEST INFRASTRUCTURE ONLY).

Follows AllReduceDistGradAggregator<float>::AggregateGradientsImpl
(Source/1BitSGD/AllReduceDistGradAggregator.h:237-566) and the V2 twin
QuantizedMPICommunicatorImpl::QuantizedAggregate<float>
(Source/1BitSGD/QuantizedDistributedCommunicator.h:285-539) step by step, with the K MPI
ranks simulated in one process and the MPI messages replaced by array copies.  The
arithmetic of every quantize / unquantize call is done by a backend from
``oracle.backend`` (the reference's own headers when ``RefBackend`` is used).

Parity status: the reference has no test that pins the exchange numerically (only
training-loss tolerances), and its owner adds received stripes in MPI arrival order
(:389-421), which is not deterministic for K >= 3.  This restatement fixes the order to
"own stripe first, then sources by ascending rank"; that choice is the pin.

Arrays: an fp32 M x N column-major matrix is a C-contiguous numpy array of shape (N, M),
so a column stripe [start, start+n) is the row slice ``a[start:start+n]``.
"""
import numpy as np


def stripe(num_cols, rank, K):
    """GetStripeForNode (AllReduceDistGradAggregator.h:56-65): (start column, number of columns)."""
    per, rem = divmod(num_cols, K)
    return per * rank + min(rem, rank), per + (1 if rank < rem else 0)


class ExchangeState:
    """Per-rank persistent state: the pre-aggregation residual (M x N) and the stripe residual
    (M x n_rank) of every tensor, zero-initialised (1BitSGD/MatrixQuantizer.h:27-30;
    AllReduceDistGradAggregator.h:87, :97)."""

    def __init__(self, shapes, K, dtype=np.float32):
        self.shapes = [tuple(s) for s in shapes]  # (M, N) per tensor
        self.K = K
        self.dtype = dtype  # np.float64 with the double checkers (ElemType = double)
        self.res = [[np.zeros((N, M), dtype) for (M, N) in self.shapes] for _ in range(K)]
        self.sres = [[np.zeros((stripe(N, r, K)[1], M), dtype) for (M, N) in self.shapes] for r in range(K)]

    def reset(self):
        """ResetResidue on every quantizer (AllReduceDistGradAggregator.h:121-136)."""
        for per_rank in self.res + self.sres:
            for a in per_rank:
                a[...] = 0


def _each_rank(executor, fn, K):
    """Run fn(r) for every simulated rank: serially, or on `executor` threads (one per rank, as the reference runs one
    single-threaded quantizer per MPI rank; the C checkers release the GIL while they compute)."""
    if executor is None:
        for r in range(K):
            fn(r)
    else:
        for f in [executor.submit(fn, r) for r in range(K)]:
            f.result()


def aggregate_step(backend, state, grads, bits, zero_thr=True, self_quant=True, v2_identity_at_k1=False, executor=None):
    """One AggregateGradients call on all K simulated ranks.

    ``grads[r][i]`` is rank r's (N_i, M_i) float32 gradient; it is overwritten with the aggregate,
    as the reference does (gradients are aggregated in place, :281, :521).
    Returns ``packed[r][i]``: the fully gathered packed matrix each rank unquantized from
    (identical on all ranks), for wire-format comparison.
    """
    K, shapes = state.K, state.shapes
    T = len(shapes)
    if K == 1 and v2_identity_at_k1:
        # QuantizedDistributedCommunicator.h:75-81: a single worker returns its inputs untouched.
        return None
    col_bytes = [backend.packed_col_bytes(M, bits) for (M, N) in shapes]

    # step 1 (:290-300): every rank quantizes every gradient against its own residual, in place.
    packed = [[np.zeros(shapes[i][1] * col_bytes[i], np.uint8) for i in range(T)] for _ in range(K)]

    def quantize_all(r):
        for i in range(T):
            backend.quantize(grads[r][i], state.res[r][i], state.res[r][i], packed[r][i], bits, zero_thr)

    _each_rank(executor, quantize_all, K)

    if K == 1:
        # V1 with one rank: the own stripe is unquantized into the gradient (:366-375); no stripe is ever
        # received, so the requantization at :429-435 never fires; the final unquantize (:516-522) rewrites
        # the gradient from the same packed data.
        for i in range(T):
            backend.unquantize(packed[0][i], grads[0][i], bits, add=False)
        return packed

    # steps 2-5: the owner of each stripe builds the aggregate inside its own gradient slice and requantizes.
    agg_packed = [[None] * T for _ in range(K)]

    def own_stripes(r):
        for i in range(T):
            M, N = shapes[i]
            s, n = stripe(N, r, K)
            if n == 0:
                continue
            C = col_bytes[i]
            agg = grads[r][i][s:s + n]  # ColumnSlice view of the gradient (:281)
            if self_quant:
                backend.unquantize(packed[r][i][s * C:(s + n) * C], agg, bits, add=False)  # :366-375
            for src in range(K):  # fixed order: ascending source rank (reference: arrival order, :389-421)
                if src == r:
                    continue
                backend.unquantize(packed[src][i][s * C:(s + n) * C], agg, bits, add=True)  # :421
            out = np.zeros(n * C, np.uint8)
            backend.quantize(agg, state.sres[r][i], state.sres[r][i], out, bits, zero_thr)  # :429-435
            agg_packed[r][i] = out

    _each_rank(executor, own_stripes, K)

    # steps 7-9 (:459-522): all-gather of the requantized stripes, then every rank unquantizes everything.
    gathered = []
    for i in range(T):
        M, N = shapes[i]
        C = col_bytes[i]
        full = np.zeros(N * C, np.uint8)
        for r in range(K):
            s, n = stripe(N, r, K)
            if n:
                full[s * C:(s + n) * C] = agg_packed[r][i]
        gathered.append(full)
    def unquantize_all(r):
        for i in range(T):
            backend.unquantize(gathered[i], grads[r][i], bits, add=False)

    _each_rank(executor, unquantize_all, K)
    return [gathered for _ in range(K)]


def owner_of(col, num_cols, K):
    """Rank whose stripe (GetStripeForNode) holds column `col` of a matrix with `num_cols` columns."""
    per, rem = divmod(num_cols, K)
    big = (per + 1) * rem
    if col < big:
        return col // (per + 1)
    return rem + (col - big) // per


def aggregate_columns(backend, owner, g, res, sres, bits, zero_thr=True, self_quant=True):
    """The exchange restricted to a set of columns that share one owner rank.

    A column's aggregate depends on that column alone -- its K gradients, its K pre-aggregation residuals and its
    owner's stripe residual -- and on who owns it only through the order of the owner's sum (own stripe first, then the
    sources by ascending rank).  So the steps of ``aggregate_step`` can be replayed for any sample of columns of a
    full-size tensor.

    g[r], res[r]: (n, M) float32 per rank r (n sampled columns); res[r] is updated in place to the new residual.
    sres: (n, M) float32, the owner's stripe residual of these columns, updated in place.
    Returns (out, packed): the aggregate every rank ends with, (n, M) float32, and the n requantized packed columns.
    With K == 1 this is V1's quantize -> unquantize round trip (no stripe requantization, :429 never fires).
    """
    K = len(g)
    n, M = g[0].shape
    C = backend.packed_col_bytes(M, bits)
    packed = []
    for r in range(K):
        p = np.zeros(n * C, np.uint8)
        backend.quantize(np.ascontiguousarray(g[r]), res[r], res[r], p, bits, zero_thr)
        packed.append(p)
    out = np.zeros((n, M), np.float32)
    if K == 1:
        backend.unquantize(packed[0], out, bits, add=False)
        return out, packed[0]
    if self_quant:
        agg = np.zeros((n, M), np.float32)
        backend.unquantize(packed[owner], agg, bits, add=False)
    else:
        agg = np.ascontiguousarray(g[owner]).copy()
    for src in range(K):
        if src != owner:
            backend.unquantize(packed[src], agg, bits, add=True)
    requant = np.zeros(n * C, np.uint8)
    backend.quantize(agg, sres, sres, requant, bits, zero_thr)
    backend.unquantize(requant, out, bits, add=False)
    return out, requant


def dense_sum(grads):
    """The unquantized arm (gradientBits = 32): the fp32 sum over the ranks, added in ascending rank order with one rounding
    per addition.  The reference leaves the order to its MPI / NCCL all-reduce (SimpleDistGradAggregator.h:262-485), so it
    has no bit-level contract; the fixed order is the pin.  grads[r][i]: rank r's tensor i; returns the list of sums."""
    out = []
    for i in range(len(grads[0])):
        acc = grads[0][i].astype(np.float32, copy=True)
        for r in range(1, len(grads)):
            acc = (acc + grads[r][i]).astype(np.float32)
        out.append(acc)
    return out


def dense_sum_fp16(grads):
    """useFP16AllReduce (Source/CNTKv2LibraryDll/DistributedCommunicator.cpp:411-429): every rank's tensor is cast to half,
    the halves are added in ascending rank order (each sum taken in fp32 and rounded to half), and the result is cast back
    to fp32.  The reference leaves the order and the intermediate precision to MPI / NCCL; this fixes them."""
    K = len(grads)
    out = []
    for i in range(len(grads[0])):
        acc = grads[0][i].astype(np.float16)
        for r in range(1, K):
            acc = (acc.astype(np.float32) + grads[r][i].astype(np.float16).astype(np.float32)).astype(np.float16)
        out.append(acc.astype(np.float32))
    return out
