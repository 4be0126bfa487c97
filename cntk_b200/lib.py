"""ctypes bindings of libqagg.so (see include/qagg.h for the contract of every call).

Device buffers are passed as integers (``tensor.data_ptr()``); torch is used by callers only to own device
memory and streams.  Every wrapper raises ``QaggError`` with the library's message on a non-zero status.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libqagg.so")

ZERO_THRESHOLD = 1
SELF_QUANTIZED = 2
V2_IDENTITY_K1 = 4
UNIQUE_ID_BYTES = 128
PEER_HANDLE_BYTES = 64

EXPORTS = [
    "qagg_last_error", "qagg_abi_version", "qagg_packed_col_bytes", "qagg_packed_bytes", "qagg_stripe",
    "qagg_quantize", "qagg_unquantize", "qagg_reduce_requantize", "qagg_quantize_batch_noalloc", "qagg_quantize_to_host", "qagg_unquantize_from_host",
    "qagg_plan_create", "qagg_plan_stream_items", "qagg_stream_wait_selftest", "qagg_plan_region_bytes", "qagg_plan_tensor_offset", "qagg_plan_gather_slot_bytes", "qagg_plan_destroy",
    "qagg_unique_id", "qagg_comm_create", "qagg_comm_create_local_group", "qagg_comm_allreduce_f64", "qagg_comm_barrier", "qagg_comm_rank", "qagg_comm_size",
    "qagg_comm_destroy", "qagg_agg_create", "qagg_agg_step", "qagg_agg_step_group", "qagg_agg_step_host",
    "qagg_agg_reset_residuals", "qagg_agg_residuals", "qagg_agg_copy_residual", "qagg_agg_copy_packed", "qagg_agg_wire_bytes",
    "qagg_agg_launches_per_step", "qagg_agg_peer_handle", "qagg_agg_enable_peer", "qagg_agg_set_wait_limit", "qagg_agg_check", "qagg_wait_flags",
    "qagg_hagg_create", "qagg_hagg_chunks", "qagg_hagg_peer_handles", "qagg_hagg_enable_peer", "qagg_hagg_step", "qagg_hagg_check",
    "qagg_hagg_destroy", "qagg_agg_set_profiling", "qagg_agg_phase_ms", "qagg_agg_destroy",
    "qagg_agg_step_header", "qagg_agg_step_group_header", "qagg_agg_header_result", "qagg_agg_create_slices", "qagg_hagg_copy_only",
    "qagg_dense_create", "qagg_dense_step", "qagg_dense_step_group", "qagg_dense_peer_handle", "qagg_dense_enable_peer", "qagg_dense_check",
    "qagg_dense_wire_bytes", "qagg_dense_destroy", "qagg_agg_bind_residuals", "qagg_agg_materialize_residuals",
    "qagg_packed_col_bytes_f64", "qagg_packed_bytes_f64", "qagg_quantize_f64", "qagg_unquantize_f64",
    "qagg_sgd_update", "qagg_unquantize_sgd", "qagg_agg_bind_update", "qagg_agg_set_update", "qagg_agg_clear_status",
    "qagg_agg_f64_create", "qagg_agg_f64_step", "qagg_agg_f64_step_group", "qagg_agg_f64_reset_residuals", "qagg_agg_f64_residuals",
    "qagg_agg_f64_destroy", "qagg_agg_f64_copy_residual", "qagg_dense_set_fp16",
]


class QaggError(RuntimeError):
    pass


if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `python -m cntk_b200.build` (there is no CPU fallback)")

_lib = ctypes.CDLL(LIB_PATH)
c_i64, c_int, c_vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p

_lib.qagg_last_error.restype = ctypes.c_char_p
_lib.qagg_packed_col_bytes.restype = c_i64
_lib.qagg_packed_col_bytes.argtypes = [c_i64, c_int]
_lib.qagg_packed_bytes.restype = c_i64
_lib.qagg_packed_bytes.argtypes = [c_i64, c_i64, c_int]
_lib.qagg_stripe.argtypes = [c_i64, c_int, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64)]
_lib.qagg_quantize.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_int]
_lib.qagg_unquantize.argtypes = [c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_int]
_lib.qagg_packed_col_bytes_f64.restype = c_i64
_lib.qagg_packed_col_bytes_f64.argtypes = [c_i64, c_int]
_lib.qagg_packed_bytes_f64.restype = c_i64
_lib.qagg_packed_bytes_f64.argtypes = [c_i64, c_i64, c_int]
_lib.qagg_quantize_f64.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_int]
_lib.qagg_unquantize_f64.argtypes = [c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_int]
_lib.qagg_reduce_requantize.argtypes = [c_vp, ctypes.POINTER(c_vp), c_int, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_int]
_lib.qagg_quantize_batch_noalloc.argtypes = [c_vp, c_int, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), ctypes.POINTER(c_vp),
                                             ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), c_int, c_int]
_lib.qagg_quantize_to_host.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_int]
_lib.qagg_unquantize_from_host.argtypes = [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_int]
_lib.qagg_plan_create.argtypes = [c_int, c_int, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), c_int, ctypes.POINTER(c_vp)]
_lib.qagg_plan_region_bytes.restype = c_i64
_lib.qagg_plan_region_bytes.argtypes = [c_vp, c_int]
_lib.qagg_plan_tensor_offset.restype = c_i64
_lib.qagg_plan_tensor_offset.argtypes = [c_vp, c_int, c_int]
_lib.qagg_plan_gather_slot_bytes.restype = c_i64
_lib.qagg_plan_gather_slot_bytes.argtypes = [c_vp]
_lib.qagg_plan_destroy.argtypes = [c_vp]
_lib.qagg_stream_wait_selftest.argtypes = [c_vp, c_int, c_vp, c_vp]
_lib.qagg_plan_stream_items.restype = c_i64
_lib.qagg_plan_stream_items.argtypes = [c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), c_int, c_int, ctypes.POINTER(ctypes.c_int32), c_i64]
_lib.qagg_unique_id.argtypes = [c_vp]
_lib.qagg_comm_create.argtypes = [c_vp, c_int, c_int, c_int, ctypes.POINTER(c_vp)]
_lib.qagg_comm_create_local_group.argtypes = [c_int, c_int, ctypes.POINTER(c_vp)]
_lib.qagg_comm_allreduce_f64.argtypes = [c_vp, ctypes.POINTER(ctypes.c_double), c_int, c_vp]
_lib.qagg_comm_barrier.argtypes = [c_vp, c_vp]
_lib.qagg_comm_rank.argtypes = [c_vp]
_lib.qagg_comm_size.argtypes = [c_vp]
_lib.qagg_comm_destroy.argtypes = [c_vp]
_lib.qagg_agg_create.argtypes = [c_vp, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), c_int, c_int, ctypes.POINTER(c_vp)]
_lib.qagg_agg_step.argtypes = [c_vp, ctypes.POINTER(c_vp), c_vp]
_lib.qagg_agg_step_group.argtypes = [ctypes.POINTER(c_vp), c_int, ctypes.POINTER(ctypes.POINTER(c_vp)), c_vp]
_lib.qagg_agg_step_header.argtypes = [c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(ctypes.c_double), c_int, c_vp]
_lib.qagg_agg_step_group_header.argtypes = [ctypes.POINTER(c_vp), c_int, ctypes.POINTER(ctypes.POINTER(c_vp)), ctypes.POINTER(ctypes.POINTER(ctypes.c_double)), c_int, c_vp]
_lib.qagg_agg_header_result.argtypes = [c_vp, ctypes.POINTER(ctypes.c_double), c_int, c_vp]
_lib.qagg_agg_step_host.argtypes = [c_vp, ctypes.POINTER(c_vp), c_vp]
_lib.qagg_agg_reset_residuals.argtypes = [c_vp, c_vp]
_lib.qagg_sgd_update.argtypes = [c_vp, c_vp, c_vp, c_vp, c_i64, ctypes.c_float, ctypes.c_float, ctypes.c_float]
_lib.qagg_unquantize_sgd.argtypes = [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, ctypes.c_float, ctypes.c_float, ctypes.c_float]
_lib.qagg_agg_clear_status.argtypes = [c_vp, c_vp]
_lib.qagg_agg_f64_create.argtypes = [c_vp, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), c_int, c_int, ctypes.POINTER(c_vp)]
_lib.qagg_agg_f64_step.argtypes = [c_vp, ctypes.POINTER(c_vp), c_vp]
_lib.qagg_agg_f64_step_group.argtypes = [ctypes.POINTER(c_vp), c_int, ctypes.POINTER(ctypes.POINTER(c_vp)), c_vp]
_lib.qagg_agg_f64_reset_residuals.argtypes = [c_vp, c_vp]
_lib.qagg_agg_f64_residuals.argtypes = [c_vp, c_int, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp)]
_lib.qagg_agg_f64_destroy.argtypes = [c_vp]
_lib.qagg_dense_set_fp16.argtypes = [c_vp, c_int]
_lib.qagg_agg_f64_copy_residual.argtypes = [c_vp, c_int, c_int, c_vp, c_vp]
_lib.qagg_agg_bind_update.argtypes = [c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp)]
_lib.qagg_agg_set_update.argtypes = [c_vp, c_int, ctypes.c_float, ctypes.c_float, ctypes.c_float]
_lib.qagg_agg_bind_residuals.argtypes = [c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), c_int]
_lib.qagg_agg_materialize_residuals.argtypes = [c_vp, c_vp]
_lib.qagg_agg_residuals.argtypes = [c_vp, c_int, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp)]
_lib.qagg_agg_copy_residual.argtypes = [c_vp, c_int, c_int, c_vp, c_vp]
_lib.qagg_agg_copy_packed.argtypes = [c_vp, c_int, c_vp, c_vp]
_lib.qagg_agg_wire_bytes.restype = c_i64
_lib.qagg_agg_wire_bytes.argtypes = [c_vp]
_lib.qagg_agg_launches_per_step.argtypes = [c_vp]
_lib.qagg_agg_peer_handle.argtypes = [c_vp, c_vp]
_lib.qagg_agg_enable_peer.argtypes = [c_vp, c_vp]
_lib.qagg_agg_set_wait_limit.argtypes = [c_vp, ctypes.c_longlong]
_lib.qagg_agg_check.argtypes = [c_vp, c_vp]
_lib.qagg_wait_flags.argtypes = [c_vp, c_vp, c_int, c_int, ctypes.c_uint, ctypes.c_longlong, c_vp]
_lib.qagg_hagg_create.argtypes = [c_vp, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), c_int, c_int, c_int, ctypes.POINTER(c_vp)]
_lib.qagg_hagg_chunks.argtypes = [c_vp]
_lib.qagg_hagg_peer_handles.argtypes = [c_vp, c_vp]
_lib.qagg_hagg_enable_peer.argtypes = [c_vp, c_vp]
_lib.qagg_hagg_step.argtypes = [c_vp, ctypes.POINTER(c_vp)]
_lib.qagg_hagg_copy_only.argtypes = [c_vp, ctypes.POINTER(c_vp)]
_lib.qagg_agg_create_slices.argtypes = [c_vp, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), c_int, c_int,
                                        ctypes.POINTER(c_vp)]
_lib.qagg_hagg_check.argtypes = [c_vp]
_lib.qagg_dense_create.argtypes = [c_vp, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), ctypes.POINTER(c_vp)]
_lib.qagg_dense_step.argtypes = [c_vp, ctypes.POINTER(c_vp), c_vp]
_lib.qagg_dense_step_group.argtypes = [ctypes.POINTER(c_vp), c_int, ctypes.POINTER(ctypes.POINTER(c_vp)), c_vp]
_lib.qagg_dense_peer_handle.argtypes = [c_vp, c_vp]
_lib.qagg_dense_enable_peer.argtypes = [c_vp, c_vp]
_lib.qagg_dense_check.argtypes = [c_vp, c_vp]
_lib.qagg_dense_wire_bytes.restype = c_i64
_lib.qagg_dense_wire_bytes.argtypes = [c_vp]
_lib.qagg_dense_destroy.argtypes = [c_vp]
_lib.qagg_hagg_destroy.argtypes = [c_vp]
_lib.qagg_agg_set_profiling.argtypes = [c_vp, c_int]
_lib.qagg_agg_phase_ms.argtypes = [c_vp, ctypes.POINTER(ctypes.c_float)]
_lib.qagg_agg_destroy.argtypes = [c_vp]


def raw():
    """The ctypes handle itself (for symbol checks)."""
    return _lib


def last_error():
    return _lib.qagg_last_error().decode()


def _ok(rc):
    if rc != 0:
        raise QaggError(f"qagg error {rc}: {last_error()}")


def packed_col_bytes(M, bits):
    v = _lib.qagg_packed_col_bytes(M, bits)
    if v < 0:
        _ok(int(v))
    return int(v)


def packed_bytes(M, N, bits):
    v = _lib.qagg_packed_bytes(M, N, bits)
    if v < 0:
        _ok(int(v))
    return int(v)


def stripe(num_cols, rank, K):
    s, n = c_i64(), c_i64()
    _ok(_lib.qagg_stripe(num_cols, rank, K, ctypes.byref(s), ctypes.byref(n)))
    return int(s.value), int(n.value)


def quantize(grad_ptr, res_in_ptr, res_out_ptr, packed_ptr, M, N, bits, zero_thr=True, stream=0):
    _ok(_lib.qagg_quantize(stream, grad_ptr, res_in_ptr, res_out_ptr, packed_ptr, M, N, bits, int(bool(zero_thr))))


def unquantize(packed_ptr, out_ptr, M, N, bits, add=False, stream=0):
    _ok(_lib.qagg_unquantize(stream, packed_ptr, out_ptr, M, N, bits, int(bool(add))))


def packed_bytes_f64(M, N, bits):
    v = _lib.qagg_packed_bytes_f64(M, N, bits)
    if v < 0:
        _ok(int(v))
    return int(v)


def quantize_f64(grad_ptr, res_in_ptr, res_out_ptr, packed_ptr, M, N, bits, zero_thr=True, stream=0):
    _ok(_lib.qagg_quantize_f64(stream, grad_ptr, res_in_ptr, res_out_ptr, packed_ptr, M, N, bits, int(bool(zero_thr))))


def unquantize_f64(packed_ptr, out_ptr, M, N, bits, add=False, stream=0):
    _ok(_lib.qagg_unquantize_f64(stream, packed_ptr, out_ptr, M, N, bits, int(bool(add))))


def sgd_update(params_ptr, grads_ptr, smoothed_ptr, n, learn_rate, momentum, unit_gain, stream=0):
    """Momentum-SGD step over n values (Matrix::MomentumSGDUpdate, Source/Math/Matrix.cpp:1681-1698)."""
    _ok(_lib.qagg_sgd_update(stream, params_ptr, grads_ptr, smoothed_ptr, n, learn_rate, momentum, unit_gain))


def unquantize_sgd(packed_ptr, params_ptr, smoothed_ptr, M, N, bits, learn_rate, momentum, unit_gain, stream=0):
    """The same step with the gradient taken from a packed matrix as it is expanded."""
    _ok(_lib.qagg_unquantize_sgd(stream, packed_ptr, params_ptr, smoothed_ptr, M, N, bits, learn_rate, momentum, unit_gain))


def reduce_requantize(stripe_ptrs, self_raw_ptr, sres_in_ptr, sres_out_ptr, packed_out_ptr, M, n, bits, zero_thr=True, stream=0):
    K = len(stripe_ptrs)
    arr = (c_vp * K)(*[c_vp(p) if p else c_vp(None) for p in stripe_ptrs])
    _ok(_lib.qagg_reduce_requantize(stream, arr, K, self_raw_ptr, sres_in_ptr, sres_out_ptr, packed_out_ptr, M, n, bits,
                                    int(bool(zero_thr))))


def quantize_batch_noalloc(grad_ptrs, res_in_ptrs, res_out_ptrs, packed_ptrs, shapes, bits, zero_thr=True, stream=0):
    """qagg_quantize_batch_noalloc: one launch over several matrices, scratch in the library's fixed array (no allocation)."""
    n = len(shapes)
    arr = lambda ps: (c_vp * n)(*[c_vp(p) for p in ps])
    Ms = (c_i64 * n)(*[s[0] for s in shapes])
    Ns = (c_i64 * n)(*[s[1] for s in shapes])
    _ok(_lib.qagg_quantize_batch_noalloc(stream, n, arr(grad_ptrs), arr(res_in_ptrs), arr(res_out_ptrs), arr(packed_ptrs), Ms, Ns, bits,
                                         int(bool(zero_thr))))


def quantize_to_host(grad_ptr, res_in_ptr, res_out_ptr, dev_scratch_ptr, host_packed_ptr, M, N, bits, zero_thr=True, stream=0):
    _ok(_lib.qagg_quantize_to_host(stream, grad_ptr, res_in_ptr, res_out_ptr, dev_scratch_ptr, host_packed_ptr, M, N, bits,
                                   int(bool(zero_thr))))


def unquantize_from_host(host_packed_ptr, dev_scratch_ptr, out_ptr, M, N, bits, add=False, stream=0):
    _ok(_lib.qagg_unquantize_from_host(stream, host_packed_ptr, dev_scratch_ptr, out_ptr, M, N, bits, int(bool(add))))


class Plan:
    """Host-only wire layout of rank `rank` of K (qagg_plan_*)."""

    def __init__(self, rank, K, shapes, bits):
        T = len(shapes)
        Ms = (c_i64 * T)(*[s[0] for s in shapes])
        Ns = (c_i64 * T)(*[s[1] for s in shapes])
        h = c_vp()
        _ok(_lib.qagg_plan_create(rank, K, T, Ms, Ns, bits, ctypes.byref(h)))
        self.h, self.rank, self.K, self.shapes, self.bits = h, rank, K, [tuple(s) for s in shapes], bits

    def region_bytes(self, peer):
        v = int(_lib.qagg_plan_region_bytes(self.h, peer))
        if v < 0:
            _ok(v)
        return v

    def tensor_offset(self, peer, tensor):
        v = int(_lib.qagg_plan_tensor_offset(self.h, peer, tensor))
        if v < 0:
            _ok(v)
        return v

    @property
    def gather_slot_bytes(self):
        return int(_lib.qagg_plan_gather_slot_bytes(self.h))

    def destroy(self):
        if self.h:
            _lib.qagg_plan_destroy(self.h)
            self.h = None


def stream_items(shapes, bits=1, num_sms=148):
    """Work items of the streaming quantize kernel for a tensor set: list of (tensor, first column, columns) in queue
    order (qagg_plan_stream_items; host arithmetic only)."""
    T = len(shapes)
    Ms = (c_i64 * T)(*[s[0] for s in shapes])
    Ns = (c_i64 * T)(*[s[1] for s in shapes])
    n = int(_lib.qagg_plan_stream_items(T, Ms, Ns, bits, num_sms, None, 0))
    if n < 0:
        _ok(n)
    buf = (ctypes.c_int32 * (3 * max(n, 1)))()
    n2 = int(_lib.qagg_plan_stream_items(T, Ms, Ns, bits, num_sms, buf, n))
    if n2 < 0:
        _ok(n2)
    return [(buf[3 * k], buf[3 * k + 1], buf[3 * k + 2]) for k in range(n)]


def stream_wait_selftest(max_tries, status_ptr, cycles_ptr=0, stream=0):
    _ok(_lib.qagg_stream_wait_selftest(stream, max_tries, status_ptr, cycles_ptr))


def wait_flags(flags_ptr, n, skip, value, max_polls, status_ptr, stream=0):
    _ok(_lib.qagg_wait_flags(stream, flags_ptr, n, skip, value, max_polls, status_ptr))


def unique_id():
    buf = ctypes.create_string_buffer(UNIQUE_ID_BYTES)
    _ok(_lib.qagg_unique_id(buf))
    return buf.raw


class Comm:
    def __init__(self, handle):
        self.h = handle

    @staticmethod
    def create(unique_id_bytes, rank, K, device):
        h = c_vp()
        buf = ctypes.create_string_buffer(unique_id_bytes, UNIQUE_ID_BYTES) if unique_id_bytes else None
        _ok(_lib.qagg_comm_create(buf, rank, K, device, ctypes.byref(h)))
        return Comm(h)

    @staticmethod
    def local_group(K, device):
        arr = (c_vp * K)()
        _ok(_lib.qagg_comm_create_local_group(K, device, arr))
        return [Comm(c_vp(arr[i])) for i in range(K)]

    def allreduce_f64(self, values, stream=0):
        arr = (ctypes.c_double * len(values))(*values)
        _ok(_lib.qagg_comm_allreduce_f64(self.h, arr, len(values), stream))
        return list(arr)

    def barrier(self, stream=0):
        _ok(_lib.qagg_comm_barrier(self.h, stream))

    @property
    def rank(self):
        return _lib.qagg_comm_rank(self.h)

    @property
    def size(self):
        return _lib.qagg_comm_size(self.h)

    def destroy(self):
        if self.h:
            _ok(_lib.qagg_comm_destroy(self.h))
            self.h = None


class Aggregator:
    """qagg_aggregator handle.  ``shapes`` is a list of (M, N)."""

    def __init__(self, comm, shapes, bits, flags=ZERO_THRESHOLD | SELF_QUANTIZED, whole_cols=None, first_cols=None):
        """whole_cols / first_cols: tensor i is columns [first_cols[i], first_cols[i] + N) of a matrix of whole_cols[i] columns."""
        self.comm, self.shapes, self.bits, self.flags = comm, [tuple(s) for s in shapes], bits, flags
        T = len(shapes)
        Ms = (c_i64 * T)(*[s[0] for s in shapes])
        Ns = (c_i64 * T)(*[s[1] for s in shapes])
        h = c_vp()
        if whole_cols is None:
            _ok(_lib.qagg_agg_create(comm.h, T, Ms, Ns, bits, flags, ctypes.byref(h)))
        else:
            _ok(_lib.qagg_agg_create_slices(comm.h, T, Ms, Ns, (c_i64 * T)(*whole_cols), (c_i64 * T)(*first_cols), bits, flags, ctypes.byref(h)))
        self.h = h

    def _ptrs(self, ptrs):
        return (c_vp * len(ptrs))(*[c_vp(p) for p in ptrs])

    def step(self, grad_ptrs, stream=0):
        _ok(_lib.qagg_agg_step(self.h, self._ptrs(grad_ptrs), stream))

    def step_header(self, grad_ptrs, header, stream=0):
        """One step that also sums `header` (a list of floats) over the ranks; fetch the sum with header_result()."""
        arr = (ctypes.c_double * len(header))(*header)
        _ok(_lib.qagg_agg_step_header(self.h, self._ptrs(grad_ptrs), arr, len(header), stream))

    def header_result(self, n, stream=0):
        out = (ctypes.c_double * max(n, 1))()
        _ok(_lib.qagg_agg_header_result(self.h, out, n, stream))
        return [float(out[i]) for i in range(n)]

    def step_host(self, host_grad_ptrs, stream=0):
        _ok(_lib.qagg_agg_step_host(self.h, self._ptrs(host_grad_ptrs), stream))

    def bind_residuals(self, value_ptrs, stripe_ptrs, keep_plain=False):
        """Caller-owned residual buffers (device pointers; stripe pointer 0 where this rank owns no column)."""
        _ok(_lib.qagg_agg_bind_residuals(self.h, self._ptrs(value_ptrs), (c_vp * len(stripe_ptrs))(*[c_vp(p) if p else c_vp(None) for p in stripe_ptrs]),
                                         int(bool(keep_plain))))

    def clear_status(self, stream=0):
        _ok(_lib.qagg_agg_clear_status(self.h, stream))

    def bind_update(self, param_ptrs, smoothed_ptrs):
        """Parameter and smoothed-gradient matrices for the fused learner step (None, None unbinds)."""
        if param_ptrs is None and smoothed_ptrs is None:
            _ok(_lib.qagg_agg_bind_update(self.h, None, None))
        else:
            _ok(_lib.qagg_agg_bind_update(self.h, self._ptrs(param_ptrs), self._ptrs(smoothed_ptrs)))

    def set_update(self, enabled, learn_rate=0.0, momentum=0.0, unit_gain=1.0):
        """While enabled, every step ends in the momentum-SGD update of the bound matrices instead of writing gradients."""
        _ok(_lib.qagg_agg_set_update(self.h, int(bool(enabled)), learn_rate, momentum, unit_gain))

    def materialize_residuals(self, stream=0):
        _ok(_lib.qagg_agg_materialize_residuals(self.h, stream))

    def reset_residuals(self, stream=0):
        _ok(_lib.qagg_agg_reset_residuals(self.h, stream))

    def residual_ptrs(self, tensor):
        r, s = c_vp(), c_vp()
        _ok(_lib.qagg_agg_residuals(self.h, tensor, ctypes.byref(r), ctypes.byref(s)))
        return r.value, s.value

    def copy_residual(self, tensor, which, dst_ptr, stream=0):
        _ok(_lib.qagg_agg_copy_residual(self.h, tensor, which, dst_ptr, stream))

    def copy_packed(self, tensor, dst_ptr, stream=0):
        _ok(_lib.qagg_agg_copy_packed(self.h, tensor, dst_ptr, stream))

    def peer_handle(self):
        buf = ctypes.create_string_buffer(PEER_HANDLE_BYTES)
        _ok(_lib.qagg_agg_peer_handle(self.h, buf))
        return buf.raw

    def enable_peer(self, handles):
        """handles: the K peer handles (bytes), in rank order."""
        blob = b"".join(handles)
        assert len(blob) == PEER_HANDLE_BYTES * len(handles)
        _ok(_lib.qagg_agg_enable_peer(self.h, ctypes.create_string_buffer(blob, len(blob))))

    def set_wait_limit(self, max_polls):
        _ok(_lib.qagg_agg_set_wait_limit(self.h, max_polls))

    def check(self, stream=0):
        _ok(_lib.qagg_agg_check(self.h, stream))

    def set_profiling(self, enabled):
        _ok(_lib.qagg_agg_set_profiling(self.h, int(bool(enabled))))

    def phase_ms(self):
        """[quantize, scatter, reduce-requantize, all-gather, unquantize] device milliseconds of the last profiled step."""
        out = (ctypes.c_float * 5)()
        _ok(_lib.qagg_agg_phase_ms(self.h, out))
        return [float(x) for x in out]

    @property
    def wire_bytes(self):
        return int(_lib.qagg_agg_wire_bytes(self.h))

    @property
    def launches_per_step(self):
        return int(_lib.qagg_agg_launches_per_step(self.h))

    def destroy(self):
        if self.h:
            _ok(_lib.qagg_agg_destroy(self.h))
            self.h = None


class DenseAggregator:
    """qagg_dense_aggregator: unquantized fp32 sum over the ranks (gradientBits = 32)."""

    def __init__(self, comm, shapes):
        T = len(shapes)
        Ms = (c_i64 * T)(*[s[0] for s in shapes])
        Ns = (c_i64 * T)(*[s[1] for s in shapes])
        h = c_vp()
        _ok(_lib.qagg_dense_create(comm.h, T, Ms, Ns, ctypes.byref(h)))
        self.h = h

    def set_fp16(self, enabled):
        _ok(_lib.qagg_dense_set_fp16(self.h, int(bool(enabled))))

    def step(self, grad_ptrs, stream=0):
        _ok(_lib.qagg_dense_step(self.h, (c_vp * len(grad_ptrs))(*[c_vp(p) for p in grad_ptrs]), stream))

    def peer_handle(self):
        buf = ctypes.create_string_buffer(PEER_HANDLE_BYTES)
        _ok(_lib.qagg_dense_peer_handle(self.h, buf))
        return buf.raw

    def enable_peer(self, handles):
        blob = b"".join(handles)
        _ok(_lib.qagg_dense_enable_peer(self.h, ctypes.create_string_buffer(blob, len(blob))))

    def check(self, stream=0):
        _ok(_lib.qagg_dense_check(self.h, stream))

    @property
    def wire_bytes(self):
        return int(_lib.qagg_dense_wire_bytes(self.h))

    def destroy(self):
        if self.h:
            _ok(_lib.qagg_dense_destroy(self.h))
            self.h = None


def dense_step_group(aggs, grad_ptrs, stream=0):
    K = len(aggs)
    ha = (c_vp * K)(*[a.h for a in aggs])
    rows = [(c_vp * len(g))(*[c_vp(p) for p in g]) for g in grad_ptrs]
    pp = (ctypes.POINTER(c_vp) * K)(*[ctypes.cast(r, ctypes.POINTER(c_vp)) for r in rows])
    _ok(_lib.qagg_dense_step_group(ha, K, pp, stream))


class HostAggregator:
    """qagg_host_aggregator: aggregation of gradients held in host memory, chunk-pipelined over PCIe."""

    def __init__(self, comm, shapes, bits, flags=ZERO_THRESHOLD | SELF_QUANTIZED, chunks=6):
        T = len(shapes)
        Ms = (c_i64 * T)(*[s[0] for s in shapes])
        Ns = (c_i64 * T)(*[s[1] for s in shapes])
        h = c_vp()
        _ok(_lib.qagg_hagg_create(comm.h, T, Ms, Ns, bits, flags, chunks, ctypes.byref(h)))
        self.h, self.T = h, T
        self.chunks = int(_lib.qagg_hagg_chunks(h))

    def peer_handles(self):
        buf = ctypes.create_string_buffer(PEER_HANDLE_BYTES * self.chunks)
        _ok(_lib.qagg_hagg_peer_handles(self.h, buf))
        return buf.raw

    def enable_peer(self, handles_per_rank):
        blob = b"".join(handles_per_rank)
        _ok(_lib.qagg_hagg_enable_peer(self.h, ctypes.create_string_buffer(blob, len(blob))))

    def step(self, host_grad_ptrs):
        _ok(_lib.qagg_hagg_step(self.h, (c_vp * len(host_grad_ptrs))(*[c_vp(p) for p in host_grad_ptrs])))

    def copy_only(self, host_grad_ptrs):
        _ok(_lib.qagg_hagg_copy_only(self.h, (c_vp * len(host_grad_ptrs))(*[c_vp(p) for p in host_grad_ptrs])))

    def check(self):
        _ok(_lib.qagg_hagg_check(self.h))

    def destroy(self):
        if self.h:
            _ok(_lib.qagg_hagg_destroy(self.h))
            self.h = None


def step_group(aggs, grad_ptrs, stream=0, headers=None):
    """grad_ptrs[r][i]: device pointers of rank r's gradients; headers[r]: rank r's header values (optional)."""
    K = len(aggs)
    ha = (c_vp * K)(*[a.h for a in aggs])
    rows = [(c_vp * len(g))(*[c_vp(p) for p in g]) for g in grad_ptrs]
    pp = (ctypes.POINTER(c_vp) * K)(*[ctypes.cast(r, ctypes.POINTER(c_vp)) for r in rows])
    if headers is None:
        _ok(_lib.qagg_agg_step_group(ha, K, pp, stream))
        return
    n = len(headers[0])
    hrows = [(ctypes.c_double * n)(*h) for h in headers]
    hp = (ctypes.POINTER(ctypes.c_double) * K)(*[ctypes.cast(r, ctypes.POINTER(ctypes.c_double)) for r in hrows])
    _ok(_lib.qagg_agg_step_group_header(ha, K, pp, hp, n, stream))


class AggregatorF64:
    """AllReduceDistGradAggregator<double>: the striped aggregation for double gradients (qagg_agg_f64_*)."""

    def __init__(self, comm, shapes, bits, flags=ZERO_THRESHOLD | SELF_QUANTIZED):
        T = len(shapes)
        M = (c_i64 * max(T, 1))(*[s[0] for s in shapes])
        N = (c_i64 * max(T, 1))(*[s[1] for s in shapes])
        h = c_vp()
        _ok(_lib.qagg_agg_f64_create(comm.h, T, M, N, bits, flags, ctypes.byref(h)))
        self.h, self.T = h, T

    def _ptrs(self, ptrs):
        assert len(ptrs) == self.T
        return (c_vp * max(self.T, 1))(*[c_vp(p) if p else c_vp(None) for p in ptrs])

    def step(self, grad_ptrs, stream=0):
        _ok(_lib.qagg_agg_f64_step(self.h, self._ptrs(grad_ptrs), stream))

    def reset_residuals(self, stream=0):
        _ok(_lib.qagg_agg_f64_reset_residuals(self.h, stream))

    def residual_ptrs(self, tensor):
        r, s = c_vp(), c_vp()
        _ok(_lib.qagg_agg_f64_residuals(self.h, tensor, ctypes.byref(r), ctypes.byref(s)))
        return r.value, s.value

    def copy_residual(self, tensor, which, dst_ptr, stream=0):
        _ok(_lib.qagg_agg_f64_copy_residual(self.h, tensor, which, dst_ptr, stream))

    def destroy(self):
        if self.h:
            _ok(_lib.qagg_agg_f64_destroy(self.h))
            self.h = None


def step_group_f64(aggs, grad_ptrs, stream=0):
    """One step of every rank of an in-process group of double aggregators."""
    K = len(aggs)
    handles = (c_vp * K)(*[a.h for a in aggs])
    rows = [a._ptrs(p) for a, p in zip(aggs, grad_ptrs)]
    table = (ctypes.POINTER(c_vp) * K)(*[ctypes.cast(r, ctypes.POINTER(c_vp)) for r in rows])
    _ok(_lib.qagg_agg_f64_step_group(handles, K, table, stream))
