"""Helpers of the GPU parity tests: device buffers via torch, calls through the C ABI (cntk_b200.lib)."""
import numpy as np
import torch

from cntk_b200 import lib

DEV = "cuda:0"


def dev(a):
    """numpy -> device tensor (same bytes)."""
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def gpu_quantize(g, res, bits, zero_thr):
    """g, res: device float32 tensors of shape (N, M) (column-major M x N). res updated in place. Returns packed tensor."""
    N, M = g.shape
    packed = torch.zeros(lib.packed_bytes(M, N, bits), dtype=torch.uint8, device=DEV)
    lib.quantize(g.data_ptr(), res.data_ptr(), res.data_ptr(), packed.data_ptr(), M, N, bits, zero_thr)
    return packed


def gpu_unquantize(packed, out, bits, add):
    N, M = out.shape
    lib.unquantize(packed.data_ptr(), out.data_ptr(), M, N, bits, add)


def assert_same_bits(a, b, what):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    assert a.shape == b.shape, what
    if a.dtype == np.float32:
        a, b = a.view(np.uint32), b.view(np.uint32)
    if not np.array_equal(a, b):
        bad = np.argwhere(a != b)
        raise AssertionError(f"{what}: {len(bad)} of {a.size} elements differ; first at {bad[0].tolist()}: "
                             f"{a[tuple(bad[0])]:#x} vs {b[tuple(bad[0])]:#x}")
