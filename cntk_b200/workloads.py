"""Gradient-set shapes of the benchmark configurations (rows M x columns N per tensor, column-major fp32).

CNTK stores the weight of Times(W, x) with rows = output dimension, so a 429 -> 2048 layer is a 2048 x 429 matrix
and its bias a 2048 x 1 column.  These are shape lists only; values are synthetic (seeded normal / Laplace draws).
"""


def speech_dnn():
    """Speech feed-forward DNN: 429 -> 2048 -> (x6) 2048 -> 9304 with biases: 16 tensors, 45,122,648 values."""
    shapes = [(2048, 429)] + [(2048, 2048)] * 6 + [(9304, 2048)]
    shapes += [(2048, 1)] * 7 + [(9304, 1)]
    return shapes


def resnet50():
    """ResNet-50 (3-4-6-3 bottlenecks): 53 conv weights as [out_ch, in_ch*kh*kw], 106 BN scale/bias vectors,
    FC 1000 x 2048 and its bias: 161 tensors, 25,557,032 values."""
    shapes = []

    def conv(out_ch, in_ch, k):
        shapes.append((out_ch, in_ch * k * k))
        shapes.append((out_ch, 1))  # BN scale
        shapes.append((out_ch, 1))  # BN bias

    conv(64, 3, 7)
    in_ch = 64
    for width, blocks in ((64, 3), (128, 4), (256, 6), (512, 3)):
        for b in range(blocks):
            conv(width, in_ch, 1)
            conv(width, width, 3)
            conv(width * 4, width, 1)
            if b == 0:
                conv(width * 4, in_ch, 1)  # projection shortcut
            in_ch = width * 4
    shapes.append((1000, 2048))
    shapes.append((1000, 1))
    return shapes


def lstm_lm():
    """LSTM language model: 50000 x 512 embedding (90% of columns zero), two LSTM layers (2048 x 1024 + bias 2048),
    512 x 50000 softmax: 55,398,400 values."""
    return [(50000, 512), (2048, 1024), (2048, 1), (2048, 1024), (2048, 1), (512, 50000)]


def round_trip_2048():
    return [(2048, 2048)]


def sweep(k):
    """1024 rows, 1024 * 4^k columns (k = 0..5: 1 Mi .. 1 Gi values)."""
    return [(1024, 1024 * 4 ** k)]


def total_values(shapes):
    return sum(m * n for m, n in shapes)


def packed_bytes(shapes, bits):
    return sum(n * (8 + 4 * ((m * bits + 31) // 32)) for m, n in shapes)


def algorithmic_bytes(shapes, bits, K):
    """Bytes one rank must move through HBM per step when every input and output is touched exactly once:
    quantize 12V + P, owner reduce 8V/K + P(1 + 1/K), unquantize 4V + P  (V values, P packed bytes)."""
    V, P = total_values(shapes), packed_bytes(shapes, bits)
    k1 = 12 * V + P
    k3 = 4 * V + P
    k2 = 0 if K == 1 else 8 * V / K + P * (1 + 1 / K)
    return {"quantize": k1, "reduce_requantize": k2, "unquantize": k3, "total": k1 + k2 + k3}


def dense_algorithmic_bytes(shapes, K):
    """Unquantized fp32 arm: bytes one rank must move through its HBM per step when every buffer is touched once: read the
    gradients (4V), land the K received slices (4V), read them for the sum (4V), land the gathered result (4V), read it and
    write the gradients (8V): 24V.  (With one rank the arm does nothing.)"""
    return 0 if K == 1 else 24 * total_values(shapes)
