"""Work items of the streaming quantize kernel (host arithmetic, no GPU): every column of every tensor belongs to exactly
one item, items respect the kernel's limits, and the queue is ordered the way the kernel's load balance relies on."""
import pytest

from cntk_b200 import lib, workloads

PKWORDS = 2560        # shared-memory words for an item's packed columns (quantize kernel)
TILE_VALUES = 1536    # values per chunk


def chunk_rows(cols):
    return min(256, (TILE_VALUES // cols) // 32 * 32)


def check_cover(shapes, items):
    seen = [[] for _ in shapes]
    for t, c0, n in items:
        assert 0 <= t < len(shapes) and n >= 1 and c0 >= 0 and c0 + n <= shapes[t][1]
        seen[t].append((c0, n))
    for t, (M, N) in enumerate(shapes):
        cols = sorted(seen[t])
        if M == 0 or N == 0:
            assert not cols
            continue
        pos = 0
        for c0, n in cols:
            assert c0 == pos, f"tensor {t}: gap or overlap at column {pos}"
            pos += n
        assert pos == N


@pytest.mark.parametrize("name", ["speech_dnn", "resnet50", "lstm_lm", "round_trip_2048"])
@pytest.mark.parametrize("sms", [1, 148])
def test_quantize_items_cover_every_column_once(name, sms):
    shapes = getattr(workloads, name)()
    items = lib.stream_items(shapes, bits=1, num_sms=sms)
    check_cover(shapes, items)
    for t, c0, n in items:
        M = shapes[t][0]
        Q = (M + 31) // 32
        assert n <= 32 and n * Q <= PKWORDS
        assert n * chunk_rows(n) <= TILE_VALUES


def test_speech_set_queue_order_and_widths():
    shapes = workloads.speech_dnn()
    items = lib.stream_items(shapes, bits=1, num_sms=148)
    # at least eight columns per item wherever the tensor has them (the walkers' add chains set the pace below that)
    for t, c0, n in items:
        N = shapes[t][1]
        if N >= 8 and c0 + n < N:
            assert n >= 8
    # the queue starts with the items of most chunks (the tall tensor and its single-column bias) ...
    def chunks(t, n):
        M = shapes[t][0]
        r = chunk_rows(n)
        return -(-M // r)
    first = [chunks(t, n) for t, c0, n in items[:256]]
    assert min(first) >= 37
    # ... and ends on short items: the last tenth has no item longer than a 12-column item of a 2048-row matrix (16 chunks
    # of 128 rows)
    tail = [chunks(t, n) for t, c0, n in items[-len(items) // 10:]]
    assert max(tail) <= 16
    # items hold at most 24 K values wherever the eight-column minimum allows
    for t, c0, n in items:
        assert n <= 8 or shapes[t][0] * n <= 24576
    # deterministic
    assert items == lib.stream_items(shapes, bits=1, num_sms=148)


def test_bad_arguments():
    with pytest.raises(lib.QaggError):
        lib.stream_items([(2048, 16)], bits=3)
    with pytest.raises(lib.QaggError):
        lib.stream_items([(200000, 4)], bits=1)  # packed column does not fit the kernel's shared-memory budget
    assert lib.stream_items([], bits=1) == []
    assert lib.stream_items([(0, 5), (7, 0)], bits=1) == []
