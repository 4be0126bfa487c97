"""Index arithmetic of the streaming quantize kernel restated in Python (no GPU): an element thread owns fixed 16-byte
positions (column, four rows) of every chunk and moves its (packed word, bit) pair from chunk to chunk by a fixed step
instead of dividing; row i of a column must land on bit i // Q of word i % Q (the reference's packed layout,
Source/Math/ColumnQuantizer.h:36-40, 90-147), every row exactly once, for any column height and item width -- including
columns so short that a chunk wraps through several bit positions (Q < 4) and heights that are not a multiple of 4."""
import pytest

TILE_VALUES = 1536
ETHREADS = 192
U = 2


def chunk_rows(cols):
    return min(256, (TILE_VALUES // cols) // 32 * 32)


def walk_item(M, nc):
    """Returns {(column, row): (word, bit)} as the kernel's element threads would produce it."""
    Q = (M + 31) // 32
    R = chunk_rows(nc)
    R4 = R // 4
    nchunks = (M + R - 1) // R
    advK, advW = R // Q, R % Q
    out = {}
    for et in range(ETHREADS):
        for u in range(U):
            f = et + ETHREADS * u
            if f >= nc * R4:
                continue
            c, r = f // R4, 4 * (f % R4)
            pk, pw = r // Q, r % Q
            for q in range(nchunks):
                row = q * R + r
                if row < M:
                    nv = min(4, M - row)
                    flat = nv == 4 and pw + 3 < Q
                    for i in range(nv):
                        if flat:
                            w, k = pw + i, pk
                        else:
                            over = (pw + i) // Q
                            w, k = pw + i - over * Q, pk + over
                        assert (c, row + i) not in out
                        out[(c, row + i)] = (w, k)
                pw += advW
                pk += advK
                if pw >= Q:
                    pw -= Q
                    pk += 1
    return out, Q


@pytest.mark.parametrize("M", [1, 3, 31, 32, 33, 64, 70, 96, 100, 127, 129, 291 * 4, 2048, 2049, 9304])
@pytest.mark.parametrize("nc", [1, 2, 3, 6, 8, 16, 24, 32])
def test_every_row_lands_on_its_word_and_bit(M, nc):
    got, Q = walk_item(M, nc)
    assert len(got) == M * nc
    for (c, row), (w, k) in got.items():
        assert (w, k) == (row % Q, row // Q)
        assert k < 32
