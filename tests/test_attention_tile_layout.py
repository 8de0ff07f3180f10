"""Shared-memory layout of the tensor-core attention kernels' staged tiles,
checked on the host through the functions the kernels themselves use
(vitb200_attention_tile_index / _lane_column; no GPU needed).

A 64-row tile must map its elements one-to-one into 64 x pitch floats, the four
lanes of a quad must split the head dimension between them, and the kernels'
three access patterns must need the minimum number of shared-memory wavefronts
(no bank conflict): the 128-bit loads of product_rows (a lane reads 16-byte
chunks of its head-dimension slice from row 8n + g), the 64- or 128-bit loads
of product_columns (lane (g, t) reads its output columns g * hd/8 ... from rows
8s + 2t and 8s + 2t + 1) and the 128-bit stores of the staging pass.
"""
import pytest


@pytest.fixture(scope="module")
def lib(vit_host_module):
    return vit_host_module.load_backend_library()


def wavefronts(accesses, floats, lanes_per_phase):
    """Shared-memory wavefronts a warp-wide access needs: the hardware serves
    128 bytes per phase (8 lanes of 128 bits, 16 lanes of 64 bits); within a
    phase a bank (4 bytes wide, 32 of them) serves one address."""
    total = 0
    for first in range(0, 32, lanes_per_phase):
        banks = {}
        for start in accesses[first:first + lanes_per_phase]:
            for offset in range(start, start + floats):
                banks.setdefault(offset % 32, set()).add(offset)
        total += max(len(addresses) for addresses in banks.values())
    return total


LANES = [(lane >> 2, lane & 3) for lane in range(32)]   # (g, t)


@pytest.mark.parametrize("head_dim", [16, 32, 64])
def test_tile_layout_is_one_to_one_and_conflict_free(lib, head_dim):
    index = lambda row, col: lib.vitb200_attention_tile_index(head_dim, row, col)
    column = lambda t, e: lib.vitb200_attention_lane_column(head_dim, t, e)
    pitch = {16: 16, 32: 36, 64: 64}[head_dim]
    offsets = {index(row, col) for row in range(64) for col in range(head_dim)}
    assert len(offsets) == 64 * head_dim
    assert min(offsets) == 0 and max(offsets) < 64 * pitch
    # 16-byte chunks stay whole and aligned.
    for row in range(64):
        for col in range(0, head_dim, 4):
            base = index(row, col)
            assert base % 4 == 0
            assert [index(row, col + i) for i in range(4)] == [base + i for i in range(4)]
    # The quad's four lanes cover every column once.
    slice_len = head_dim // 4
    assert sorted(column(t, e) for t in range(4) for e in range(slice_len)) == \
        list(range(head_dim))
    # product_rows: 128-bit loads, rows 8n + g.
    for n in range(8):
        for chunk in range(slice_len // 4):
            accesses = [index(8 * n + g, column(t, 4 * chunk)) for g, t in LANES]
            assert wavefronts(accesses, 4, 8) == 4
    # product_columns: rows 8s + 2t (+ 1), the lane's hd / 8 output columns.
    outputs = head_dim // 8
    for s in range(8):
        for second in (0, 1):
            if outputs == 2:
                accesses = [index(8 * s + 2 * t + second, 2 * g) for g, t in LANES]
                assert wavefronts(accesses, 2, 16) == 2
            else:
                for chunk in range(outputs // 4):
                    accesses = [index(8 * s + 2 * t + second, outputs * g + 4 * chunk)
                                for g, t in LANES]
                    assert wavefronts(accesses, 4, 8) == 4
    # Staging: thread i stores the 16-byte chunk i of the row-major tile.
    per_row = head_dim // 4
    for first in range(0, 64 * per_row, 32):
        accesses = [index(i // per_row, 4 * (i % per_row))
                    for i in range(first, first + 32)]
        assert wavefronts(accesses, 4, 8) == 4


def test_layout_queries_reject_bad_arguments(lib):
    assert lib.vitb200_attention_tile_index(48, 0, 0) == -1
    assert lib.vitb200_attention_tile_index(16, 64, 0) == -1
    assert lib.vitb200_attention_tile_index(16, 0, 16) == -1
    assert lib.vitb200_attention_lane_column(64, 4, 0) == -1
    assert lib.vitb200_attention_lane_column(64, 0, 16) == -1
