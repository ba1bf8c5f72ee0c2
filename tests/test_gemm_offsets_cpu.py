"""The GEMM producer's bulk copies stay inside the operand buffers.

The metadata and scale-factor tiles are fetched with plain bulk copies that have no bounds
check, so their offsets are restated here exactly as the producer warp of
sharq_b200/csrc/gemm.cu computes them and compared, over a grid of shapes and kernel variants
(single-CTA 128/256-wide tiles, CTA pairs), with the buffer sizes the C ABI reports
(sharq_get_sparse_nvfp4_buffer_sizes / sharq_get_fused_sparse_residual_buffer_sizes).
"""
import ctypes
import itertools

import pytest

from sharq_b200 import _lib


def _sizes(m, n, k):
    lib = _lib.lib()
    sp = (ctypes.c_int64 * 4)()
    assert lib.sharq_get_sparse_nvfp4_buffer_sizes(m, n, k, sp) == 0
    fu = (ctypes.c_int64 * 5)()
    assert lib.sharq_get_fused_sparse_residual_buffer_sizes(m, n, k, fu) == 0
    return {"a_comp": sp[0], "e": sp[1], "sfa": sp[2], "sfb": sp[3], "q_res": fu[3], "sf_res": fu[4]}


def _producer_reads(m, n, k, bn, pair):
    """Yield (buffer, offset, nbytes) of every plain bulk copy of one GEMM launch."""
    bands = bn // 128
    k_stages = (k + 255) // 256
    aligned_m = (m + 127) // 128 * 128
    a_bands, b_bands = aligned_m // 128, (n + 127) // 128
    tiles_sp, tiles_d = k // 128, k // 64
    m_units = (m + 255) // 256 if pair else (m + 127) // 128
    n_tiles = (n + bn - 1) // bn
    for tile in range(m_units * n_tiles):
        for cta_rank in ((0, 1) if pair else (0,)):
            m_tile = 2 * (tile % m_units) + cta_rank if pair else tile % m_units
            n_tile = tile // m_units
            a_band = min(m_tile, a_bands - 1)
            b_band = [min(n_tile * bands + b, b_bands - 1) for b in range(bands)]
            for it in range(k_stages):
                n_sp = min(2, tiles_sp - 2 * it)
                n_d = min(4, tiles_d - 4 * it)
                yield "sf_res", (a_band * tiles_d + 4 * it) * 512, n_d * 512
                yield "e", (it * aligned_m + a_band * 128) * 16, 2048
                yield "sfa", (a_band * tiles_sp + 2 * it) * 512, n_sp * 512
                for b in range(bands):
                    yield "sfb", (b_band[b] * tiles_d + 4 * it) * 512, n_d * 512
                    yield "sfb", (b_band[b] * tiles_sp + 2 * it) * 512, n_sp * 512


M_CASES = (1, 16, 127, 128, 129, 256, 257, 300, 384, 2100, 2176)
N_CASES = (8, 128, 200, 256, 300, 384, 640, 4096)
K_CASES = (128, 256, 384, 896, 4096)


@pytest.mark.parametrize("bn,pair", [(128, False), (256, False), (256, True)])
def test_bulk_copies_stay_inside_the_buffers(bn, pair):
    for m, n, k in itertools.product(M_CASES, N_CASES, K_CASES):
        size = _sizes(m, n, k)
        for name, off, nbytes in _producer_reads(m, n, k, bn, pair):
            assert off >= 0 and off + nbytes <= size[name], (name, m, n, k, bn, pair, off, nbytes, size[name])


@pytest.mark.parametrize("cols_per_warp", [64, 128])
def test_scatter_epilogue_stages_and_stores_every_piece_once(cols_per_warp):
    """The scatter-mode epilogue of gemm.cu, restated: a warp owns 32 rows x cols_per_warp columns; per
    pass it stages 64 columns of 16 rows (lane l of the active half writes its row's eight 16-byte
    chunks c at slot c ^ (row & 7) of a 128-byte shared-memory row), then every lane reads chunk
    (lane & 7) of row it*4 + (lane >> 3) and stores it.  Every (row, 16-byte chunk) of the warp's
    block must be written to shared memory once and stored once, from the slot it was written to,
    and a store instruction must cover 4 rows x 128 contiguous bytes."""
    stored = {}
    for c in range(cols_per_warp // 64):
        for hrow in range(2):
            stage = {}
            for lane in range(32):
                if lane >> 4 != hrow:
                    continue
                srow = lane & 15
                for chunk_base in (0, 4):
                    for v in range(4):
                        slot = (srow, (chunk_base + v) ^ (srow & 7))
                        assert slot not in stage
                        stage[slot] = (lane, 64 * c + 8 * (chunk_base + v))  # (row in the warp's block, first column)
            assert len(stage) == 16 * 8
            for it in range(4):
                pieces = []
                for lane in range(32):
                    r = it * 4 + (lane >> 3)
                    src_row, col = stage[(r, (lane & 7) ^ (r & 7))]
                    grow, gcol = 16 * hrow + r, 64 * c + (lane & 7) * 8
                    assert (src_row, col) == (grow, gcol)  # the piece read back is the one that belongs there
                    assert (grow, gcol) not in stored
                    stored[(grow, gcol)] = True
                    pieces.append((grow, gcol))
                for q in range(4):  # each quarter-warp: one row, eight consecutive 16-byte pieces = 128 bytes
                    rows = {p[0] for p in pieces[8 * q:8 * q + 8]}
                    cols = [p[1] for p in pieces[8 * q:8 * q + 8]]
                    assert len(rows) == 1 and cols == list(range(cols[0], cols[0] + 64, 8))
    assert len(stored) == 32 * (cols_per_warp // 8)


@pytest.mark.parametrize("m,n,world", [(2048, 4096, 8), (2048, 4096, 2), (1024, 3584, 4), (256, 128, 2)])
def test_scatter_epilogue_addresses_land_in_the_senders_block(m, n, world):
    """Scatter mode of gemm.cu, restated: the 128-row tile m_tile belongs to GPU owner = m_tile * 128 / rows
    (rows = M / world); its stores go to d_peer[owner] + (rank - owner) * rows * N + global_row * N + col, which
    must be element (rank, global_row - owner * rows, col) of the owner's collection buffer [world][rows, N]."""
    rows = m // world
    assert rows % 128 == 0
    for rank in range(world):
        for m_tile in range(m // 128):
            owner = (m_tile * 128) // rows
            base = (rank - owner) * rows * n  # relative to d_peer[owner]
            for grow in (m_tile * 128, m_tile * 128 + 127):
                for col in (0, n - 8):
                    off = base + grow * n + col
                    local_row = grow - owner * rows
                    assert 0 <= local_row < rows
                    assert off == (rank * rows + local_row) * n + col
                    assert 0 <= off < world * rows * n
