"""Descriptor arithmetic of the attention kernels against a model of the 128-byte-swizzled UMMA operand
layouts (``csrc/flash_attn.cu``, ``csrc/flash_attn_bwd.cu``; the same conventions as the GEMM kernel, whose
four operand layouts are checked on hardware).

Model: a tile is made of rows of 128 bytes; the 16-byte chunk ``c`` of row ``r`` is stored at chunk
``c ^ (r & 7)`` (what a TMA load with the 128-byte swizzle writes and what the kernels' own stores write);
a fetch XORs address bits [4:6] with bits [7:9].  For one K = 16 step

* a K-major operand reads element ``(row, k)`` at ``start + (row % 8) * 128 + (row // 8) * SBO + 2 k``,
* an MN-major operand reads element ``(mn, k)`` at
  ``start + 2 (mn % 64) + (mn // 64) * LBO + (k % 8) * 128 + (k // 8) * SBO``.

The test builds the tiles the kernels build and checks that the start-address advances they use select
the intended sub-matrices.
"""

import numpy as np

TILE = 128 * 128          # bytes of a [128 x 64] bf16 tile


def _swz(byte):
    return byte ^ (((byte >> 7) & 7) << 4)


def _write_rows(smem, base, mat):
    for r in range(mat.shape[0]):
        for c in range(8):
            phys = base + r * 128 + ((c ^ (r & 7)) << 4)
            smem[phys // 2: phys // 2 + 8] = mat[r, c * 8:(c + 1) * 8]


def _fetch_k_major(smem, start, sbo, rows):
    return np.array([[smem[_swz(start + (r % 8) * 128 + (r // 8) * sbo + 2 * k) // 2] for k in range(16)] for r in range(rows)])


def _fetch_mn_major(smem, start, lbo, sbo, mn_extent):
    return np.array([[smem[_swz(start + 2 * (mn % 64) + (mn // 64) * lbo + (k % 8) * 128 + (k // 8) * sbo) // 2]
                      for k in range(16)] for mn in range(mn_extent)])


def test_attention_operand_layouts():
    rng = np.random.default_rng(0)
    smem = np.zeros(4 * TILE // 2)
    p = rng.standard_normal((128, 128))              # P or dS: [query][key], two blocks of 64 keys one tile apart
    _write_rows(smem, 0, p[:, :64])
    _write_rows(smem, TILE, p[:, 64:])
    v = rng.standard_normal((128, 64))               # V, K, Q or dO: [row][64]
    _write_rows(smem, 2 * TILE, v)
    for k in range(8):
        # forward P V and backward dS K: A = P as K-major operand, 16 keys per step
        a = _fetch_k_major(smem, (k >> 2) * TILE + (k & 3) * 32, 1024, 128)
        assert np.array_equal(a, p[:, 16 * k:16 * k + 16])
        # B = V (rows are the reduction index): MN-major, 16 rows = 2048 bytes per step
        b = _fetch_mn_major(smem, 2 * TILE + k * 2048, 8192, 1024, 64)
        assert np.array_equal(b, v[16 * k:16 * k + 16].T)
        # backward P^T dO and dS^T Q: A = the same bytes read transposed, key blocks LBO = one tile apart
        at = _fetch_mn_major(smem, k * 2048, TILE, 1024, 128)
        assert np.array_equal(at, p[16 * k:16 * k + 16, :].T)
    for k in range(4):
        # S = Q K^T and dP = dO V^T: both operands K-major, 16 of the 64 head dimensions per step
        a = _fetch_k_major(smem, 2 * TILE + k * 32, 1024, 128)
        assert np.array_equal(a, v[:, 16 * k:16 * k + 16])
