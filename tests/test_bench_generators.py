"""CPU: the synthetic mask generators and size formulas of bench.py against brute force at small sizes."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402


def test_block_dilated_csr_is_the_block_level_pattern():
    L, B, step = 2048, 128, 4
    row_off, col = bench.make_block_dilated_csr(L, B, step, "cpu")
    nb = L // B
    want = np.zeros((L, L), dtype=bool)
    for b in range(nb):
        for k in range(-2, 3):
            c = b + step * k
            if 0 <= c < nb:
                want[b * B:(b + 1) * B, c * B:(c + 1) * B] = True
    got = np.zeros((L, L), dtype=bool)
    ro = row_off.numpy()
    rows = np.repeat(np.arange(L), np.diff(ro))
    got[rows, col.numpy()] = True
    assert np.array_equal(got, want)
    assert ro[-1] == want.sum() == col.numel()
    for r in (0, 5 * B + 3, L - 1):  # ascending columns inside a row
        c = col[ro[r]:ro[r + 1]].numpy()
        assert np.all(np.diff(c) > 0)


def test_coo_graph_is_sorted_unique_and_contains_the_band():
    L, band = 4096, 8
    rows, cols = bench.make_coo_graph(L, band, 3, "cpu", mean_deg=4, max_deg=64)
    key = rows.numpy().astype(np.int64) * L + cols.numpy()
    assert np.all(np.diff(key) > 0)                       # (row, col) ascending, no duplicates
    present = set(key.tolist())
    for i in (0, 1, 100, L - 1):
        for j in range(max(0, i - band), min(L, i + band + 1)):
            assert i * L + j in present
    assert cols.min() >= 0 and cols.max() < L


def test_implicit_nnz_formulas_match_dense_masks():
    from oracle import dense_sdpa  # the checker's mask builders

    L = 600
    G = np.array([3, 200, 599], dtype=np.int32)
    for kind, p0, p1 in (("local", 37, 0), ("local_1d_dilated", 20, 2), ("local_2d_dilated", 100, 3),
                         ("global_no_local", 15, 0)):
        want = int(dense_sdpa.mask_chunk(kind, L, 0, L, p0, p1, G).sum())
        got = bench.implicit_nnz(kind, L, p0, p1, torch.from_numpy(G) if kind == "global_no_local" else None, 0, L)
        assert got == want, (kind, got, want)
        half = bench.implicit_nnz(kind, L, p0, p1, torch.from_numpy(G) if kind == "global_no_local" else None, 100, 400)
        assert half == int(dense_sdpa.mask_chunk(kind, L, 100, 400, p0, p1, G).sum())
