"""The reference's dense CPU attention path, restated for timing and checking.

TEST INFRASTRUCTURE ONLY (checker and CPU baseline; never on the product path).

verification/verify.py:61-63 defines the reference's own oracle as
    with sdpa_kernel(SDPBackend.MATH):
        torch.nn.functional.scaled_dot_product_attention(q, k, v, bool_mask)
on a dense [L, L] boolean mask. That script cannot be imported (it needs the compiled CUDA modules and
runs at import), and an [L, L] mask does not fit beyond L ~ 64K, so the same call is made here on row
chunks: chunk rows x all L keys, with the mask chunk built from the closed-form index sets
(verify.py:184-205, 376-382, 423-431). Same math, same torch kernel, all host threads.
"""
from __future__ import annotations

import os
import time

import torch
from torch.nn.attention import SDPBackend, sdpa_kernel


def mask_chunk(kind: str, L: int, r0: int, r1: int, p0: int, p1: int = 0, G=None) -> torch.Tensor:
    """Boolean [r1-r0, L] slice of the dense mask, True = attend."""
    i = torch.arange(r0, r1).unsqueeze(1)
    j = torch.arange(L).unsqueeze(0)
    if kind == "local":
        return (i - j).abs() <= p0
    if kind == "local_1d_dilated":
        s = p1 + 1
        return ((i - j).abs() <= p0 * s) & ((i - j) % s == 0)
    if kind == "local_2d_dilated":
        s, B = p1 + 1, p0
        return ((i // B) == (j // B)) & ((i % B) % s == 0) & ((j % B) % s == 0)
    if kind == "global_no_local":
        isg = torch.zeros(L, dtype=torch.bool)
        isg[torch.as_tensor(G, dtype=torch.long)] = True
        return (isg[r0:r1].unsqueeze(1) | isg.unsqueeze(0)) & ((i - j).abs() > p0)
    raise ValueError(kind)


def sdpa_rows(q_rows: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    with sdpa_kernel(SDPBackend.MATH):
        return torch.nn.functional.scaled_dot_product_attention(q_rows, k, v, mask)


def time_dense_cpu(kind: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, p0: int, p1: int = 0, G=None,
                   chunk_rows: int = 1024, budget_s: float = 15.0, max_chunks: int | None = None,
                   nnz_of_rows=None, mask_fn=None):
    """Time the dense masked SDPA-MATH path on evenly spaced row chunks until ~budget_s is spent.

    Returns dict(seconds, rows, chunks, nnz, threads, cores). `nnz_of_rows(r0, r1)` gives the mask
    non-zeros of a row range (for the effective nnz-FLOP/s figure); mask construction is outside the
    timed region, as it is in the reference script. `mask_fn(r0, r1)` replaces the closed-form mask chunk
    (explicit masks: the caller scatters its CSR/COO entries into a dense boolean chunk)."""
    chunk_of = mask_fn if mask_fn is not None else (lambda a, b: mask_chunk(kind, q.shape[0], a, b, p0, p1, G))
    L = q.shape[0]
    n_chunks_total = (L + chunk_rows - 1) // chunk_rows
    plan = min(max_chunks or n_chunks_total, n_chunks_total)
    starts = [int(c * n_chunks_total / plan) * chunk_rows for c in range(plan)]
    # warm-up on one chunk (thread pool, allocator)
    m0 = chunk_of(0, min(chunk_rows, L))
    sdpa_rows(q[: m0.shape[0]], k, v, m0)
    spent, rows, nnz, done = 0.0, 0, 0, 0
    for r0 in starts:
        r1 = min(L, r0 + chunk_rows)
        mask = chunk_of(r0, r1)
        t0 = time.perf_counter()
        sdpa_rows(q[r0:r1], k, v, mask)
        spent += time.perf_counter() - t0
        rows += r1 - r0
        nnz += int(mask.sum().item()) if nnz_of_rows is None else int(nnz_of_rows(r0, r1))
        done += 1
        if spent >= budget_s:
            break
    return {"seconds": spent, "rows": rows, "chunks": done, "nnz": nnz, "threads": torch.get_num_threads(),
            "cores": os.cpu_count()}
