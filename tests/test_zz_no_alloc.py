"""GPU: the allocation-free COO entry point (spfa_coo_forward_f32_static) against the workspace variant.

Some hosts of this library may not allocate device memory when they call it (a server that owns the whole
device budget through its own pool, a section where cudaMalloc's device-wide synchronisation is not
acceptable). For them the COO row pointers live in a static device array inside the library. This file is
collected last on purpose: if the variant ever breaks, every other test has already run.

The calls go straight through the C ABI with raw pointers -- no workspace, no torch allocation between the
two back-to-back calls -- and must reproduce the existing entry point within the gather path's tolerance
(the two run the same kernels, so the results are in fact identical)."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import random_csr, seeded_qkv

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _call_static(lib, Q, K, V, rows, cols, st, row_begin, use_nan):
    m, l, O = st
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.spfa_coo_forward_f32_static(p(Q), p(K), p(V), p(rows), p(cols), rows.shape[0], p(m), p(l), p(O),
                                           row_begin, Q.shape[0], K.shape[0], Q.shape[1], int(use_nan), stream)


def test_static_scratch_matches_workspace_variant_twice_in_a_row(pkg):
    capi = pkg.capi
    lib = capi.lib()
    assert lib.spfa_coo_static_max_rows() == 262144
    cases = []
    for L, Lk, d, density, seed in ((700, 900, 64, 0.03, 1), (1500, 1500, 32, 0.01, 2)):
        Q, K, V = seeded_qkv(L, d, seed, Lk)
        mask, row_off, col = random_csr(L, Lk, density, seed + 10, empty_rows=(0, L // 2, L - 1))
        rows = np.repeat(np.arange(L, dtype=np.int64), np.diff(row_off.astype(np.int64)))
        cases.append((_dev(Q), _dev(K), _dev(V), _dev(rows), _dev(col.astype(np.int32))))
    # reference results from the existing entry point (it allocates its workspace through torch)
    want = []
    for Q, K, V, rows, cols in cases:
        st = capi.new_state(Q.shape[0], Q.shape[1])
        capi.coo_forward(Q, K, V, rows, cols, *st, use_nan=True)
        want.append(tuple(t.clone() for t in st))
    # all buffers exist before the calls under test; two calls in a row share the static array
    states = [capi.new_state(Q.shape[0], Q.shape[1]) for Q, *_ in cases]
    warm = capi.new_state(cases[0][0].shape[0], cases[0][0].shape[1])
    assert _call_static(lib, *cases[0], warm, 0, True) == 0  # first call on the device: resolves the array's address
    del st  # a leftover state of the loop above would be freed (not allocated) when the name is bound again below
    torch.cuda.synchronize()
    # the property the entry point exists for: the calls below take no device memory, neither from the driver
    # (free memory of the device unchanged) nor from torch's caching allocator
    free_before, alloc_before, reserved_before = (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(),
                                                  torch.cuda.memory_reserved())
    for (Q, K, V, rows, cols), st in zip(cases, states):
        assert _call_static(lib, Q, K, V, rows, cols, st, 0, True) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_allocated() == alloc_before and torch.cuda.memory_reserved() == reserved_before
    for st, ref in zip(states, want):
        for got, exp in zip(st, ref):
            g, e = got.cpu().double().numpy(), exp.cpu().double().numpy()
            assert np.array_equal(np.isnan(g), np.isnan(e))
            fin = np.isfinite(e)
            assert np.array_equal(np.isfinite(g), fin)
            assert np.max(np.abs(g[fin] - e[fin]), initial=0.0) <= TOL
    # a row shard (rows 200..500 of the first case) through the same array, after the calls above
    Q, K, V, rows, cols = cases[0]
    st = capi.new_state(300, Q.shape[1])
    assert _call_static(lib, Q[200:500].contiguous(), K, V, rows, cols, st, 200, True) == 0
    torch.cuda.synchronize()
    for got, exp in zip(st, want[0]):
        g, e = got.cpu().double().numpy(), exp[200:500].cpu().double().numpy()
        fin = np.isfinite(e)
        assert np.array_equal(np.isnan(g), np.isnan(e)) and np.max(np.abs(g[fin] - e[fin]), initial=0.0) <= TOL
    assert capi.last_device_error() == 0


def test_static_scratch_empty_mask_small_dimension_and_foreign_entries(pkg):
    """An empty mask with use_nan (every row NaN), d = 16, and row shards whose entry list holds only entries of
    other rows before or after them."""
    capi = pkg.capi
    lib = capi.lib()
    L, d = 300, 16
    Q, K, V = (_dev(x) for x in seeded_qkv(L, d, 5))
    none = torch.zeros(0, dtype=torch.int64, device="cuda")
    st = capi.new_state(L, d)
    assert _call_static(lib, Q, K, V, none, none.to(torch.int32), st, 0, True) == 0
    torch.cuda.synchronize()
    assert torch.isnan(st[2]).all() and torch.isinf(st[0]).all() and not st[1].any()
    mask, row_off, col = random_csr(L, L, 0.05, 3)
    rows = _dev(np.repeat(np.arange(L, dtype=np.int64), np.diff(row_off.astype(np.int64))))
    cols = _dev(col.astype(np.int32))
    want = capi.new_state(L, d)
    capi.coo_forward(Q, K, V, rows, cols, *want, use_nan=True)
    for rb, re, keep in ((100, 200, rows < 200), (100, 200, rows >= 100), (0, 50, rows >= 100)):
        st = capi.new_state(re - rb, d)
        assert _call_static(lib, Q[rb:re].contiguous(), K, V, rows[keep].contiguous(), cols[keep].contiguous(), st, rb, True) == 0
        torch.cuda.synchronize()
        if rb == 0:  # rows 0..49 have no entry in the list: NaN rows
            assert torch.isnan(st[2]).all()
        else:
            assert (st[2] - want[2][rb:re]).abs().max().item() <= TOL and torch.equal(st[1], want[1][rb:re])
    assert capi.last_device_error() == 0


def test_static_scratch_rejects_more_rows_than_it_holds(pkg):
    capi = pkg.capi
    lib = capi.lib()
    d = 16
    n = int(lib.spfa_coo_static_max_rows()) + 1
    Q = torch.zeros(n, d, device="cuda")
    K = torch.zeros(8, d, device="cuda")
    rows = torch.zeros(1, dtype=torch.int64, device="cuda")
    cols = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = capi.new_state(n, d)
    rc = _call_static(lib, Q, K, K, rows, cols, st, 0, False)
    assert rc == -11 and "maximum" in capi.status_string(rc)
    torch.cuda.synchronize()
    assert torch.isinf(st[0]).all() and not st[1].any()  # nothing was launched
