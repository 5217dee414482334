"""GPU: the index set the TENSOR-CORE path visits, checked exactly, and the benchmarked configurations.

The tiled kernels decide "does row i attend to key j" with their own predicates (per-row intervals, chunk
classes, exclusion intervals, bit masks of explicit dense tiles), not with the column generators the gather
kernels use, so their index set is probed through the arithmetic itself with inputs that make every step
exact in TF32/FP32:

    Q = 0                      every score is 0, every probability exp2(0) = 1.0
    V[j] = one-hot((j // div) mod d)   div in {1, d}: the two passes together identify keys modulo d*d

Then l(i) = |J(i)| exactly (counts below 2^24 are exact in fp32) and round(O(i, c) * l(i)) is the number of
keys of J(i) whose ((j // div) mod d) equals c. Both are compared with torch.equal against the same
histograms of the oracle's closed-form index sets (oracle/spfa_oracle.c: implicit_csr), i.e. a key that is
dropped, added, or swapped for another residue fails the test.
"""
import numpy as np
import pytest
import torch

from conftest import random_csr, seeded_qkv

pytestmark = pytest.mark.gpu

TOL_GATHER = 1e-5
TOL_TILED = 2e-3


@pytest.fixture(scope="module")
def capi(pkg):
    assert torch.cuda.is_available()
    c = pkg.capi
    c.lib()
    yield c
    c.set_path(c.PATH_AUTO)


@pytest.fixture(autouse=True)
def no_device_timeouts(capi):
    yield
    assert capi.last_device_error() == 0, "a tiled kernel reported a timed-out wait"


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def residue_histogram(row_off, col, n_rows, n_keys, d, div):
    """[n_rows, d] int64: entries of row r whose ((col // div) mod d) is c. Columns >= n_keys are skipped
    (the ABI skips them). Computed with torch on the GPU from the oracle's (or the caller's) CSR arrays."""
    off = torch.from_numpy(np.asarray(row_off).astype(np.int64)).cuda()
    c = torch.from_numpy(np.asarray(col).astype(np.int64)).cuda()
    rows = torch.repeat_interleave(torch.arange(n_rows, device="cuda"), off[1:] - off[:-1])
    keep = c < n_keys
    key = rows[keep] * d + (c[keep] // div) % d
    return torch.bincount(key, minlength=n_rows * d).view(n_rows, d)


def assert_exact_index_set(capi, forward, row_off, col, n_rows, n_keys, d, expect_tiled=True, what=""):
    """forward(Q, K, V, m, l, O) runs one operator call on n_rows query rows and n_keys keys."""
    g = torch.Generator(device="cuda").manual_seed(5)
    Q = torch.zeros(n_rows, d, device="cuda")
    K = torch.randn(n_keys, d, device="cuda", generator=g)
    j = torch.arange(n_keys, device="cuda")
    for div in (1, d):
        V = torch.zeros(n_keys, d, device="cuda")
        V[j, (j // div) % d] = 1.0
        want = residue_histogram(row_off, col, n_rows, n_keys, d, div)
        n = want.sum(1)
        st = capi.new_state(n_rows, d)
        forward(Q, K, V, *st)
        torch.cuda.synchronize()
        if expect_tiled:
            assert capi.last_path() == capi.PATH_TILED, f"{what}: expected the tiled path"
        m, l, O = st
        assert torch.equal(l, n.float()), f"{what} div={div}: key count differs on rows " \
                                          f"{torch.nonzero(l != n.float()).flatten()[:8].tolist()}"
        live = n > 0
        assert torch.equal(m[live], torch.zeros_like(m[live])) and torch.isinf(m[~live]).all()
        got = torch.round(O * l[:, None]).long()
        assert torch.equal(got, want), f"{what} div={div}: per-residue key counts differ on rows " \
                                       f"{torch.nonzero((got != want).any(1)).flatten()[:8].tolist()}"


# ------------------------------------------------------------------------------------------------------
# (a) exact index sets on the tiled path
# ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("L,d,w", [(65536, 64, 256), (1, 64, 0), (127, 32, 60), (129, 64, 128), (1000, 128, 33),
                                    (1000, 64, 999), (385, 32, 64), (4096, 128, 300)])
def test_local_index_set_exact_on_the_tiled_path(capi, orc, L, d, w):
    capi.set_path(capi.PATH_TILED)
    row_off, col = orc.implicit_csr("local", L, w)
    assert_exact_index_set(capi, lambda Q, K, V, m, l, O: capi.local_forward(Q, K, V, m, l, O, w), row_off, col, L, L,
                           d, what=f"local L={L} d={d} w={w}")


@pytest.mark.parametrize("L,d,w,rb,re", [(65536, 64, 256, 12345, 23456), (5000, 128, 100, 1, 4999),
                                          (3000, 32, 40, 2900, 3000)])
def test_local_row_shards_index_set_exact(capi, orc, L, d, w, rb, re):
    capi.set_path(capi.PATH_TILED)
    row_off, col = orc.implicit_csr("local", L, w, row_begin=rb, row_end=re)
    assert_exact_index_set(capi, lambda Q, K, V, m, l, O: capi.local_forward(Q, K, V, m, l, O, w, rb, re), row_off,
                           col, re - rb, L, d, what=f"local shard [{rb},{re}) of L={L}")


@pytest.mark.parametrize("L,d,w,dil,rb,re", [(131072, 128, 512, 1, 0, None), (131072, 128, 512, 2, 70001, 90002),
                                              (5000, 64, 40, 2, 0, None), (5000, 32, 33, 6, 0, None),
                                              (5000, 64, 20, 15, 0, None), (4099, 128, 50, 3, 1234, 3210),
                                              (777, 64, 100, 4, 0, None)])
def test_local_1d_dilated_index_set_exact_on_the_tiled_path(capi, orc, L, d, w, dil, rb, re):
    capi.set_path(capi.PATH_TILED)
    re = L if re is None else re
    row_off, col = orc.implicit_csr("local_1d_dilated", L, w, dil, row_begin=rb, row_end=re)
    assert_exact_index_set(
        capi, lambda Q, K, V, m, l, O: capi.local_1d_dilated_forward(Q, K, V, m, l, O, w, dil, rb, re), row_off, col,
        re - rb, L, d, what=f"l1d L={L} d={d} w={w} dil={dil} rows [{rb},{re})")


@pytest.mark.parametrize("L,d,w,nG,rb,re,dups", [(4096, 64, 50, 300, 0, None, True), (3000, 128, 17, 64, 0, None, False),
                                                  (8192, 32, 100, 1024, 1000, 7000, True),
                                                  (131072, 128, 256, 64, 0, None, False),
                                                  (20000, 64, 0, 32, 5, 19999, True)])
def test_global_no_local_index_set_exact_on_the_tiled_path(capi, orc, L, d, w, nG, rb, re, dups):
    """Both launches of the strip: ordinary rows x gathered listed keys (mode 1) and listed rows x all keys
    (mode 2, split key range + combine)."""
    capi.set_path(capi.PATH_TILED)
    re = L if re is None else re
    rng = np.random.default_rng(L + nG)
    G = rng.choice(L, nG, replace=False).astype(np.int32)  # list order: unsorted
    if dups:
        G[nG // 2] = G[0]
        G[nG - 1] = G[1]
    row_off, col = orc.implicit_csr("global_no_local", L, w, G=G, row_begin=rb, row_end=re)
    Gd = dev(G)
    assert_exact_index_set(
        capi, lambda Q, K, V, m, l, O: capi.global_no_local_forward(Q, K, V, m, l, O, Gd, w, rb, re), row_off, col,
        re - rb, L, d, what=f"gnl L={L} d={d} w={w} nG={nG} rows [{rb},{re})")


@pytest.mark.parametrize("L,d,w,nG,rb,re", [(4096, 64, 50, 300, 0, None), (3000, 128, 33, 64, 0, None),
                                             (8192, 32, 100, 1024, 1000, 7000), (65536, 64, 256, 64, 0, None)])
def test_fused_band_and_global_keys_index_set_exact(capi, orc, L, d, w, nG, rb, re):
    """The fused Local + Global-no-local pass (band tiles and gathered global-key tiles in one kernel, global rows as
    a strip over all keys): the union of the two closed-form index sets, exactly."""
    capi.set_path(capi.PATH_TILED)
    re = L if re is None else re
    G = np.random.default_rng(L + nG).choice(L, nG, replace=False).astype(np.int32)
    off_a, col_a = orc.implicit_csr("local", L, w, row_begin=rb, row_end=re)
    off_b, col_b = orc.implicit_csr("global_no_local", L, w, G=G, row_begin=rb, row_end=re)
    # union of two disjoint index sets, row by row
    na, nb = np.diff(off_a.astype(np.int64)), np.diff(off_b.astype(np.int64))
    row_off = np.concatenate([[0], np.cumsum(na + nb)]).astype(np.int64)
    col = np.empty(int(row_off[-1]), dtype=np.int64)
    rows_a = np.repeat(np.arange(re - rb), na)
    rows_b = np.repeat(np.arange(re - rb), nb)
    col[row_off[rows_a] + (np.arange(col_a.size) - off_a.astype(np.int64)[rows_a])] = col_a
    col[row_off[rows_b] + na[rows_b] + (np.arange(col_b.size) - off_b.astype(np.int64)[rows_b])] = col_b
    Gd = dev(G)
    assert_exact_index_set(
        capi, lambda Q, K, V, m, l, O: capi.bigbird_forward(Q, K, V, m, l, O, Gd, w, None, None, rb, re), row_off, col,
        re - rb, L, d, what=f"fused band + globals L={L} d={d} w={w} nG={nG} rows [{rb},{re})")


@pytest.mark.parametrize("L,Lk,d,half,density,shuffle", [(1000, 1300, 64, 70, 0.004, True), (700, 700, 32, 40, 0.003, False),
                                                         (515, 2048, 128, 90, 0.002, True)])
def test_explicit_dense_tiles_index_set_exact(capi, L, Lk, d, half, density, shuffle):
    """CSR mask = band + scattered entries, stored unsorted, with some columns >= Lk (skipped by the ABI): the
    dense (row block, key tile) pairs run on the tiled kernel under bit masks, the rest on the gather kernel; the
    union must be the stored index set exactly."""
    rng = np.random.default_rng(L * 7 + d)
    i = np.arange(L)[:, None]
    j = np.arange(Lk)[None, :]
    mask = (np.abs(i * Lk // L - j) <= half) | (rng.random((L, Lk)) < density)
    mask[5] = False  # an empty row
    rows_, cols_ = np.nonzero(mask)
    counts = np.bincount(rows_, minlength=L)
    row_off = np.zeros(L + 1, dtype=np.int64)
    row_off[1:] = np.cumsum(counts)
    col = cols_.astype(np.int64)
    # a few out-of-range columns spliced into existing rows (replacing real ones, so offsets stay valid)
    bad = rng.choice(col.size, 20, replace=False)
    col[bad] = Lk + rng.integers(0, 50, 20)
    if shuffle:
        for r in range(L):
            rng.shuffle(col[row_off[r]:row_off[r + 1]])
    ro, co = dev(row_off), dev(col.astype(np.int32))
    capi.set_path(capi.PATH_TILED)
    assert_exact_index_set(capi, lambda Q, K, V, m, l, O: capi.csr_forward(Q, K, V, ro, co, m, l, O), row_off, col, L,
                           Lk, d, what=f"explicit L={L} Lk={Lk} d={d}")


# ------------------------------------------------------------------------------------------------------
# (b) the CSR benchmark configuration itself: L = 4096, d = 64, eye + Bernoulli(0.01), every row vs the oracle
# ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("offsets,columns", [(torch.int64, torch.int32), (torch.uint64, torch.uint32),
                                             (torch.int32, torch.int32)])
def test_csr_benchmark_configuration_vs_oracle(capi, orc, offsets, columns):
    import bench

    L, d = 4096, 64
    seed = 1000 + sorted(bench.WORKLOADS).index("csr")
    row_off, col = bench.make_csr_mask(L, seed, torch.device("cuda"))
    Q, K, V = bench.make_qkv(L, d, seed, torch.device("cuda"))
    nnz = int(row_off[-1])
    assert 150_000 < nnz < 200_000 and int((row_off[1:] - row_off[:-1]).min()) >= 1
    want = orc.csr_forward(Q.cpu().numpy(), K.cpu().numpy(), V.cpu().numpy(), row_off.cpu().numpy(), col.cpu().numpy())
    ro = row_off.view(torch.uint64) if offsets == torch.uint64 else row_off.to(offsets)
    co = col.view(torch.uint32) if columns == torch.uint32 else col
    for path, tol in ((capi.PATH_AUTO, TOL_GATHER), (capi.PATH_GATHER, TOL_GATHER), (capi.PATH_TILED, TOL_TILED)):
        capi.set_path(path)
        st = capi.new_state(L, d)
        capi.csr_forward(Q, K, V, ro, co, *st)
        m, l, O = (t.cpu().double().numpy() for t in st)
        assert np.abs(O - want[2]).max() <= tol, f"path {path}"
        np.testing.assert_allclose(l, want[1], rtol=4e-3 if tol > 1e-4 else 1e-4)
        np.testing.assert_allclose(m, want[0], rtol=2e-3 if tol > 1e-4 else 1e-5, atol=tol)
    capi.set_path(capi.PATH_AUTO)
    # the same mask through the drop-in module
    import __graft_entry__ as entry

    mod = entry.load().binding("spfa_csr")
    st = capi.new_state(L, d)
    mod.forward(Q, K, V, ro, co, torch.ones(1, device="cuda"), *st, False)
    assert np.abs(st[2].cpu().double().numpy() - want[2]).max() <= TOL_GATHER
    # ... and as a COO mask with the same index widths
    rows = torch.repeat_interleave(torch.arange(L, device="cuda"), row_off[1:] - row_off[:-1])
    ri = rows.view(torch.uint64) if offsets == torch.uint64 else rows.to(offsets)
    for call in (lambda s_: capi.coo_forward(Q, K, V, ri, co, *s_),
                 lambda s_: entry.load().binding("spfa_coo").forward(Q, K, V, ri, co, torch.ones(1, device="cuda"), *s_, False)):
        st = capi.new_state(L, d)
        call(st)
        assert np.abs(st[2].cpu().double().numpy() - want[2]).max() <= TOL_GATHER


# ------------------------------------------------------------------------------------------------------
# (d) the reference's own kernels beside the AUTO (tensor-core) path at the benchmarked sizes
# ------------------------------------------------------------------------------------------------------
def _ref_module(kind):
    import importlib.util
    import os

    from conftest import ROOT

    spec = importlib.util.spec_from_file_location("spfa_build_ref", os.path.join(ROOT, "oracle", "build_ref.py"))
    br = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(br)
    mod = br.load(kind)
    if mod is None:
        pytest.skip("oracle/_ref/ not built (needs the reference tree at build time)")
    return mod


def _rows_dropping_a_chunk(n_keys, mepi):
    """Rows on which the unmodified reference drops its last chunk: key count an exact multiple (>= 2x) of its
    chunk length (sp_flatt_local_kernel.cu:82-93, sp_flatt_global_no_local_kernel.cu:120-131)."""
    return (n_keys % mepi == 0) & (n_keys >= 2 * mepi)


def test_reference_local_kernel_beside_the_tiled_path_at_config_size(capi, orc):
    L, d, w = 65536, 64, 256
    ref = _ref_module("local")
    g = torch.Generator(device="cuda").manual_seed(1002)
    Q, K, V = (torch.randn(L, d, device="cuda", generator=g) for _ in range(3))
    st_ref = capi.new_state(L, d)
    with torch.cuda.stream(torch.cuda.default_stream()):
        ref.forward(Q, K, V, *st_ref, w)
    torch.cuda.synchronize()
    capi.set_path(capi.PATH_AUTO)
    st = capi.new_state(L, d)
    capi.local_forward(Q, K, V, *st, w)
    torch.cuda.synchronize()
    assert capi.last_path() == capi.PATH_TILED
    i = torch.arange(L, device="cuda")
    n = torch.clamp(i + w + 1, max=L) - torch.clamp(i - w, min=0)
    bad = _rows_dropping_a_chunk(n, orc.ref_mepi("local", d))
    assert int(bad.sum()) == 12  # i = 19, 65, 111, 157, 203, 249 and their mirror images
    ok = ~bad
    assert (st[2][ok] - st_ref[2][ok]).abs().max().item() <= TOL_TILED
    assert torch.allclose(st[1][ok], st_ref[1][ok], rtol=4e-3) and torch.allclose(st[0][ok], st_ref[0][ok], rtol=2e-3, atol=TOL_TILED)
    assert (st[2][bad] - st_ref[2][bad]).abs().max().item() > 1e-4  # the reference really differs there


def test_reference_global_kernel_beside_the_tiled_path_at_config_size(capi, orc):
    L, d, w, nG = 131072, 128, 256, 64
    ref = _ref_module("global_no_local")
    g = torch.Generator(device="cuda").manual_seed(1003)
    Q, K, V = (torch.randn(L, d, device="cuda", generator=g) for _ in range(3))
    G = np.sort(np.random.default_rng(1003).choice(L, nG, replace=False)).astype(np.int32)
    Gd = dev(G)
    # key counts per row (closed form): listed rows see L - |W(i)| keys, the others the listed keys outside W(i)
    i = torch.arange(L, device="cuda")
    lo, hi = torch.clamp(i - w, min=0), torch.clamp(i + w + 1, max=L)
    Gs = torch.from_numpy(G.astype(np.int64)).cuda()
    inside = torch.searchsorted(Gs, hi) - torch.searchsorted(Gs, lo)
    isg = torch.zeros(L, dtype=torch.bool, device="cuda")
    isg[Gs] = True
    n = torch.where(isg, L - (hi - lo), nG - inside)
    assert int(n.min()) > 0  # the reference divides 0/0 on key-less rows
    st_ref = capi.new_state(L, d)
    with torch.cuda.stream(torch.cuda.default_stream()):
        ref.forward(Q, K, V, *st_ref, Gd, w)
    torch.cuda.synchronize()
    capi.set_path(capi.PATH_AUTO)
    st = capi.new_state(L, d)
    capi.global_no_local_forward(Q, K, V, *st, Gd, w)
    torch.cuda.synchronize()
    assert capi.last_path() == capi.PATH_TILED
    ok = ~_rows_dropping_a_chunk(n, orc.ref_mepi("global_no_local", d))
    assert int(ok.sum()) > L // 2
    assert (st[2][ok] - st_ref[2][ok]).abs().max().item() <= TOL_TILED
    assert torch.allclose(st[1][ok], st_ref[1][ok], rtol=4e-3) and torch.allclose(st[0][ok], st_ref[0][ok], rtol=2e-3, atol=TOL_TILED)
