"""CPU: the oracle against the fixtures made by the reference's own verification script, against an
independent dense numpy restatement, and its emulation of the reference's chunk-walk defects."""
import numpy as np
import pytest

from conftest import golden_calls, random_csr, seeded_qkv, unpack_mask

L, D = 256, 32


def _replay(orc, golden, call_fn):
    """Replay the recorded calls; state persists across calls that were not given a fresh state."""
    q, k, v = golden["q"], golden["k"], golden["v"]
    state, results = None, []
    for c in golden_calls(golden):
        if int(c["fresh"]):
            state = orc.new_state(L, D)
        state = call_fn(c, q, k, v, state)
        results.append((c, tuple(s.copy() for s in state)))
    return results


def _oracle_call(orc):
    def fn(c, q, k, v, state):
        op = c["op"]
        if op == "csr":
            return orc.csr_forward(q, k, v, c["row_off"], c["col"], state, bool(c["use_nan"]))
        if op == "coo":
            return orc.coo_forward(q, k, v, c["row"], c["col"], state, bool(c["use_nan"]))
        if op == "global_no_local":
            return orc.implicit_forward(op, q, k, v, int(c["p0"]), G=c["G"], state=state)
        return orc.implicit_forward(op, q, k, v, int(c["p0"]), int(c.get("p1", 0)), state=state,
                                    use_nan=bool(c.get("use_nan", 0)))
    return fn


# which recorded SDPA output each call of the script is graded against (None: intermediate chained call)
EXPECT = ["g_torch_out", "g_torch_out", "g_torch_out", "V", "g_torch_out", "g_torch_out", None, None, "g_torch_out",
          "g_torch_out_1d", "g_torch_out_2d", "g_torch_out_2d"]


def test_fixture_shape(golden):
    calls = golden_calls(golden)
    assert [c["op"] for c in calls] == ["csr", "coo", "local", "local", "global_no_local", "csr", "local",
                                        "global_no_local", "csr", "local_1d_dilated", "local_2d_dilated",
                                        "local_2d_dilated"]
    assert golden["q"].shape == (L, D)


def test_oracle_matches_reference_script_outputs(orc, golden):
    """Every scenario of verification/verify.py: oracle == the script's SDPA-MATH result."""
    for i, (c, (m, l, O)) in enumerate(_replay(orc, golden, _oracle_call(orc))):
        key = EXPECT[i]
        if key is None:
            continue
        want = golden["v"] if key == "V" else c[key]
        live = ~np.isnan(O).any(axis=1)
        if i == 11:  # use_nan=True: rows without keys are NaN here, 0 in current torch's SDPA
            dead = ~unpack_mask(c["g_mask_2d"], L).any(axis=1)
            assert np.array_equal(~live, dead)
            assert np.all(want[dead] == 0)
        else:
            assert live.all()
        # the script's own bar is allclose(rtol=1e-5, atol=1e-8) in fp32; the oracle is fp64
        np.testing.assert_allclose(O[live], want[live].astype(np.float64), rtol=2e-5, atol=2e-6, err_msg=f"call {i}")


def test_known_answer_identity_window(orc, golden):
    """Local with window 0 attends only to itself: output == V exactly (verify.py:158-177)."""
    q, k, v = golden["q"], golden["k"], golden["v"]
    m, l, O = orc.implicit_forward("local", q, k, v, 0)
    assert np.array_equal(O, v.astype(np.float64))
    assert np.array_equal(l, np.ones(L))


@pytest.mark.parametrize("call,kind,mask_key", [(4, "global_no_local", "g_mask_g"), (9, "local_1d_dilated", "g_mask_1d"),
                                                (10, "local_2d_dilated", "g_mask_2d"), (11, "local_2d_dilated", "g_mask_2d")])
def test_index_sets_equal_reference_mask_builders(orc, golden, call, kind, mask_key):
    """Closed-form index sets == the dense masks built by the script's own loops, bit for bit."""
    c = golden_calls(golden)[call]
    want = unpack_mask(c[mask_key], L)
    G = c.get("G")
    row_off, col = orc.implicit_csr(kind, L, int(c["p0"]), int(c.get("p1", 0)), G=G)
    got = np.zeros((L, L), dtype=bool)
    rows = np.repeat(np.arange(L), np.diff(row_off.astype(np.int64)))
    got[rows, col] = True
    assert got.sum() == len(col), "duplicate (row, key) pairs"
    assert np.array_equal(got, want)
    assert np.array_equal(orc.dense_mask(kind, L, int(c["p0"]), int(c.get("p1", 0)), G=G), want)


@pytest.mark.parametrize("kind,p0,p1", [("local", 0, 0), ("local", 7, 0), ("local", 199, 0), ("local_1d_dilated", 5, 0),
                                         ("local_1d_dilated", 9, 3), ("local_1d_dilated", 199, 6),
                                         ("local_2d_dilated", 8, 0), ("local_2d_dilated", 40, 3),
                                         ("local_2d_dilated", 50, 49), ("global_no_local", 0, 0),
                                         ("global_no_local", 13, 0), ("global_no_local", 199, 0)])
def test_c_oracle_equals_dense_numpy(orc, kind, p0, p1):
    """Two independent restatements (gather-based C, dense numpy) agree on index sets and outputs."""
    Ls, d = 200, 16
    Q, K, V = seeded_qkv(Ls, d, 11)
    G = np.array([5, 0, 150, 199, 77], dtype=np.int32) if kind == "global_no_local" else None
    mask = orc.dense_mask(kind, Ls, p0, p1, G)
    row_off, col = orc.implicit_csr(kind, Ls, p0, p1, G=G)
    got = np.zeros((Ls, Ls), dtype=bool)
    got[np.repeat(np.arange(Ls), np.diff(row_off.astype(np.int64))), col] = True
    assert np.array_equal(got, mask)
    rng = np.random.default_rng(3)
    st = (rng.standard_normal(Ls), rng.random(Ls) + 0.5, rng.standard_normal((Ls, d)))  # a non-trivial incoming state
    a = orc.implicit_forward(kind, Q, K, V, p0, p1, G=G, state=tuple(s.copy() for s in st), use_nan=True)
    b = orc.dense_forward(Q, K, V, mask, state=tuple(s.copy() for s in st), use_nan=(kind == "local_2d_dilated"))
    for x, y in zip(a, b):
        np.testing.assert_allclose(x, y, rtol=1e-12, atol=1e-12, equal_nan=True)


def test_csr_coo_explicit_agree_with_dense(orc):
    Ls, Lk, d = 150, 170, 32
    Q, K, V = seeded_qkv(Ls, d, 5, Lk)
    mask, row_off, col = random_csr(Ls, Lk, 0.05, 9, empty_rows=(0, 17, 149))
    want = orc.dense_forward(Q, K, V, mask, use_nan=True)
    got = orc.csr_forward(Q, K, V, row_off, col, use_nan=True)
    rows = np.repeat(np.arange(Ls, dtype=np.uint64), np.diff(row_off.astype(np.int64)))
    got2 = orc.coo_forward(Q, K, V, rows, col, use_nan=True)
    for x, y, z in zip(got, want, got2):
        np.testing.assert_allclose(x, y, rtol=1e-12, atol=1e-12, equal_nan=True)
        np.testing.assert_array_equal(x, z)
    # row shard of a COO list: rows [40, 90) given the whole list
    sub = orc.coo_forward(Q[40:90], K, V, rows, col, use_nan=True, row_begin=40)
    np.testing.assert_array_equal(sub[2], got[2][40:90])


def test_chained_masks_equal_their_union(orc):
    """State chaining (verify.py:337-352): disjoint masks applied in sequence == one pass over the union."""
    Ls, d, w = 128, 32, 6
    Q, K, V = seeded_qkv(Ls, d, 21)
    G = np.array([3, 64, 100], dtype=np.int32)
    band = orc.dense_mask("local", Ls, w)
    glob = orc.dense_mask("global_no_local", Ls, w, G=G)
    assert not (band & glob).any()
    st = orc.implicit_forward("local", Q, K, V, w)
    st = orc.implicit_forward("global_no_local", Q, K, V, w, G=G, state=st)
    want = orc.dense_forward(Q, K, V, band | glob)
    for x, y in zip(st, want):
        np.testing.assert_allclose(x, y, rtol=1e-12, atol=1e-12)


def test_reference_chunk_walk_defects(orc):
    """ref_mepi mode reproduces which keys the unpatched reference kernels really visit."""
    assert orc.ref_mepi("local", 64) == 46 and orc.ref_mepi("local", 128) == 22 and orc.ref_mepi("local", 32) == 93
    assert orc.ref_mepi("global_no_local", 32) == 92
    # Local, L=65536, w=256, d=64: rows whose key count is an exact >=2x multiple of 46 lose their last chunk
    Lb, w, mepi = 65536, 256, 46
    bad = []
    for i in list(range(0, 600)) + list(range(Lb - 600, Lb)):
        n_true = min(Lb, i + w + 1) - max(0, i - w)
        n_ref = orc.lib().spfa_oracle_row_cols(0, i, Lb, w, 0, None, 0, mepi, None)
        if n_ref != n_true:
            bad.append(i)
            assert n_true % mepi == 0 and n_true - n_ref == mepi
    assert bad == [19, 65, 111, 157, 203, 249] + [Lb - 1 - i for i in (249, 203, 157, 111, 65, 19)]
    # 1D dilated: window base advances by mepi instead of mepi*s -> fewer distinct keys
    cols = np.zeros(2000, dtype=np.uint32)
    n = orc.lib().spfa_oracle_row_cols(1, 5000, 131072, 512, 1, None, 0, 22, cols.ctypes.data)
    assert n == 1025 and len(np.unique(cols[:n])) == 519
