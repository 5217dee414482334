"""ctypes/numpy front end of the CPU oracle (spfa_oracle.c) plus an independent dense-numpy restatement.

TEST INFRASTRUCTURE ONLY: the checker the CUDA library is compared against. Nothing in the product
package imports this module; only the tests, the smoke check and the benchmark's CPU-baseline leg do.

Two independent restatements live here so they can be checked against each other and against the
fixtures made from the reference's own verification script (tests/golden/):

* the C library (gather-based, fp64, any size) -- `csr_forward`, `coo_forward`, `implicit_forward`,
  `implicit_csr`;
* `dense_mask(...)` + `dense_forward(...)`: a dense boolean mask built with vectorised closed forms and
  a dense fp64 masked softmax, the numpy twin of the mask builders and the
  `scaled_dot_product_attention(q, k, v, mask)` oracle in verification/verify.py:61-63,184-205,376-382,423-431.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "spfa_oracle.c")
_LIB = os.path.join(_HERE, "_build", "libspfa_oracle.so")

KIND = {"local": 0, "local_1d_dilated": 1, "local_2d_dilated": 2, "global_no_local": 3}
# maskElePerIter families of the reference host code
MEPI_FAMILY = {"csr": 0, "local": 0, "local_1d_dilated": 0, "local_2d_dilated": 0, "coo": 1, "global_no_local": 2}


def build(force: bool = False) -> str:
    """Compile spfa_oracle.c with gcc into oracle/_build/ (no-op when up to date)."""
    if (not force) and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC):
        return _LIB
    os.makedirs(os.path.dirname(_LIB), exist_ok=True)
    tmp = _LIB + f".tmp{os.getpid()}"
    subprocess.check_call(["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", "-o", tmp, _SRC, "-lm"])
    os.replace(tmp, _LIB)
    return _LIB


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        _lib.spfa_oracle_ref_mepi.restype = i64
        _lib.spfa_oracle_ref_mepi.argtypes = [i32, i32]
        _lib.spfa_oracle_row_cols.restype = i64
        _lib.spfa_oracle_row_cols.argtypes = [i32, i64, i64, i64, i64, vp, i64, i64, vp]
        _lib.spfa_oracle_csr_forward.restype = None
        _lib.spfa_oracle_csr_forward.argtypes = [vp] * 8 + [i64, i64, i32, i32, i64]
        _lib.spfa_oracle_coo_forward.restype = None
        _lib.spfa_oracle_coo_forward.argtypes = [vp] * 5 + [i64] + [vp] * 3 + [i64, i64, i64, i32, i32, i64]
        _lib.spfa_oracle_implicit_forward.restype = None
        _lib.spfa_oracle_implicit_forward.argtypes = [i32] + [vp] * 6 + [i64, i32, i64, i64, vp, i64, i32, i64, i64, i64]
        _lib.spfa_oracle_implicit_csr.restype = i64
        _lib.spfa_oracle_implicit_csr.argtypes = [i32, i64, i64, i64, vp, i64, i64, i64, i64, vp, vp]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def ref_mepi(family: str, d: int) -> int:
    """maskElePerIter the unpatched reference uses on a 48 KiB-smem GPU (46 at d=64, 22 at d=128)."""
    return int(lib().spfa_oracle_ref_mepi(MEPI_FAMILY[family], d))


def new_state(n_rows: int, d: int):
    """Initial softmax state: m=-inf, l=0, O=0 (fp64)."""
    return (np.full(n_rows, -np.inf), np.zeros(n_rows), np.zeros((n_rows, d)))


def csr_forward(Q, K, V, row_off, col, state=None, use_nan=False, ref_mepi_=0):
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    n_rows, d = Q.shape
    row_off = np.ascontiguousarray(np.asarray(row_off).astype(np.uint64))
    col = np.ascontiguousarray(np.asarray(col).astype(np.uint32))
    m, l, O = new_state(n_rows, d) if state is None else state
    lib().spfa_oracle_csr_forward(_p(Q), _p(K), _p(V), _p(row_off), _p(col), _p(m), _p(l), _p(O),
                                  n_rows, K.shape[0], d, int(use_nan), int(ref_mepi_))
    return m, l, O


def coo_forward(Q, K, V, row, col, state=None, use_nan=False, row_begin=0, ref_mepi_=0):
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    n_rows, d = Q.shape
    row = np.ascontiguousarray(np.asarray(row).astype(np.uint64))
    col = np.ascontiguousarray(np.asarray(col).astype(np.uint32))
    m, l, O = new_state(n_rows, d) if state is None else state
    lib().spfa_oracle_coo_forward(_p(Q), _p(K), _p(V), _p(row), _p(col), row.shape[0], _p(m), _p(l), _p(O),
                                  int(row_begin), n_rows, K.shape[0], d, int(use_nan), int(ref_mepi_))
    return m, l, O


def implicit_forward(kind: str, Q, K, V, p0, p1=0, G=None, state=None, use_nan=False,
                     row_begin=0, row_end=None, ref_mepi_=0):
    """Q holds rows [row_begin, row_end) only; K, V hold all L rows."""
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    L, d = K.shape
    row_end = L if row_end is None else row_end
    n_rows = row_end - row_begin
    assert Q.shape[0] == n_rows
    Gc = None if G is None else np.ascontiguousarray(np.asarray(G, dtype=np.int32))
    m, l, O = new_state(n_rows, d) if state is None else state
    lib().spfa_oracle_implicit_forward(KIND[kind], _p(Q), _p(K), _p(V), _p(m), _p(l), _p(O), L, d,
                                       int(p0), int(p1), _p(Gc), 0 if Gc is None else Gc.shape[0],
                                       int(use_nan), int(row_begin), int(row_end), int(ref_mepi_))
    return m, l, O


def implicit_csr(kind: str, L, p0, p1=0, G=None, row_begin=0, row_end=None, ref_mepi_=0):
    """Index set of an implicit mask as (row_off uint64[n_rows+1], col uint32[nnz]) in visiting order."""
    row_end = L if row_end is None else row_end
    n_rows = row_end - row_begin
    Gc = None if G is None else np.ascontiguousarray(np.asarray(G, dtype=np.int32))
    nG = 0 if Gc is None else Gc.shape[0]
    row_off = np.zeros(n_rows + 1, dtype=np.uint64)
    nnz = lib().spfa_oracle_implicit_csr(KIND[kind], L, int(p0), int(p1), _p(Gc), nG, row_begin, row_end,
                                         int(ref_mepi_), _p(row_off), None)
    col = np.zeros(max(int(nnz), 1), dtype=np.uint32)
    lib().spfa_oracle_implicit_csr(KIND[kind], L, int(p0), int(p1), _p(Gc), nG, row_begin, row_end,
                                   int(ref_mepi_), _p(row_off), _p(col))
    return row_off, col[: int(nnz)]


def implicit_nnz(kind: str, L, p0, p1=0, G=None, row_begin=0, row_end=None) -> int:
    row_end = L if row_end is None else row_end
    Gc = None if G is None else np.ascontiguousarray(np.asarray(G, dtype=np.int32))
    row_off = np.zeros(row_end - row_begin + 1, dtype=np.uint64)
    return int(lib().spfa_oracle_implicit_csr(KIND[kind], L, int(p0), int(p1), _p(Gc),
                                              0 if Gc is None else Gc.shape[0], row_begin, row_end, 0,
                                              _p(row_off), None))


# ------------------------------------------------------------------------------------------------
# Independent dense numpy restatement (small L only).
# ------------------------------------------------------------------------------------------------
def dense_mask(kind: str, L: int, p0: int, p1: int = 0, G=None) -> np.ndarray:
    """Boolean [L, L] mask, True = attend. Vectorised closed forms of the reference's index sets."""
    i = np.arange(L)[:, None]
    j = np.arange(L)[None, :]
    if kind == "local":  # sp_flatt_local_kernel.cu:24-28
        return np.abs(i - j) <= p0
    if kind == "local_1d_dilated":  # sp_flatt_local_1d_dilated_kernel.cu:25-29,102
        s = p1 + 1
        return (np.abs(i - j) <= p0 * s) & ((i - j) % s == 0)
    if kind == "local_2d_dilated":  # sp_flatt_local_2d_dilated_kernel.cu:26-39,123
        s, B = p1 + 1, p0
        same = (i // B) == (j // B)
        return same & ((i % B) % s == 0) & ((j % B) % s == 0)
    if kind == "global_no_local":  # sp_flatt_global_no_local_kernel.cu:38-64,135-162
        isg = np.zeros(L, dtype=bool)
        isg[np.asarray(G, dtype=np.int64)] = True
        return (isg[:, None] | isg[None, :]) & (np.abs(i - j) > p0)
    raise ValueError(kind)


def dense_forward(Q, K, V, mask, state=None, use_nan=False):
    """fp64 dense masked softmax(QK^T/sqrt(d))V merged into (m, l, O); empty rows untouched / NaN."""
    Q, K, V = (np.asarray(x, dtype=np.float64) for x in (Q, K, V))
    n_rows, d = Q.shape
    m, l, O = new_state(n_rows, d) if state is None else state
    S = (Q @ K.T) / np.sqrt(d)
    S = np.where(mask, S, -np.inf)
    live = mask.any(axis=1)
    with np.errstate(invalid="ignore", over="ignore"):
        mloc = S.max(axis=1)
        m_out = np.maximum(m, mloc)
        P = np.exp(S - np.where(np.isfinite(m_out), m_out, 0.0)[:, None])
        P = np.where(mask, P, 0.0)
        a = l * np.exp(m - m_out)
        a = np.where(np.isnan(a), 0.0, a)
        l_out = a + P.sum(axis=1)
        O_out = (a[:, None] * O + P @ V) / l_out[:, None]
    m2, l2, O2 = m.copy(), l.copy(), O.copy()
    m2[live], l2[live], O2[live] = m_out[live], l_out[live], O_out[live]
    if use_nan:
        O2[~live] = np.nan
    return m2, l2, O2
