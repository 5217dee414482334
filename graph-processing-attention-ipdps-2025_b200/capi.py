"""ctypes view of the C ABI (include/spfa_b200.h) for callers that hold torch CUDA tensors.

Every function here is a thin argument marshaller: it checks dtype/device/contiguity, allocates the
workspace the entry point asks for with torch's caching allocator, passes raw device pointers and the
current torch stream, and raises on a non-zero status. No arithmetic happens in Python and there is no
CPU path: if ``lib/libspfa_b200.so`` is missing, loading raises.

Row-range arguments (``row_begin``/``row_end``) select the query rows one GPU works on; Q/m/l/O then
hold only those rows while K/V hold all L rows. The reference API is single-GPU and has no such
argument (README.md:10); with the defaults these calls behave exactly like its ``forward`` functions.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libspfa_b200.so")

OK = 0
PATH_AUTO, PATH_GATHER, PATH_TILED = 0, 1, 2
MASK_KIND = {"local": 0, "local_1d_dilated": 1, "local_2d_dilated": 2, "global_no_local": 3}

# every symbol include/spfa_b200.h declares (checked by the CPU test-suite)
EXPORTS = (
    "spfa_status_string", "spfa_abi_version", "spfa_set_path", "spfa_get_path", "spfa_last_path", "spfa_launch_count", "spfa_last_device_error",
    "spfa_csr_workspace_bytes", "spfa_csr_forward_f32",
    "spfa_coo_workspace_bytes", "spfa_coo_min_workspace_bytes", "spfa_coo_forward_f32",
    "spfa_selftest_wait_limit", "spfa_explicit_plan_bytes", "spfa_csr_plan_build", "spfa_coo_plan_build", "spfa_planned_forward_f32", "spfa_planned_forward_keys_f32", "spfa_planned_forward_parts_f32", "spfa_coo_static_max_rows", "spfa_coo_forward_f32_static",
    "spfa_local_workspace_bytes", "spfa_local_forward_f32",
    "spfa_local_1d_dilated_workspace_bytes", "spfa_local_1d_dilated_forward_f32",
    "spfa_local_2d_dilated_workspace_bytes", "spfa_local_2d_dilated_forward_f32",
    "spfa_global_no_local_workspace_bytes", "spfa_global_no_local_forward_f32",
    "spfa_mask_count", "spfa_mask_fill",
    "spfa_dense_mask_offsets", "spfa_dense_mask_fill", "spfa_bigbird_workspace_bytes", "spfa_bigbird_forward_f32",
    "spfa_local_forward_batched_f32", "spfa_local_1d_dilated_forward_batched_f32", "spfa_local_2d_dilated_forward_batched_f32",
    "spfa_global_no_local_forward_batched_f32", "spfa_csr_forward_batched_f32", "spfa_coo_forward_batched_f32",
    "spfa_csr_forward_16", "spfa_coo_forward_16", "spfa_local_forward_16", "spfa_local_1d_dilated_forward_16",
    "spfa_local_2d_dilated_forward_16", "spfa_global_no_local_workspace_bytes_16", "spfa_global_no_local_forward_16",
    "spfa_csr_workspace_bytes_idx32", "spfa_csr_forward_f32_idx32", "spfa_coo_forward_f32_idx32", "spfa_coo_plan_build_idx32",
)

_lib = None


class SpfaError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"spfa_b200 status {status}: {text}")
        self.status = status


def lib() -> ctypes.CDLL:
    """Load the C-ABI library (once) and declare its signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is not built; run `python {os.path.join(_HERE, 'build.py')}`. "
                          "There is no CPU fallback.")
    L = ctypes.CDLL(LIB_PATH)
    i64, i32, vp, sz = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t
    L.spfa_status_string.restype = ctypes.c_char_p
    L.spfa_status_string.argtypes = [i32]
    L.spfa_abi_version.restype = i32
    L.spfa_set_path.restype = None
    L.spfa_set_path.argtypes = [i32]
    L.spfa_get_path.restype = i32
    L.spfa_last_path.restype = i32
    L.spfa_launch_count.restype = i64
    L.spfa_last_device_error.restype = i32
    L.spfa_csr_workspace_bytes.restype = sz
    L.spfa_csr_workspace_bytes.argtypes = [i64, i64, i64, i32]
    L.spfa_csr_forward_f32.restype = i32
    L.spfa_csr_forward_f32.argtypes = [vp] * 5 + [i64] + [vp] * 3 + [i64, i64, i32, i32, vp, sz, vp]
    L.spfa_coo_workspace_bytes.restype = sz
    L.spfa_coo_workspace_bytes.argtypes = [i64, i64, i64, i32]
    L.spfa_coo_min_workspace_bytes.restype = sz
    L.spfa_coo_min_workspace_bytes.argtypes = [i64]
    L.spfa_coo_forward_f32.restype = i32
    L.spfa_coo_forward_f32.argtypes = [vp] * 5 + [i64] + [vp] * 3 + [i64, i64, i64, i32, i32, vp, sz, vp]
    L.spfa_csr_workspace_bytes_idx32.restype = sz
    L.spfa_csr_workspace_bytes_idx32.argtypes = [i64, i64, i64, i32]
    L.spfa_csr_forward_f32_idx32.restype = i32
    L.spfa_csr_forward_f32_idx32.argtypes = L.spfa_csr_forward_f32.argtypes
    L.spfa_coo_forward_f32_idx32.restype = i32
    L.spfa_coo_forward_f32_idx32.argtypes = L.spfa_coo_forward_f32.argtypes
    L.spfa_coo_plan_build_idx32.restype = i32
    L.spfa_coo_plan_build_idx32.argtypes = [vp, vp, i64, i64, i64, i64, i32, vp, sz, vp]
    L.spfa_csr_forward_16.restype = i32
    L.spfa_csr_forward_16.argtypes = [i32] + [vp] * 5 + [i64] + [vp] * 3 + [i64, i64, i32, i32, vp]
    L.spfa_coo_forward_16.restype = i32
    L.spfa_coo_forward_16.argtypes = [i32] + [vp] * 5 + [i64] + [vp] * 3 + [i64, i64, i64, i32, i32, vp, sz, vp]
    L.spfa_local_forward_16.restype = i32
    L.spfa_local_forward_16.argtypes = [i32] + [vp] * 6 + [i64, i32, i64, i64, i64, vp]
    L.spfa_local_1d_dilated_forward_16.restype = i32
    L.spfa_local_1d_dilated_forward_16.argtypes = [i32] + [vp] * 6 + [i64, i32, i64, i64, i64, i64, vp]
    L.spfa_local_2d_dilated_forward_16.restype = i32
    L.spfa_local_2d_dilated_forward_16.argtypes = [i32] + [vp] * 6 + [i64, i32, i64, i64, i32, i64, i64, vp]
    L.spfa_global_no_local_workspace_bytes_16.restype = sz
    L.spfa_global_no_local_workspace_bytes_16.argtypes = [i64, i64]
    L.spfa_global_no_local_forward_16.restype = i32
    L.spfa_global_no_local_forward_16.argtypes = [i32] + [vp] * 7 + [i64, i64, i32, i64, i64, i64, vp, sz, vp]
    L.spfa_local_forward_batched_f32.restype = i32
    L.spfa_local_forward_batched_f32.argtypes = [vp] * 6 + [i64, i64, i32, i64, i64, i64, vp, sz, vp]
    L.spfa_local_1d_dilated_forward_batched_f32.restype = i32
    L.spfa_local_1d_dilated_forward_batched_f32.argtypes = [vp] * 6 + [i64, i64, i32, i64, i64, i64, i64, vp, sz, vp]
    L.spfa_local_2d_dilated_forward_batched_f32.restype = i32
    L.spfa_local_2d_dilated_forward_batched_f32.argtypes = [vp] * 6 + [i64, i64, i32, i64, i64, i32, i64, i64, vp, sz, vp]
    L.spfa_global_no_local_forward_batched_f32.restype = i32
    L.spfa_global_no_local_forward_batched_f32.argtypes = [vp] * 6 + [i64, vp, i64, i64, i32, i64, i64, i64, vp, sz, vp]
    L.spfa_csr_forward_batched_f32.restype = i32
    L.spfa_csr_forward_batched_f32.argtypes = [vp] * 5 + [i64] + [vp] * 3 + [i64, i64, i64, i32, i32, vp, sz, vp]
    L.spfa_coo_forward_batched_f32.restype = i32
    L.spfa_coo_forward_batched_f32.argtypes = [vp] * 5 + [i64] + [vp] * 3 + [i64, i64, i64, i64, i32, i32, vp, sz, vp]
    L.spfa_bigbird_workspace_bytes.restype = sz
    L.spfa_bigbird_workspace_bytes.argtypes = [i64, i64, i32, i64, i64]
    L.spfa_bigbird_forward_f32.restype = i32
    L.spfa_bigbird_forward_f32.argtypes = [vp] * 7 + [i64, vp, vp, i64, i64, i32, i64, i64, i64, vp, sz, vp]
    L.spfa_dense_mask_offsets.restype = i32
    L.spfa_dense_mask_offsets.argtypes = [vp, i64, i64, vp, vp]
    L.spfa_dense_mask_fill.restype = i32
    L.spfa_dense_mask_fill.argtypes = [vp, i64, i64, vp, vp, vp, vp]
    L.spfa_explicit_plan_bytes.restype = sz
    L.spfa_explicit_plan_bytes.argtypes = [i64, i64, i64, i32]
    L.spfa_csr_plan_build.restype = i32
    L.spfa_csr_plan_build.argtypes = [vp, vp, i64, i64, i64, i32, vp, sz, vp]
    L.spfa_coo_plan_build.restype = i32
    L.spfa_coo_plan_build.argtypes = [vp, vp, i64, i64, i64, i64, i32, vp, sz, vp]
    L.spfa_planned_forward_f32.restype = i32
    L.spfa_planned_forward_f32.argtypes = [vp] * 6 + [i64, i64, i64, i32, i32, vp, sz, vp]
    L.spfa_planned_forward_keys_f32.restype = i32
    L.spfa_planned_forward_keys_f32.argtypes = [vp] * 6 + [i64, i64, i64, i32, i32, vp, sz, i64, i64, vp]
    L.spfa_planned_forward_parts_f32.restype = i32
    L.spfa_planned_forward_parts_f32.argtypes = [vp] * 6 + [i64, i64, i64, i32, i32, vp, sz, i64, i64, i32, vp]
    L.spfa_coo_static_max_rows.restype = i64
    L.spfa_coo_forward_f32_static.restype = i32
    L.spfa_coo_forward_f32_static.argtypes = [vp] * 5 + [i64] + [vp] * 3 + [i64, i64, i64, i32, i32, vp]
    for name in ("spfa_local", "spfa_local_1d_dilated", "spfa_local_2d_dilated"):
        f = getattr(L, name + "_workspace_bytes")
        f.restype = sz
        f.argtypes = [i64, i64, i32]
    L.spfa_local_forward_f32.restype = i32
    L.spfa_local_forward_f32.argtypes = [vp] * 6 + [i64, i32, i64, i64, i64, vp, sz, vp]
    L.spfa_local_1d_dilated_forward_f32.restype = i32
    L.spfa_local_1d_dilated_forward_f32.argtypes = [vp] * 6 + [i64, i32, i64, i64, i64, i64, vp, sz, vp]
    L.spfa_local_2d_dilated_forward_f32.restype = i32
    L.spfa_local_2d_dilated_forward_f32.argtypes = [vp] * 6 + [i64, i32, i64, i64, i32, i64, i64, vp, sz, vp]
    L.spfa_global_no_local_workspace_bytes.restype = sz
    L.spfa_global_no_local_workspace_bytes.argtypes = [i64, i64, i32, i64]
    L.spfa_global_no_local_forward_f32.restype = i32
    L.spfa_global_no_local_forward_f32.argtypes = [vp] * 7 + [i64, i64, i32, i64, i64, i64, vp, sz, vp]
    L.spfa_mask_count.restype = i32
    L.spfa_mask_count.argtypes = [i32, i64, i64, i64, vp, i64, i64, i64, vp, vp]
    L.spfa_mask_fill.restype = i32
    L.spfa_mask_fill.argtypes = [i32, i64, i64, i64, vp, i64, i64, i64, vp, vp, vp]
    _lib = L
    return L


def status_string(status: int) -> str:
    return lib().spfa_status_string(status).decode()


def check(status: int) -> None:
    if status != OK:
        raise SpfaError(status, status_string(status))


def set_path(path: int) -> None:
    lib().spfa_set_path(path)


def get_path() -> int:
    return lib().spfa_get_path()


def last_path() -> int:
    return lib().spfa_last_path()


def last_device_error() -> int:
    """Synchronise and return (then clear) the tiled kernels' error word; 0 means no bounded wait gave up."""
    return int(lib().spfa_last_device_error())


def selftest_wait_limit(device=None) -> None:
    """Launch the wait-limit self-test (see include/spfa_b200.h); last_device_error() returns 9001 afterwards."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        lib().spfa_selftest_wait_limit.restype = ctypes.c_int
        lib().spfa_selftest_wait_limit.argtypes = [ctypes.c_void_p]
        check(lib().spfa_selftest_wait_limit(_stream(dev)))


def launch_count() -> int:
    return int(lib().spfa_launch_count())


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _f32(*ts):
    dev = ts[0].device
    for t in ts:
        if not t.is_cuda:
            raise SpfaError(-1, "tensors must be CUDA tensors (there is no CPU path)")
        if t.dtype != torch.float32 or not t.is_contiguous() or t.device != dev:
            raise SpfaError(-1, "floating tensors must be contiguous float32 on one device")
    return dev


def workspace(nbytes: int, dev) -> tuple[torch.Tensor | None, ctypes.c_void_p | None, int]:
    """A 256-byte aligned scratch buffer from torch's caching allocator (kept alive by the caller)."""
    if nbytes == 0:
        return None, None, 0
    buf = torch.empty(nbytes + 256, dtype=torch.uint8, device=dev)
    p = (buf.data_ptr() + 255) & ~255
    return buf, ctypes.c_void_p(p), nbytes


def _as_u64(t):
    if t.dtype not in (torch.uint64, torch.int64, torch.int32) or not t.is_contiguous():
        raise SpfaError(-1, "row offsets/indices must be contiguous torch.uint64 (or int64, or int32)")
    return t


def _idx32(t) -> bool:
    """Row offsets / row indices stored as 32-bit integers take the *_idx32 entry points."""
    return t.dtype == torch.int32


def _as_u32(t):
    if t.dtype not in (torch.uint32, torch.int32) or not t.is_contiguous():
        raise SpfaError(-1, "column indices must be contiguous torch.uint32 (or int32)")
    return t


def csr_forward(Q, K, V, row_off, col_ind, m, l, O, use_nan=False):
    """Rows of Q attend to K/V rows col_ind[row_off[r]:row_off[r+1]]. Q may be a row shard; row_off then
    holds that shard's n_rows+1 offsets (indexing col_ind as passed)."""
    dev = _f32(Q, K, V, m, l, O)
    with torch.cuda.device(dev):
        n_rows, d = Q.shape
        nnz = col_ind.shape[0]
        if _idx32(row_off):
            buf, wp, wb = workspace(lib().spfa_csr_workspace_bytes_idx32(n_rows, nnz, K.shape[0], d), dev)
            check(lib().spfa_csr_forward_f32_idx32(_ptr(Q), _ptr(K), _ptr(V), _ptr(_as_u64(row_off)), _ptr(_as_u32(col_ind)),
                                                   nnz, _ptr(m), _ptr(l), _ptr(O), n_rows, K.shape[0], d, int(use_nan),
                                                   wp, wb, _stream(dev)))
            return O
        buf, wp, wb = workspace(lib().spfa_csr_workspace_bytes(n_rows, nnz, K.shape[0], d), dev)
        if KEEP_LAST_CSR_WORKSPACE:  # diagnostics only: keeps the scratch buffer alive until the next call
            global _last_csr_workspace
            _last_csr_workspace = (buf, wp.value if wp else 0, d)
        check(lib().spfa_csr_forward_f32(_ptr(Q), _ptr(K), _ptr(V), _ptr(_as_u64(row_off)), _ptr(_as_u32(col_ind)),
                                         nnz, _ptr(m), _ptr(l), _ptr(O), n_rows, K.shape[0], d, int(use_nan), wp,
                                         wb, _stream(dev)))
    return O


_last_csr_workspace = None
KEEP_LAST_CSR_WORKSPACE = False  # set True to make last_csr_dense_tiles() meaningful (tests do)


def last_csr_dense_tiles() -> int:
    """Diagnostics: how many (row block, key tile) pairs the most recent csr_forward call of this process ran on
    the tiled kernel (0 if it took the gather path). Synchronises."""
    if not _last_csr_workspace or _last_csr_workspace[0] is None or last_path() != PATH_TILED:
        return 0
    buf, p, d = _last_csr_workspace
    off = p - buf.data_ptr()
    words = int(buf[off:off + 8].view(torch.int64).item())  # the plan's mask pool counter sits first
    return words // (2 * 128)  # 64-key tiles: two 32-bit mask words per row


def coo_forward(Q, K, V, row_ind, col_ind, m, l, O, use_nan=False, row_begin=0):
    """Row-sorted COO mask. Q holds rows [row_begin, row_begin+Q.shape[0]); (row_ind, col_ind) must contain
    every entry of those rows (entries of other rows are ignored)."""
    dev = _f32(Q, K, V, m, l, O)
    with torch.cuda.device(dev):
        n_rows, d = Q.shape
        buf, wp, wb = workspace(lib().spfa_coo_workspace_bytes(n_rows, row_ind.shape[0], K.shape[0], d), dev)
        fn = lib().spfa_coo_forward_f32_idx32 if _idx32(row_ind) else lib().spfa_coo_forward_f32
        check(fn(_ptr(Q), _ptr(K), _ptr(V), _ptr(_as_u64(row_ind)), _ptr(_as_u32(col_ind)),
                                         row_ind.shape[0], _ptr(m), _ptr(l), _ptr(O), row_begin, n_rows, K.shape[0],
                                         d, int(use_nan), wp, wb, _stream(dev)))
    return O


class ExplicitPlan:
    """Inspector output for one CSR/COO mask (device memory), reusable across forward calls on that mask."""

    def __init__(self, buf, ptr, nbytes, n_rows, nnz, n_keys, d):
        self.buf, self.ptr, self.nbytes = buf, ptr, nbytes
        self.n_rows, self.nnz, self.n_keys, self.d = n_rows, nnz, n_keys, d


def _new_plan(n_rows, nnz, n_keys, d, dev):
    need = lib().spfa_explicit_plan_bytes(n_rows, nnz, n_keys, d)
    if need == 0:
        raise SpfaError(-1, "no dense-tile plan for this shape (d must be 32, 64 or 128 and the mask non-empty)")
    buf, wp, wb = workspace(need, dev)
    return ExplicitPlan(buf, wp, wb, n_rows, nnz, n_keys, d)


def _reuse_or_new(out, n_rows, nnz, n_keys, d, dev):
    if out is None:
        return _new_plan(n_rows, nnz, n_keys, d, dev)
    if (out.n_rows, out.nnz, out.n_keys, out.d) != (n_rows, nnz, n_keys, d):
        raise SpfaError(-1, "`out` was allocated for another shape")
    return out


def csr_plan(row_off, col_ind, n_keys, d, out: ExplicitPlan | None = None):
    """Run the inspector once for a CSR mask of row_off.numel()-1 rows over n_keys keys. `out`: an earlier plan of
    the same shape whose memory is refilled instead of allocating (callers that re-inspect every step)."""
    dev = col_ind.device
    with torch.cuda.device(dev):
        plan = _reuse_or_new(out, row_off.shape[0] - 1, col_ind.shape[0], n_keys, d, dev)
        check(lib().spfa_csr_plan_build(_ptr(_as_u64(row_off)), _ptr(_as_u32(col_ind)), plan.nnz, plan.n_rows, n_keys, d,
                                        plan.ptr, plan.nbytes, _stream(dev)))
    return plan


def coo_plan(row_ind, col_ind, n_rows, n_keys, d, row_begin=0, out: ExplicitPlan | None = None):
    """Run the inspector once for the rows [row_begin, row_begin + n_rows) of a row-sorted COO mask (`out` as in
    csr_plan)."""
    dev = col_ind.device
    with torch.cuda.device(dev):
        plan = _reuse_or_new(out, n_rows, col_ind.shape[0], n_keys, d, dev)
        fn = lib().spfa_coo_plan_build_idx32 if _idx32(row_ind) else lib().spfa_coo_plan_build
        check(fn(_ptr(_as_u64(row_ind)), _ptr(_as_u32(col_ind)), plan.nnz, row_begin, n_rows, n_keys, d, plan.ptr,
                 plan.nbytes, _stream(dev)))
    return plan


def planned_forward(Q, K, V, m, l, O, plan: ExplicitPlan, use_nan=False):
    """Forward from a stored plan: dense tiles on the tiled kernel, the other entries on the gather kernel."""
    dev = _f32(Q, K, V, m, l, O)
    if Q.shape[0] != plan.n_rows or K.shape[0] != plan.n_keys or Q.shape[1] != plan.d:
        raise SpfaError(-1, "the plan was built for another shape")
    with torch.cuda.device(dev):
        check(lib().spfa_planned_forward_f32(_ptr(Q), _ptr(K), _ptr(V), _ptr(m), _ptr(l), _ptr(O), plan.n_rows, plan.nnz,
                                             plan.n_keys, plan.d, int(use_nan), plan.ptr, plan.nbytes, _stream(dev)))
    return O


PLAN_DENSE_TILES, PLAN_RESIDUAL = 1, 2


def planned_forward_parts(Q, K, V, m, l, O, plan: ExplicitPlan, key_begin: int, key_end: int, parts: int, use_nan=False):
    """planned_forward_keys for the dense tiles (PLAN_DENSE_TILES), the residual entries (PLAN_RESIDUAL) or both."""
    dev = _f32(Q, K, V, m, l, O)
    if Q.shape[0] != plan.n_rows or K.shape[0] != plan.n_keys or Q.shape[1] != plan.d:
        raise SpfaError(-1, "the plan was built for another shape")
    with torch.cuda.device(dev):
        check(lib().spfa_planned_forward_parts_f32(_ptr(Q), _ptr(K), _ptr(V), _ptr(m), _ptr(l), _ptr(O), plan.n_rows,
                                                   plan.nnz, plan.n_keys, plan.d, int(use_nan), plan.ptr, plan.nbytes,
                                                   int(key_begin), int(key_end), int(parts), _stream(dev)))
    return O


def planned_forward_keys(Q, K, V, m, l, O, plan: ExplicitPlan, key_begin: int, key_end: int, use_nan=False):
    """One pass of a forward split along the key axis: the plan's dense tiles and residual entries whose key lies in
    [key_begin, key_end). Only those K/V rows are read, so a pass can run as soon as its chunk of K/V is on the device."""
    dev = _f32(Q, K, V, m, l, O)
    if Q.shape[0] != plan.n_rows or K.shape[0] != plan.n_keys or Q.shape[1] != plan.d:
        raise SpfaError(-1, "the plan was built for another shape")
    with torch.cuda.device(dev):
        check(lib().spfa_planned_forward_keys_f32(_ptr(Q), _ptr(K), _ptr(V), _ptr(m), _ptr(l), _ptr(O), plan.n_rows,
                                                  plan.nnz, plan.n_keys, plan.d, int(use_nan), plan.ptr, plan.nbytes,
                                                  int(key_begin), int(key_end), _stream(dev)))
    return O


def bigbird_forward(Q, K, V, m, l, O, global_inds, local_size_each_dir, row_off=None, col_ind=None, row_begin=0,
                    row_end=None):
    """Local(w) + Global-no-local(global_inds, w) + an optional disjoint CSR part (row_off/col_ind of the rows
    [row_begin, row_end)) in one call: what the reference composes from three chained forward calls."""
    dev = _f32(Q, K, V, m, l, O)
    L, row_end = _rows(Q, K, row_begin, row_end)
    if global_inds.dtype != torch.int32 or not global_inds.is_contiguous() or global_inds.device != dev:
        raise SpfaError(-1, "global_inds must be a contiguous torch.int32 tensor on Q's device")
    nnz = 0 if col_ind is None else col_ind.shape[0]
    with torch.cuda.device(dev):
        d, nG = Q.shape[1], global_inds.shape[0]
        buf, wp, wb = workspace(lib().spfa_bigbird_workspace_bytes(L, Q.shape[0], d, nG, nnz), dev)
        check(lib().spfa_bigbird_forward_f32(_ptr(Q), _ptr(K), _ptr(V), _ptr(m), _ptr(l), _ptr(O),
                                             _ptr(global_inds) if nG else None, nG,
                                             _ptr(_as_u64(row_off)) if nnz else None, _ptr(_as_u32(col_ind)) if nnz else None,
                                             nnz, L, d, int(local_size_each_dir), row_begin, row_end, wp, wb, _stream(dev)))
    return O


def forward_batched(kind, Q, K, V, m, l, O, *, p0=0, p1=0, global_inds=None, row_off=None, row_ind=None, col_ind=None,
                    use_nan=False, row_begin=0, row_end=None):
    """n_slices attention problems sharing one mask (batch x heads): Q, O [S, rows, d], K, V [S, Lk, d], m, l [S, rows]
    (float32, contiguous). Local and Local-1D-dilated run all slices in one launch; explicit masks are inspected once."""
    dev = _f32(Q, K, V, m, l, O)
    if Q.dim() != 3 or K.dim() != 3 or m.dim() != 2:
        raise SpfaError(-1, "batched tensors are [slices, rows, d] (m, l: [slices, rows])")
    S, n_rows, d = Q.shape
    Lk = K.shape[1]
    with torch.cuda.device(dev):
        st = _stream(dev)
        q, k, v, mm, ll, oo = (_ptr(t) for t in (Q, K, V, m, l, O))
        if kind == "csr":
            nnz = col_ind.shape[0]
            buf, wp, wb = workspace(lib().spfa_csr_workspace_bytes(n_rows, nnz, Lk, d), dev)
            rc = lib().spfa_csr_forward_batched_f32(q, k, v, _ptr(_as_u64(row_off)), _ptr(_as_u32(col_ind)), nnz, mm, ll, oo, S,
                                                    n_rows, Lk, d, int(use_nan), wp, wb, st)
        elif kind == "coo":
            nnz = col_ind.shape[0]
            buf, wp, wb = workspace(lib().spfa_coo_workspace_bytes(n_rows, nnz, Lk, d), dev)
            rc = lib().spfa_coo_forward_batched_f32(q, k, v, _ptr(_as_u64(row_ind)), _ptr(_as_u32(col_ind)), nnz, mm, ll, oo, S,
                                                    row_begin, n_rows, Lk, d, int(use_nan), wp, wb, st)
        else:
            L = Lk
            row_end = L if row_end is None else row_end
            if n_rows != row_end - row_begin:
                raise SpfaError(-1, "Q must hold rows [row_begin, row_end) of every slice")
            if kind == "local":
                rc = lib().spfa_local_forward_batched_f32(q, k, v, mm, ll, oo, S, L, d, int(p0), row_begin, row_end, None, 0, st)
            elif kind == "local_1d_dilated":
                rc = lib().spfa_local_1d_dilated_forward_batched_f32(q, k, v, mm, ll, oo, S, L, d, int(p0), int(p1), row_begin,
                                                                     row_end, None, 0, st)
            elif kind == "local_2d_dilated":
                rc = lib().spfa_local_2d_dilated_forward_batched_f32(q, k, v, mm, ll, oo, S, L, d, int(p0), int(p1),
                                                                     int(use_nan), row_begin, row_end, None, 0, st)
            elif kind == "global_no_local":
                nG = global_inds.shape[0]
                buf, wp, wb = workspace(lib().spfa_global_no_local_workspace_bytes(L, n_rows, d, nG), dev)
                rc = lib().spfa_global_no_local_forward_batched_f32(q, k, v, mm, ll, oo, S, _ptr(global_inds), nG, L, d,
                                                                    int(p0), row_begin, row_end, wp, wb, st)
            else:
                raise ValueError(kind)
        check(rc)
    return O


DTYPE_CODE = {torch.float16: 1, torch.bfloat16: 2}


def _t16(*ts):
    dev, dt = ts[0].device, ts[0].dtype
    if dt not in DTYPE_CODE:
        raise SpfaError(-1, "16-bit entry points take torch.float16 or torch.bfloat16 tensors")
    for t in ts:
        if not t.is_cuda or t.dtype != dt or not t.is_contiguous() or t.device != dev:
            raise SpfaError(-1, "floating tensors must be contiguous CUDA tensors of one 16-bit dtype on one device")
    return dev, DTYPE_CODE[dt]


def forward_16(kind, Q, K, V, m, l, O, *, p0=0, p1=0, global_inds=None, row_off=None, row_ind=None, col_ind=None,
               use_nan=False, row_begin=0, row_end=None):
    """Native 16-bit forward of one mask family (`kind`: csr, coo, local, local_1d_dilated, local_2d_dilated,
    global_no_local) on float16 / bfloat16 tensors: 16-bit loads and stores, fp32 arithmetic, gather path."""
    dev, code = _t16(Q, K, V, m, l, O)
    n_rows, d = Q.shape
    Lk = K.shape[0]
    with torch.cuda.device(dev):
        st = _stream(dev)
        q, k, v, mm, ll, oo = (_ptr(t) for t in (Q, K, V, m, l, O))
        if kind == "csr":
            rc = lib().spfa_csr_forward_16(code, q, k, v, _ptr(_as_u64(row_off)), _ptr(_as_u32(col_ind)), col_ind.shape[0],
                                           mm, ll, oo, n_rows, Lk, d, int(use_nan), st)
        elif kind == "coo":
            buf, wp, wb = workspace(lib().spfa_coo_min_workspace_bytes(n_rows), dev)
            rc = lib().spfa_coo_forward_16(code, q, k, v, _ptr(_as_u64(row_ind)), _ptr(_as_u32(col_ind)), col_ind.shape[0],
                                           mm, ll, oo, row_begin, n_rows, Lk, d, int(use_nan), wp, wb, st)
        else:
            L, row_end = _rows(Q, K, row_begin, row_end)
            if kind == "local":
                rc = lib().spfa_local_forward_16(code, q, k, v, mm, ll, oo, L, d, int(p0), row_begin, row_end, st)
            elif kind == "local_1d_dilated":
                rc = lib().spfa_local_1d_dilated_forward_16(code, q, k, v, mm, ll, oo, L, d, int(p0), int(p1), row_begin,
                                                            row_end, st)
            elif kind == "local_2d_dilated":
                rc = lib().spfa_local_2d_dilated_forward_16(code, q, k, v, mm, ll, oo, L, d, int(p0), int(p1), int(use_nan),
                                                            row_begin, row_end, st)
            elif kind == "global_no_local":
                nG = global_inds.shape[0]
                buf, wp, wb = workspace(lib().spfa_global_no_local_workspace_bytes_16(L, nG), dev)
                rc = lib().spfa_global_no_local_forward_16(code, q, k, v, mm, ll, oo, _ptr(global_inds) if nG else None, nG,
                                                           L, d, int(p0), row_begin, row_end, wp, wb, st)
            else:
                raise ValueError(kind)
        check(rc)
    return O


def dense_mask_to_csr(mask, coo=False):
    """Dense boolean (or uint8) CUDA mask [n_rows, n_cols] -> (row_off uint64[n_rows+1], col uint32[nnz]) or, with
    coo=True, (row uint64[nnz], col uint32[nnz]): the arrays csr_forward / coo_forward take, columns ascending within
    a row. Two streaming passes over the mask on the GPU; one host synchronisation to learn nnz."""
    if not mask.is_cuda or mask.dim() != 2 or mask.dtype not in (torch.bool, torch.uint8) or not mask.is_contiguous():
        raise SpfaError(-1, "mask must be a contiguous 2-D torch.bool / torch.uint8 CUDA tensor")
    dev = mask.device
    n_rows, n_cols = mask.shape
    with torch.cuda.device(dev):
        row_off = torch.empty(n_rows + 1, dtype=torch.int64, device=dev)
        check(lib().spfa_dense_mask_offsets(_ptr(mask), n_rows, n_cols, _ptr(row_off), _stream(dev)))
        nnz = int(row_off[-1].item())
        col = torch.empty(nnz, dtype=torch.int32, device=dev)
        rows = torch.empty(nnz, dtype=torch.int64, device=dev) if coo else None
        if nnz:
            check(lib().spfa_dense_mask_fill(_ptr(mask), n_rows, n_cols, _ptr(row_off), _ptr(col),
                                             _ptr(rows) if coo else None, _stream(dev)))
    if coo:
        return rows.view(torch.uint64), col.view(torch.uint32)
    return row_off.view(torch.uint64), col.view(torch.uint32)


def _rows(Q, K, row_begin, row_end):
    L = K.shape[0]
    row_end = L if row_end is None else row_end
    if Q.shape[0] != row_end - row_begin:
        raise SpfaError(-1, f"Q must hold rows [row_begin, row_end): {Q.shape[0]} != {row_end - row_begin}")
    return L, row_end


def local_forward(Q, K, V, m, l, O, local_size_each_dir, row_begin=0, row_end=None):
    dev = _f32(Q, K, V, m, l, O)
    L, row_end = _rows(Q, K, row_begin, row_end)
    with torch.cuda.device(dev):
        d = Q.shape[1]
        buf, wp, wb = workspace(lib().spfa_local_workspace_bytes(L, Q.shape[0], d), dev)
        check(lib().spfa_local_forward_f32(_ptr(Q), _ptr(K), _ptr(V), _ptr(m), _ptr(l), _ptr(O), L, d,
                                           int(local_size_each_dir), row_begin, row_end, wp, wb, _stream(dev)))
    return O


def local_1d_dilated_forward(Q, K, V, m, l, O, local_size_each_dir, dil_factor, row_begin=0, row_end=None):
    dev = _f32(Q, K, V, m, l, O)
    L, row_end = _rows(Q, K, row_begin, row_end)
    with torch.cuda.device(dev):
        d = Q.shape[1]
        buf, wp, wb = workspace(lib().spfa_local_1d_dilated_workspace_bytes(L, Q.shape[0], d), dev)
        check(lib().spfa_local_1d_dilated_forward_f32(_ptr(Q), _ptr(K), _ptr(V), _ptr(m), _ptr(l), _ptr(O), L, d,
                                                      int(local_size_each_dir), int(dil_factor), row_begin, row_end,
                                                      wp, wb, _stream(dev)))
    return O


def local_2d_dilated_forward(Q, K, V, m, l, O, block_size, dil_factor, use_nan=False, row_begin=0, row_end=None):
    dev = _f32(Q, K, V, m, l, O)
    L, row_end = _rows(Q, K, row_begin, row_end)
    with torch.cuda.device(dev):
        d = Q.shape[1]
        buf, wp, wb = workspace(lib().spfa_local_2d_dilated_workspace_bytes(L, Q.shape[0], d), dev)
        check(lib().spfa_local_2d_dilated_forward_f32(_ptr(Q), _ptr(K), _ptr(V), _ptr(m), _ptr(l), _ptr(O), L, d,
                                                      int(block_size), int(dil_factor), int(use_nan), row_begin,
                                                      row_end, wp, wb, _stream(dev)))
    return O


def global_no_local_forward(Q, K, V, m, l, O, global_inds, local_size_each_dir, row_begin=0, row_end=None):
    dev = _f32(Q, K, V, m, l, O)
    L, row_end = _rows(Q, K, row_begin, row_end)
    if global_inds.dtype != torch.int32 or not global_inds.is_contiguous() or global_inds.device != dev:
        raise SpfaError(-1, "global_inds must be a contiguous torch.int32 tensor on Q's device")
    with torch.cuda.device(dev):
        d, nG = Q.shape[1], global_inds.shape[0]
        buf, wp, wb = workspace(lib().spfa_global_no_local_workspace_bytes(L, Q.shape[0], d, nG), dev)
        check(lib().spfa_global_no_local_forward_f32(_ptr(Q), _ptr(K), _ptr(V), _ptr(m), _ptr(l), _ptr(O),
                                                     _ptr(global_inds) if nG else None, nG, L, d,
                                                     int(local_size_each_dir), row_begin, row_end, wp, wb,
                                                     _stream(dev)))
    return O


def visited_pairs(kind: str, L: int, p0: int, p1: int = 0, global_inds=None, row_begin=0, row_end=None,
                  device="cuda"):
    """(row_off int64[n_rows+1], col uint32[nnz]) of the (row, key) pairs an implicit mask visits, in
    visiting order, produced on the GPU by the kernels' own column generators."""
    row_end = L if row_end is None else row_end
    n_rows = row_end - row_begin
    dev = torch.device(device)
    with torch.cuda.device(dev):
        counts = torch.zeros(max(n_rows, 1), dtype=torch.int64, device=dev)
        nG = 0 if global_inds is None else global_inds.shape[0]
        check(lib().spfa_mask_count(MASK_KIND[kind], L, int(p0), int(p1), _ptr(global_inds), nG, row_begin, row_end,
                                    _ptr(counts), _stream(dev)))
        row_off = torch.zeros(n_rows + 1, dtype=torch.int64, device=dev)
        row_off[1:] = torch.cumsum(counts[:n_rows], 0)
        nnz = int(row_off[-1].item())
        col = torch.zeros(max(nnz, 1), dtype=torch.uint32, device=dev)
        check(lib().spfa_mask_fill(MASK_KIND[kind], L, int(p0), int(p1), _ptr(global_inds), nG, row_begin, row_end,
                                   _ptr(row_off), _ptr(col), _stream(dev)))
    return row_off, col[:nnz]


def new_state(n_rows: int, d: int, device="cuda"):
    """Initial softmax state the operators expect: m = -inf, l = 0, O = 0."""
    return (torch.full((n_rows,), float("-inf"), dtype=torch.float32, device=device),
            torch.zeros(n_rows, dtype=torch.float32, device=device),
            torch.zeros(n_rows, d, dtype=torch.float32, device=device))
