"""CPU: the C-ABI library loads, exports every symbol the header declares, and its host-side argument
validation answers with the documented status codes (no kernel is launched by any call here)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "spfa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(spfa_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(pkg):
    lib = pkg.capi.lib()
    names = _declared_functions()
    assert len(names) >= 19
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/spfa_b200.h but not exported"
    assert sorted(pkg.capi.EXPORTS) == sorted(n for n in names if n != "spfa_status")
    assert lib.spfa_abi_version() >= 1000


def test_bindings_are_built(pkg):
    for name in pkg.MODULES:
        assert os.path.exists(pkg.build.binding_path(name)), name


def test_status_strings_carry_reference_messages(pkg):
    s = pkg.capi.status_string
    assert s(0) == "ok"
    assert "local size specified is either negative" in s(-6)
    assert "dilation factor must be atleast 0" in s(-7)
    assert "divisor of the whole tensor" in s(-8)
    assert "less than the block/window size" in s(-9)
    assert "no global tokens" in s(-10)


def test_path_switch(pkg):
    c = pkg.capi
    c.set_path(c.PATH_GATHER)
    assert c.get_path() == c.PATH_GATHER
    c.set_path(99)  # ignored
    assert c.get_path() == c.PATH_GATHER
    c.set_path(c.PATH_AUTO)
    assert c.get_path() == c.PATH_AUTO


def test_argument_validation_without_gpu(pkg):
    """Validation happens before any CUDA call, in the reference's order of checks."""
    lib = pkg.capi.lib()
    p = ctypes.c_void_p(4096)  # never dereferenced: all these calls fail validation first
    L, d = 1024, 64
    f = lib.spfa_local_forward_f32
    assert f(p, p, p, p, p, p, L, 2048, 5, 0, L, None, 0, None) == -2    # embedded dimension beyond 1024
    assert f(p, p, p, p, p, p, L, 0, 5, 0, L, None, 0, None) == -2
    assert f(p, p, p, p, p, p, L, 48, -1, 0, L, None, 0, None) == -6     # d = 48 is accepted (generic gather kernel)
    assert f(ctypes.c_void_p(4100), p, p, p, p, p, L, 50, -1, 0, L, None, 0, None) == -6  # rows of 50 floats: 4-byte alignment
    assert f(p, p, p, p, p, p, L, d, -1, 0, L, None, 0, None) == -6      # negative window
    assert f(p, p, p, p, p, p, L, d, L, 0, L, None, 0, None) == -6       # window > L-1
    assert f(p, p, p, p, p, p, L, d, 5, 10, 5, None, 0, None) == -1      # bad row range
    assert f(None, p, p, p, p, p, L, d, 5, 0, L, None, 0, None) == -1    # null pointer
    assert f(ctypes.c_void_p(4100), p, p, p, p, p, L, d, 5, 0, L, None, 0, None) == -1  # misaligned
    g = lib.spfa_local_1d_dilated_forward_f32
    assert g(p, p, p, p, p, p, L, d, 5, -1, 0, L, None, 0, None) == -7
    assert g(p, p, p, p, p, p, L, d, L, 1, 0, L, None, 0, None) == -6
    h = lib.spfa_local_2d_dilated_forward_f32
    assert h(p, p, p, p, p, p, L, d, 48, 0, 0, 0, L, None, 0, None) == -8   # 1024 % 48 != 0
    assert h(p, p, p, p, p, p, L, d, 64, -2, 0, 0, L, None, 0, None) == -7
    assert h(p, p, p, p, p, p, L, d, 64, 64, 0, 0, L, None, 0, None) == -9  # 64 / 65 < 1
    q = lib.spfa_global_no_local_forward_f32
    assert q(p, p, p, p, p, p, None, 0, L, d, 5, 0, L, None, 0, None) == -10
    assert q(p, p, p, p, p, p, p, L + 1, L, d, 5, 0, L, None, 0, None) == -10
    assert q(p, p, p, p, p, p, p, 4, L, d, L, 0, L, None, 0, None) == -6
    assert q(p, p, p, p, p, p, p, 4, L, d, 5, 0, L, None, 0, None) == -3    # workspace missing
    assert lib.spfa_global_no_local_workspace_bytes(L, L, d, 4) > 0
    c = lib.spfa_coo_forward_f32
    assert c(p, p, p, p, p, 10, p, p, p, 0, L, L, d, 0, None, 0, None) == -3
    assert lib.spfa_coo_min_workspace_bytes(L) >= 8 * (L + 1)
    assert lib.spfa_coo_workspace_bytes(L, 1000, L, d) == lib.spfa_coo_min_workspace_bytes(L)  # small mask: gather
    big = lib.spfa_coo_workspace_bytes(1 << 20, 1 << 27, 1 << 20, d)   # large mask: room for the dense-tile split
    assert big >= (1 << 27) * 4 + lib.spfa_coo_min_workspace_bytes(1 << 20)
    assert lib.spfa_csr_workspace_bytes(1 << 20, 1 << 27, 1 << 20, 16) == 0          # d = 16 has no tiled path
    assert lib.spfa_csr_forward_f32(p, p, p, None, p, 10, p, p, p, L, L, d, 0, None, 0, None) == -1
    # stored plans: sizes and argument checks (no launch without a GPU)
    need = lib.spfa_explicit_plan_bytes(L, 5000, L, d)
    assert need > lib.spfa_coo_min_workspace_bytes(L) + 4 * 5000
    assert lib.spfa_explicit_plan_bytes(L, 5000, L, 16) == 0 and lib.spfa_explicit_plan_bytes(L, 0, L, d) == 0
    assert lib.spfa_csr_plan_build(p, p, 5000, L, L, d, None, 0, None) == -3         # no plan memory
    assert lib.spfa_csr_plan_build(p, p, 5000, L, L, 16, p, need, None) == -1        # d without a tiled path
    assert lib.spfa_csr_plan_build(p, p, 5000, L, L, 48, p, need, None) == -1        # d = 48: gather path only
    assert lib.spfa_csr_plan_build(p, p, 5000, L, L, 4096, p, need, None) == -2      # d not supported at all
    assert lib.spfa_coo_plan_build(None, p, 5000, 0, L, L, d, p, need, None) == -1
    assert lib.spfa_planned_forward_f32(p, p, p, p, p, p, L, 5000, L, d, 0, p, need - 1, None) == -3


def test_capi_refuses_cpu_tensors(pkg):
    import torch

    c = pkg.capi
    t = torch.zeros(8, 16)
    with pytest.raises(c.SpfaError):
        c.local_forward(t, t, t, torch.zeros(8), torch.zeros(8), t.clone(), 1)


def test_host_pipeline_chunk_planning(pkg):
    """Pure host logic of hostio: chunk edges cover the rows exactly once on unit multiples, and every chunk waits
    for the chunk that holds the last key row it can read."""
    h = pkg.hostio
    for n_rows, n_chunks, unit in ((65536, 8, 256), (3000, 5, 256), (700, 5, 256), (2048, 8, 128), (1, 3, 256), (257, 2, 256)):
        e = h.chunk_edges(n_rows, n_chunks, unit)
        assert e[0] == 0 and e[-1] == n_rows and all(b > a for a, b in zip(e, e[1:]))
        assert all(x % unit == 0 for x in e[:-1]) and len(e) - 1 <= max(1, n_chunks)
        for halo in (0, 1, 255, 256, 1000, 10 ** 6):
            for c in range(len(e) - 1):
                last = h.chunk_needed_last(e, c, halo, n_rows)
                need = min(n_rows, e[c + 1] + halo) - 1
                assert e[last] <= need < e[last + 1] and last >= c
