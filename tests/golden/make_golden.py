"""Generate tests/golden/verify_script_L256_d32.npz by running the reference's OWN verification script.

The reference ships no golden vectors; its only test is verification/verify.py, which needs a GPU and
the six compiled modules. This generator runs that script unmodified (read from the reference tree,
its location: environment variable SPFA_REFERENCE_DIR) on CPU tensors with:

  * torch/random seeded, so the run is reproducible;
  * stand-in modules spfa_csr/.../spfa_global_no_local whose forward() is the CPU oracle
    (oracle/spfa_oracle.py) -- the script therefore grades the ORACLE with its own
    "Test Passed/Failed" checks against torch SDPA-MATH, and this generator refuses to write
    fixtures unless every check prints "Test Passed" (one torch-version caveat, see main());
  * every forward() call recorded: operator, arguments (mask arrays, parameters), the state it was
    given, and the script's SDPA-MATH result / dense boolean mask in scope at that moment.

What lands in the fixture therefore comes from the reference's code: its inputs, its mask builders
(verify.py:184-205, 237-259, 376-382, 423-431), its dense `scaled_dot_product_attention` outputs
(verify.py:61-63 etc.). Tests replay the recorded calls through the oracle (CPU) and through the CUDA
library (GPU) and compare with the recorded SDPA outputs.

Run:  python tests/golden/make_golden.py        (needs the reference tree; not needed to run tests)
"""
from __future__ import annotations

import contextlib
import io
import os
import random
import runpy
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REFERENCE = os.environ.get("SPFA_REFERENCE_DIR", "/root/reference")
OUT = os.path.join(HERE, "verify_script_L256_d32.npz")
SEED = 20251125

sys.path.insert(0, ROOT)
from __graft_entry__ import load_oracle  # noqa: E402

orc = load_oracle()
calls: list[dict] = []


def _np(t):
    if t.dtype in (torch.uint64,):
        return t.view(torch.int64).numpy().astype(np.uint64)
    if t.dtype in (torch.uint32,):
        return t.view(torch.int32).numpy().astype(np.uint32)
    return t.detach().numpy()


def _record(op, frame_globals, m, l, O, **args):
    snap = {"op": op, "fresh": bool(torch.isinf(m).all() and (l == 0).all()), **args}
    # the SDPA result and dense mask the script will compare this call against
    for key in ("torch_out", "torch_out_1d", "torch_out_2d", "mask_g", "mask_3", "mask_1d", "mask_2d"):
        v = frame_globals.get(key)
        if isinstance(v, torch.Tensor):
            snap["g_" + key] = v.detach().clone().numpy()
    calls.append(snap)


def _state(m, l, O):
    return (m.double().numpy().copy(), l.double().numpy().copy(), O.double().numpy().copy())


def _write_back(state, m, l, O):
    m.copy_(torch.from_numpy(state[0]).float())
    l.copy_(torch.from_numpy(state[1]).float())
    O.copy_(torch.from_numpy(state[2]).float())
    return O


def _stub(name, fn):
    mod = types.ModuleType(name)
    mod.forward = fn
    sys.modules[name] = mod


def csr_forward(q, k, v, row_off, col, w_val, m, l, O, use_nan):
    _record("csr", sys._getframe(1).f_globals, m, l, O, row_off=_np(row_off), col=_np(col), use_nan=bool(use_nan))
    return _write_back(orc.csr_forward(q.numpy(), k.numpy(), v.numpy(), _np(row_off), _np(col), _state(m, l, O),
                                       use_nan), m, l, O)


def coo_forward(q, k, v, row, col, w_val, m, l, O, use_nan):
    _record("coo", sys._getframe(1).f_globals, m, l, O, row=_np(row), col=_np(col), use_nan=bool(use_nan))
    return _write_back(orc.coo_forward(q.numpy(), k.numpy(), v.numpy(), _np(row), _np(col), _state(m, l, O),
                                       use_nan), m, l, O)


def local_forward(q, k, v, m, l, O, w):
    _record("local", sys._getframe(1).f_globals, m, l, O, p0=int(w))
    return _write_back(orc.implicit_forward("local", q.numpy(), k.numpy(), v.numpy(), w, state=_state(m, l, O)),
                       m, l, O)


def l1d_forward(q, k, v, m, l, O, w, dil):
    _record("local_1d_dilated", sys._getframe(1).f_globals, m, l, O, p0=int(w), p1=int(dil))
    return _write_back(orc.implicit_forward("local_1d_dilated", q.numpy(), k.numpy(), v.numpy(), w, dil,
                                            state=_state(m, l, O)), m, l, O)


def l2d_forward(q, k, v, m, l, O, B, dil, use_nan):
    _record("local_2d_dilated", sys._getframe(1).f_globals, m, l, O, p0=int(B), p1=int(dil), use_nan=bool(use_nan))
    return _write_back(orc.implicit_forward("local_2d_dilated", q.numpy(), k.numpy(), v.numpy(), B, dil,
                                            state=_state(m, l, O), use_nan=use_nan), m, l, O)


def gnl_forward(q, k, v, m, l, O, globs, w):
    _record("global_no_local", sys._getframe(1).f_globals, m, l, O, p0=int(w), G=globs.numpy().astype(np.int32))
    return _write_back(orc.implicit_forward("global_no_local", q.numpy(), k.numpy(), v.numpy(), w,
                                            G=globs.numpy(), state=_state(m, l, O)), m, l, O)


def main():
    _stub("spfa_csr", csr_forward)
    _stub("spfa_coo", coo_forward)
    _stub("spfa_local", local_forward)
    _stub("spfa_local_1d_dilated", l1d_forward)
    _stub("spfa_local_2d_dilated", l2d_forward)
    _stub("spfa_global_no_local", gnl_forward)
    torch.cuda.synchronize = lambda *a, **k: None  # the script synchronises after every call
    torch.Tensor.cuda = lambda self, *a, **k: self  # `torch.Tensor(globs).cuda()` on a CPU-only run
    torch.manual_seed(SEED)
    random.seed(SEED)
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        g = runpy.run_path(os.path.join(REFERENCE, "verification", "verify.py"), run_name="__main__")
    text = buf.getvalue()
    print(text)
    passed, failed = text.count("Test Passed"), text.count("Test Failed")
    # One check cannot pass on a current torch, whatever implements forward(): the last scenario
    # (verify.py:463-505) passes use_nan=True and expects SDPA-MATH to give NaN for rows with no key,
    # but torch >= 2.5 returns 0 there (safe softmax). It is accepted only if that is the whole story:
    # dead rows are NaN on our side and 0 on torch's, and every live row agrees.
    nan_case_ok = False
    if failed == 1 and "Test Failed: The SPFA-Local-2D-Dilated w/NaN" in text:
        live = g["mask_2d"].any(dim=1)
        ours, theirs = g["o_local_2d"], g["torch_out_2d"]
        nan_case_ok = bool(torch.isnan(ours[~live]).all() and (theirs[~live] == 0).all()
                           and torch.allclose(ours[live], theirs[live]))
        print("w/NaN scenario: torch's SDPA gives 0 (not NaN) on key-less rows; live rows agree:", nan_case_ok)
    if (failed and not nan_case_ok) or passed + failed < 12:
        raise SystemExit(f"the reference's script did not pass on the oracle: {passed} passed, {failed} failed")

    out = {"q": g["q"].numpy(), "k": g["k"].numpy(), "v": g["v"].numpy(), "n_calls": np.int64(len(calls)),
           "seed": np.int64(SEED), "script_passed": np.int64(passed)}
    for i, c in enumerate(calls):
        for key, val in c.items():
            if key == "op":
                out[f"c{i}_op"] = np.array(val)
            elif isinstance(val, np.ndarray) and val.dtype == np.bool_:
                out[f"c{i}_{key}"] = np.packbits(val, axis=1)
            elif isinstance(val, np.ndarray):
                out[f"c{i}_{key}"] = val
            else:
                out[f"c{i}_{key}"] = np.int64(val)
    np.savez_compressed(OUT, **out)
    print(f"wrote {OUT}: {len(calls)} calls, {os.path.getsize(OUT)} bytes")


if __name__ == "__main__":
    main()
