"""Shared fixtures. Tests marked `gpu` need a B200; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200, sm_100a)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load()


@pytest.fixture(scope="session")
def orc():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "verify_script_L256_d32.npz")
    return np.load(path)


def golden_calls(golden):
    """The recorded forward() calls of the reference's verification script, in order."""
    out = []
    for i in range(int(golden["n_calls"])):
        c = {}
        prefix = f"c{i}_"
        for key in golden.files:
            if key.startswith(prefix):
                c[key[len(prefix):]] = golden[key]
        c["op"] = str(c["op"])
        out.append(c)
    return out


def unpack_mask(bits, L):
    return np.unpackbits(bits, axis=1)[:, :L].astype(bool)


def seeded_qkv(L, d, seed, Lk=None):
    rng = np.random.default_rng(seed)
    Lk = L if Lk is None else Lk
    return (rng.standard_normal((L, d), dtype=np.float32), rng.standard_normal((Lk, d), dtype=np.float32),
            rng.standard_normal((Lk, d), dtype=np.float32))


def random_csr(L, Lk, density, seed, empty_rows=()):
    """eye-union-Bernoulli CSR mask with ascending columns; some rows forced empty."""
    rng = np.random.default_rng(seed)
    mask = rng.random((L, Lk)) < density
    idx = np.arange(min(L, Lk))
    mask[idx, idx] = True
    for r in empty_rows:
        mask[r] = False
    row_off = np.zeros(L + 1, dtype=np.uint64)
    row_off[1:] = np.cumsum(mask.sum(axis=1))
    col = np.nonzero(mask)[1].astype(np.uint32)
    return mask, row_off, col
