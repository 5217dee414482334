"""Compile the reference's own six CUDA extensions for sm_100a, from the sources where they lie.

TEST INFRASTRUCTURE ONLY (side-by-side comparator and the benchmark's reference arm). Nothing is
copied: nvcc/g++ read the reference tree directly (its location: environment variable SPFA_REFERENCE_DIR) and
write only into oracle/_ref/ (git-ignored). The sources are compiled unmodified; ref_shim.h is
force-included to make one dispatch macro accept the argument the reference passes.

Modules are named ref_spfa_<mask> so they never shadow the product's spfa_<mask> modules.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REFERENCE = os.environ.get("SPFA_REFERENCE_DIR", "/root/reference")

FOLDERS = {
    "csr": "Sparse_FlashAttention_CSR",
    "coo": "Sparse_FlashAttention_COO",
    "local": "Sparse_FlashAttention_Local",
    "local_1d_dilated": "Sparse_FlashAttention_Local_1D_Dilated",
    "local_2d_dilated": "Sparse_FlashAttention_Local_2D_Dilated",
    "global_no_local": "Sparse_FlashAttention_Global_No_Local",
}


def module_path(mask: str) -> str:
    return os.path.join(OUT, f"ref_spfa_{mask}" + sysconfig.get_config_var("EXT_SUFFIX"))


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout[-4000:])


def build_one(mask: str, force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    folder = os.path.join(REFERENCE, FOLDERS[mask])
    cpp = os.path.join(folder, f"sp_flatt_{mask}.cpp")
    cu = os.path.join(folder, f"sp_flatt_{mask}_kernel.cu")
    out = module_path(mask)
    shim = os.path.join(HERE, "ref_shim.h")
    if not force and os.path.exists(out) and all(os.path.getmtime(s) <= os.path.getmtime(out) for s in (cpp, cu, shim)):
        return out
    os.makedirs(OUT, exist_ok=True)
    name = f"ref_spfa_{mask}"
    inc = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        inc += ["-I", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    o_cu = os.path.join(OUT, name + "_kernel.o")
    o_cpp = os.path.join(OUT, name + "_binding.o")
    _run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-c", "-Xcompiler", "-fPIC",
          "-w", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
          "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr", "-include", shim, *defs, *inc,
          cu, "-o", o_cu])
    _run(["g++", "-O2", "-std=c++17", "-c", "-fPIC", "-w", *defs, *inc, cpp, "-o", o_cpp])
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    tmp = out + f".tmp{os.getpid()}"
    _run(["g++", "-shared", o_cu, o_cpp, "-o", tmp, "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu",
          "-ltorch_cuda", "-ltorch", "-ltorch_python", "-L", "/usr/local/cuda/lib64", "-lcudart_static", "-lrt",
          "-lpthread", "-ldl", f"-Wl,-rpath,{torch_lib}"])
    os.replace(tmp, out)
    for o in (o_cu, o_cpp):
        os.remove(o)
    return out


def build_all(force: bool = False) -> dict:
    if not os.path.isdir(REFERENCE):
        raise FileNotFoundError(f"reference tree not found at {REFERENCE}")
    with ThreadPoolExecutor(max_workers=min(6, os.cpu_count() or 1)) as ex:
        return dict(zip(FOLDERS, ex.map(lambda m: build_one(m, force), FOLDERS)))


def load(mask: str):
    """Import ref_spfa_<mask> from oracle/_ref/ (None when it was not built)."""
    import importlib.util

    import torch  # noqa: F401

    path = module_path(mask)
    if not os.path.exists(path):
        return None
    name = f"ref_spfa_{mask}"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[name] = mod
    return mod


if __name__ == "__main__":
    for k, v in build_all(force="--force" in sys.argv).items():
        print(k, v)
