"""In-tree build of the sm_100a library and the six torch-extension bindings.

    python build.py            # build what is out of date
    python build.py --force    # rebuild everything

Outputs (all under lib/, git-ignored):
    libspfa_b200.so                    C-ABI library (nvcc, -gencode arch=compute_100a,code=sm_100a)
    spfa_csr.*.so ... (six modules)    pybind/torch bindings, linked against libspfa_b200.so via $ORIGIN

Only sm_100a is targeted. There is no other backend and no CPU fallback.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
INCLUDE = os.path.join(ROOT, "include")
LIB_SO = os.path.join(LIBDIR, "libspfa_b200.so")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

# module name -> (folder, binding source); names follow the reference's setup.py files
BINDINGS = {
    "spfa_csr": ("Sparse_FlashAttention_CSR", "sp_flatt_csr.cpp"),
    "spfa_coo": ("Sparse_FlashAttention_COO", "sp_flatt_coo.cpp"),
    "spfa_local": ("Sparse_FlashAttention_Local", "sp_flatt_local.cpp"),
    "spfa_local_1d_dilated": ("Sparse_FlashAttention_Local_1D_Dilated", "sp_flatt_local_1d_dilated.cpp"),
    "spfa_local_2d_dilated": ("Sparse_FlashAttention_Local_2D_Dilated", "sp_flatt_local_2d_dilated.cpp"),
    "spfa_global_no_local": ("Sparse_FlashAttention_Global_No_Local", "sp_flatt_global_no_local.cpp"),
    "spfa_bigbird": ("Sparse_FlashAttention_BigBird", "sp_flatt_bigbird.cpp"),  # additive: the fused union of masks
}


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout)


def lib_sources() -> list[str]:
    src = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh", ".h"))]
    return src + [os.path.join(INCLUDE, "spfa_b200.h")]


def _check_band_kernel_registers(ptxas_log: str) -> None:
    """The tiled kernel re-balances registers with setmaxnreg; its budgets assume the allocation the compiler makes
    under the kernel's launch bounds: 128 registers per thread for one-sub-tile shapes, 168 for two. A toolchain that
    assigns fewer would make the library fall back to the gather path at run time: fail the build instead."""
    import re

    want = {"1": 128, "2": 168}
    for m in re.finditer(r"Compiling entry function '(_ZN4spfa4tile19band_forward_kernelILi\d+ELi\d+ELi\d+ELi(\d)E[^']*)'"
                         r".*?Used (\d+) registers", ptxas_log, flags=re.S):
        name, nsub, regs = m.group(1), m.group(2), int(m.group(3))
        if regs != want[nsub]:
            raise RuntimeError(f"{name}: ptxas assigned {regs} registers, the setmaxnreg budgets need {want[nsub]}")


def build_lib(force: bool = False, verbose: bool = False) -> str:
    """nvcc -> lib/libspfa_b200.so (static cudart; driver API reached through cudaGetDriverEntryPoint). Every .cu of
    csrc/ is compiled to an object on its own thread, then the objects are linked."""
    os.makedirs(LIBDIR, exist_ok=True)
    if not force and _newer(LIB_SO, lib_sources()):
        return LIB_SO
    cu = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cu")]
    objdir = os.path.join(LIBDIR, f"obj{os.getpid()}")
    os.makedirs(objdir, exist_ok=True)
    base = ["nvcc", *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "--extended-lambda", "-Xptxas=-v", "-Xcompiler", "-fPIC",
            "-I", INCLUDE]

    def compile_one(src: str) -> tuple[str, str]:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        r = subprocess.run([*base, "-c", src, "-o", obj], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("command failed: nvcc -c " + src + "\n" + r.stdout)
        return obj, r.stdout

    try:
        with ThreadPoolExecutor(max_workers=min(len(cu), os.cpu_count() or 1)) as ex:
            results = list(ex.map(compile_one, cu))
        log = "\n".join(out for _, out in results)
        _check_band_kernel_registers(log)
        if verbose:
            print(log)
        tmp = LIB_SO + f".tmp{os.getpid()}"
        _run(["nvcc", *NVCC_ARCH, "-shared", "-o", tmp, *[o for o, _ in results]])
        os.replace(tmp, LIB_SO)
    finally:
        for f in os.listdir(objdir):
            os.remove(os.path.join(objdir, f))
        os.rmdir(objdir)
    return LIB_SO


def binding_path(name: str) -> str:
    return os.path.join(LIBDIR, name + sysconfig.get_config_var("EXT_SUFFIX"))


def _binding_cmd(name: str, out: str) -> list[str]:
    import torch
    from torch.utils import cpp_extension as ce

    folder, src = BINDINGS[name]
    inc = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"], INCLUDE, os.path.join(HERE, "bindings")]:
        inc += ["-I", p]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-w",
            f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *inc, os.path.join(HERE, folder, src), "-o", out,
            "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-L", LIBDIR, "-lspfa_b200", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]


def build_binding(name: str, force: bool = False) -> str:
    folder, src = BINDINGS[name]
    out = binding_path(name)
    deps = [os.path.join(HERE, folder, src), os.path.join(HERE, "bindings", "binding_common.h"),
            os.path.join(INCLUDE, "spfa_b200.h")]
    if not force and _newer(out, deps):
        return out
    tmp = out + f".tmp{os.getpid()}"
    _run(_binding_cmd(name, tmp))
    os.replace(tmp, out)
    return out


def build_all(force: bool = False, verbose: bool = False) -> dict[str, str]:
    out = {"libspfa_b200": build_lib(force, verbose)}
    with ThreadPoolExecutor(max_workers=min(7, os.cpu_count() or 1)) as ex:
        for name, path in zip(BINDINGS, ex.map(lambda n: build_binding(n, force), BINDINGS)):
            out[name] = path
    return out


if __name__ == "__main__":
    built = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for k, v in built.items():
        print(f"{k}: {v}")
