"""Compiles the CUDA library (lib/libapoe.so) and the `hybrid_search` Python module for sm_100a, in-tree."""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC"]
CU_SOURCES = ["apoe_index.cu", "apoe_search.cu", "apoe_build.cu", "apoe_join_tc.cu", "apoe_prep.cu", "apoe_exact.cu", "apoe_files.cpp"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def lib_path() -> str:
    return os.path.join(LIBDIR, "libapoe.so")


def module_path() -> str:
    return os.path.join(HERE, "hybrid_search" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, "apoe_common.cuh"), os.path.join(HERE, "..", "include", "allan_poe.h")]
    objs, procs = [], []
    for src in CU_SOURCES:
        sp = os.path.join(CSRC, src)
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, [sp] + headers):
            cmd = [_nvcc(), *NVCC_FLAGS, *ARCH, "-x", "cu", "-c", sp, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"---- {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    so = lib_path()
    if force or procs or _stale(so, objs):
        subprocess.check_call([_nvcc(), "-shared", *ARCH, "-Xcompiler", "-fPIC", "-o", so, *objs, "-lcudart"])
    mod = module_path()
    mod_src = os.path.join(CSRC, "hybrid_search_py.cpp")
    if force or _stale(mod, [mod_src, so]):
        import pybind11
        inc = [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}"]
        subprocess.check_call(["/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++", "-O2", "-std=c++17", "-shared", "-fPIC",
                               "-fvisibility=hidden", *inc, mod_src, "-o", mod, f"-L{LIBDIR}", "-lapoe",
                               "-Wl,-rpath,$ORIGIN/lib"])
    return so


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(lib_path())
