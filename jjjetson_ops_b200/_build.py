"""In-tree build of the native library and the two pybind11 modules.

``build_all()`` runs nvcc on every source under ``csrc/`` for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``), links ``libjq_b200.so`` next to this file and
builds ``python/q8_1_me*.so`` and ``python/mm_q4_0_q8_1_me*.so`` against it.  nvcc
cross-compiles without a GPU, so this also serves as the "does it build" check.  The
top-level ``CMakeLists.txt`` describes the same targets for CMake users.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libjq_b200.so")
# the range-checked debug build of the same sources (-DJQ_BOUNDS_CHECK): a library of its own, used by one GPU test
CHECK_OBJ_DIR = os.path.join(PKG_DIR, "build_check")
CHECK_LIB_PATH = os.path.join(PKG_DIR, "libjq_b200_check.so")
PY_DIR = os.path.join(PKG_DIR, "python")
INCLUDE_DIR = os.path.join(os.path.dirname(PKG_DIR), "include")

CUDA_SOURCES = [
    "quantize.cu",
    "producers.cu",
    "mmq_generic.cu",
    "mmq_gemv_sm100.cu",
    "mmq_gemm_sm100.cu",
    "mmq_gemm_tc_sm100.cu",
    "mmq_gemm_f16_sm100.cu",
    "jq_capi.cu",
    "ref_compat.cpp",
    "weights_io.cpp",
    "model_q4_0.cpp",
]
HEADERS = ["jq_common.cuh", "tc_common.cuh", os.path.join(INCLUDE_DIR, "jq_b200.h"), os.path.join(INCLUDE_DIR, "jq_weights_io.h"),
           os.path.join(INCLUDE_DIR, "jq_model.h")]
BINDINGS = {"q8_1_me": "q8_1_binding.cpp", "mm_q4_0_q8_1_me": "mm_q4_0_q8_1_binding.cpp"}

NVCC_FLAGS = [*os.environ.get("JQ_EXTRA_NVCC_FLAGS", "").split(),
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build jjjetson_ops_b200")


def _host_cxx() -> str:
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")


def _mtime(path: str) -> float:
    return os.path.getmtime(path) if os.path.exists(path) else 0.0


def _newest_header() -> float:
    return max(_mtime(h if os.path.isabs(h) else os.path.join(CSRC, h)) for h in HEADERS)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def _build_library(lib_path: str, obj_dir: str, extra_flags: list[str], force: bool, verbose: bool) -> None:
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    hdr_time = _newest_header()
    jobs = []
    objs = []
    for src in CUDA_SOURCES:
        src_path = os.path.join(CSRC, src)
        obj = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if force or _mtime(obj) < max(_mtime(src_path), hdr_time):
            jobs.append([nvcc, *NVCC_FLAGS, *extra_flags, "-I", INCLUDE_DIR, "-c", src_path, "-o", obj])
    if jobs:
        if verbose:
            print("[jq build] compiling %d source(s) for sm_100a -> %s" % (len(jobs), os.path.basename(lib_path)), file=sys.stderr)
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(_run, jobs))
    if force or jobs or not os.path.exists(lib_path):
        _run([nvcc, "-shared", "-o", lib_path, *objs, "-gencode", "arch=compute_100a,code=sm_100a"])


def build_check(force: bool = False, verbose: bool = False) -> str:
    """The range-checked debug build; returns the path of ``libjq_b200_check.so``."""
    _build_library(CHECK_LIB_PATH, CHECK_OBJ_DIR, ["-DJQ_BOUNDS_CHECK"], force, verbose)
    return CHECK_LIB_PATH


def build_all(force: bool = False, verbose: bool = False) -> str:
    """Compile what is out of date; returns the path of ``libjq_b200.so``."""
    os.makedirs(PY_DIR, exist_ok=True)
    hdr_time = _newest_header()
    _build_library(LIB_PATH, OBJ_DIR, [], force, verbose)

    import pybind11  # build-time only

    ext = sysconfig.get_config_var("EXT_SUFFIX")
    py_inc = sysconfig.get_paths()["include"]
    for mod, src in BINDINGS.items():
        src_path = os.path.join(CSRC, "bindings", src)
        out = os.path.join(PY_DIR, mod + ext)
        if force or _mtime(out) < max(_mtime(src_path), _mtime(LIB_PATH), hdr_time):
            _run(
                [
                    _host_cxx(), "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
                    "-I", pybind11.get_include(), "-I", py_inc, "-I", INCLUDE_DIR,
                    src_path, "-o", out,
                    "-L", PKG_DIR, "-ljq_b200", "-Wl,-rpath,$ORIGIN/..",
                ]
            )
    return LIB_PATH


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose=True))
    if "--check" in sys.argv:
        print(build_check(force="--force" in sys.argv, verbose=True))
