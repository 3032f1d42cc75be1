"""In-tree build of the native libraries.

Two artefacts are produced next to this package (both git-ignored, both loaded at import time):

* ``paddle_b200/lib/libpd_kernels.so`` — every CUDA kernel of the framework, compiled by ``nvcc`` for
  ``sm_100a`` only, exported through a plain C ABI and loaded with ``ctypes``.
* ``paddle_b200/lib/libpd_runtime.so`` — the host runtime in C++ (flags registry, TCP store, comm
  watchdog, reshard planner, gradient bucketing), also a C ABI.

``nvcc`` cross-compiles without a GPU, so the build can run on a CPU-only machine.  Sources are
recompiled only when they (or a header) are newer than their object file.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or add it to PATH")
    return cand


def _newest_header(d: str) -> float:
    t = 0.0
    for f in os.listdir(d):
        if f.endswith((".h", ".cuh", ".hpp")):
            t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def _compile_one(cmd, src, obj, log_path):
    p = subprocess.run(cmd, capture_output=True, text=True)
    with open(log_path, "w") as f:
        f.write(" ".join(cmd) + "\n" + p.stdout + p.stderr)
    if p.returncode != 0:
        raise RuntimeError(f"compile failed for {src}:\n{p.stdout}\n{p.stderr}")
    return obj


def build_kernels(verbose: bool = False, force: bool = False, debug_bounds: bool = False) -> str:
    """Compile every ``csrc/kernels/*.cu`` for sm_100a and link ``libpd_kernels.so``.  ``debug_bounds`` builds
    ``libpd_kernels_dbg.so`` with ``-DPD_DEBUG_BOUNDS`` instead (coordinate / alignment checks in front of every TMA and
    bulk copy, see ``sm100_prims.cuh``); ``ops._lib`` loads it when ``PD_DEBUG_BOUNDS=1``."""
    kdir = os.path.join(CSRC, "kernels")
    os.makedirs(OBJ_DIR, exist_ok=True)
    if debug_bounds:
        return _build_kernels_variant(kdir, "libpd_kernels_dbg.so", "dbg_", ["-DPD_DEBUG_BOUNDS"], verbose, force)
    out = os.path.join(LIB_DIR, "libpd_kernels.so")
    srcs = sorted(f for f in os.listdir(kdir) if f.endswith(".cu"))
    hdr_t = _newest_header(kdir)
    nvcc = _nvcc()
    jobs, objs = [], []
    for s in srcs:
        src = os.path.join(kdir, s)
        obj = os.path.join(OBJ_DIR, s[:-3] + ".o")
        objs.append(obj)
        if (not force and os.path.exists(obj)
                and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_t)):
            continue
        cmd = [nvcc, *NVCC_FLAGS, "-I", kdir, "-c", src, "-o", obj]
        jobs.append((cmd, src, obj, obj + ".log"))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for fut in [ex.submit(_compile_one, *j) for j in jobs]:
                o = fut.result()
                if verbose:
                    print("compiled", os.path.basename(o), file=sys.stderr)
    if jobs or not os.path.exists(out):
        cmd = [nvcc, "-shared", "-o", out, *objs, "-lcudart", "-gencode", "arch=compute_100a,code=sm_100a"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError("link failed:\n" + p.stdout + p.stderr)
    return out


def _build_kernels_variant(kdir, lib_name, obj_prefix, extra_flags, verbose, force):
    out = os.path.join(LIB_DIR, lib_name)
    srcs = sorted(f for f in os.listdir(kdir) if f.endswith(".cu"))
    hdr_t = _newest_header(kdir)
    nvcc = _nvcc()
    jobs, objs = [], []
    for s in srcs:
        src = os.path.join(kdir, s)
        obj = os.path.join(OBJ_DIR, obj_prefix + s[:-3] + ".o")
        objs.append(obj)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_t):
            continue
        jobs.append(([nvcc, *NVCC_FLAGS, *extra_flags, "-I", kdir, "-c", src, "-o", obj], src, obj, obj + ".log"))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for fut in [ex.submit(_compile_one, *j) for j in jobs]:
                o = fut.result()
                if verbose:
                    print("compiled", os.path.basename(o), file=sys.stderr)
    if jobs or not os.path.exists(out):
        p = subprocess.run([nvcc, "-shared", "-o", out, *objs, "-lcudart", "-gencode", "arch=compute_100a,code=sm_100a"],
                           capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError("link failed:\n" + p.stdout + p.stderr)
    return out


def build_runtime(verbose: bool = False, force: bool = False, sanitize: str | None = None) -> str:
    """Compile ``csrc/runtime/*.cc`` into ``libpd_runtime.so`` (host-only C++).  ``sanitize`` = ``"address"`` or
    ``"thread"`` builds ``libpd_runtime_<sanitize>.so`` with that sanitizer (the reference's ``-DSANITIZER_TYPE``
    builds, CMakeLists.txt:311-378); it is loaded when ``PD_RUNTIME_SANITIZER`` names it and the sanitizer run-time
    is preloaded into the interpreter."""
    if sanitize not in (None, "address", "thread", "undefined"):
        raise ValueError("sanitize must be 'address', 'thread' or 'undefined'")
    rdir = os.path.join(CSRC, "runtime")
    os.makedirs(OBJ_DIR, exist_ok=True)
    tag = f"_{sanitize}" if sanitize else ""
    out = os.path.join(LIB_DIR, f"libpd_runtime{tag}.so")
    srcs = sorted(f for f in os.listdir(rdir) if f.endswith(".cc"))
    if not srcs:
        return ""
    hdr_t = _newest_header(rdir)
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    if sanitize:
        cxx = _sanitizer_toolchain(sanitize)[0]
        if cxx is None:
            raise RuntimeError(f"no installed compiler ships the {sanitize} sanitizer run-time")
    san = [f"-fsanitize={sanitize}", "-g", "-O1", "-fno-omit-frame-pointer"] if sanitize else []
    flags = [f for f in CXX_FLAGS if not (sanitize and f.startswith("-O"))] + san
    jobs, objs = [], []
    for s in srcs:
        src = os.path.join(rdir, s)
        obj = os.path.join(OBJ_DIR, f"rt{tag}_" + s[:-3] + ".o")
        objs.append(obj)
        if (not force and os.path.exists(obj)
                and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_t)):
            continue
        jobs.append(([cxx, *flags, "-I", rdir, "-c", src, "-o", obj], src, obj, obj + ".log"))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for fut in [ex.submit(_compile_one, *j) for j in jobs]:
                fut.result()
    if jobs or not os.path.exists(out):
        p = subprocess.run([cxx, "-shared", "-o", out, *objs, "-pthread", *san[:1]], capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError("link failed:\n" + p.stdout + p.stderr)
    return out


def _sanitizer_toolchain(sanitize: str):
    """(compiler, path of its sanitizer run-time): the first of $CXX, g++ on PATH, /usr/bin/g++ that ships one."""
    name = {"address": "libasan.so", "thread": "libtsan.so", "undefined": "libubsan.so"}[sanitize]
    for cxx in (os.environ.get("CXX"), shutil.which("g++"), "/usr/bin/g++", shutil.which("gcc")):
        if not cxx or not os.path.exists(cxx):
            continue
        p = subprocess.run([cxx, f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip()
        if os.path.isabs(p) and os.path.exists(p):
            return cxx, os.path.realpath(p)
    return None, ""


def sanitizer_runtime_library(sanitize: str) -> str:
    """Path of the sanitizer run-time to put in ``LD_PRELOAD`` of a process that loads the sanitized runtime into
    an unsanitized interpreter ("" when no installed compiler ships it)."""
    return _sanitizer_toolchain(sanitize)[1]


def build_all(verbose: bool = False, force: bool = False):
    return build_kernels(verbose, force), build_runtime(verbose, force)


if __name__ == "__main__":
    if "--debug-bounds" in sys.argv:
        print(build_kernels(verbose=True, force="--force" in sys.argv, debug_bounds=True))
    else:
        k, r = build_all(verbose=True, force="--force" in sys.argv)
        print(k)
        print(r)
