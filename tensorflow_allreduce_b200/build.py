"""In-tree build of the native library (C++ runtime + sm_100a CUDA kernels).

`python -m tensorflow_allreduce_b200.build` compiles every source under `csrc/` and links
`lib/libbcoll.so` next to the package, so the binary travels with the source tree. The CUDA
runtime is linked statically and driver entry points are looked up at run time, so the library
also loads on machines without a GPU (the CPU collectives and the control plane work there).

Stands where the reference has its Bazel rule `tf_custom_op_library(mpi_collectives.so, ...)`
(tensorflow/contrib/mpi_collectives/BUILD:38-46).
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = LIBDIR / "obj"
LIB = LIBDIR / "libbcoll.so"
LIB_DEBUG = LIBDIR / "libbcoll_debug.so"   # same sources with -DBC_DEBUG: bounds-checked kernels

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.environ.get("NVCC", str(Path(CUDA_HOME) / "bin" / "nvcc"))
CXX = os.environ.get("CXX", "g++")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "--extended-lambda", "-Xcompiler", "-fPIC,-Wall"]
CXX_FLAGS = ["-O2", "-g1", "-fPIC", "-std=c++17", "-Wall", "-pthread", f"-I{CUDA_HOME}/include"]


def _sources():
    cc = sorted(p for p in CSRC.rglob("*.cc") if "selftest" not in p.parts)
    cu = sorted(p for p in CSRC.rglob("*.cu"))
    return cc, cu


def _headers_mtime() -> float:
    hs = list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _obj_for(src: Path, debug: bool = False) -> Path:
    rel = src.relative_to(CSRC)
    return (LIBDIR / "obj_debug" if debug else OBJDIR) / ("_".join(rel.parts) + ".o")


def _compile(src: Path, obj: Path, verbose: bool, extra: list[str]) -> None:
    if src.suffix == ".cu":
        cmd = [NVCC] + NVCC_FLAGS + extra + ["-c", str(src), "-o", str(obj)]
    else:
        cmd = [CXX] + CXX_FLAGS + extra + ["-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stderr.strip() or r.stdout.strip()):
        print(r.stdout, r.stderr, flush=True)


def _fingerprint(debug: bool) -> str:
    """Hash of every source and header and of the compiler flags: what a built library is valid for."""
    import hashlib

    h = hashlib.sha256()
    cc, cu = _sources()
    hs = sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")))
    for p in cc + cu + hs:
        h.update(str(p.relative_to(CSRC)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS + (["-DBC_DEBUG"] if debug else [])).encode())
    return h.hexdigest()


def _stamp(debug: bool) -> Path:
    return LIBDIR / (".fingerprint_debug" if debug else ".fingerprint")


def needs_build(debug: bool = False) -> bool:
    """True when the library is missing or was built from other sources. The record of what it
    was built from is a hash beside it, so a copy or checkout that changes file times neither
    forces a rebuild nor hides an edit; without that record the file times decide."""
    lib = LIB_DEBUG if debug else LIB
    if not lib.exists():
        return True
    stamp = _stamp(debug)
    if stamp.exists():
        return stamp.read_text().strip() != _fingerprint(debug)
    cc, cu = _sources()
    newest = max([p.stat().st_mtime for p in cc + cu] + [_headers_mtime()])
    return newest > lib.stat().st_mtime


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, debug: bool = False) -> Path:
    """Compile what changed and link the shared library. Returns its path. `debug=True` builds the
    bounds-checked variant (`-DBC_DEBUG`, `lib/libbcoll_debug.so`) instead."""
    if shutil.which(NVCC) is None and not Path(NVCC).exists():
        raise RuntimeError(f"nvcc not found at {NVCC}; set CUDA_HOME or NVCC")
    LIB = LIB_DEBUG if debug else globals()["LIB"]
    (LIBDIR / "obj_debug" if debug else OBJDIR).mkdir(parents=True, exist_ok=True)
    cc, cu = _sources()
    hm = _headers_mtime()
    todo = []
    objs = []
    for src in cc + cu:
        obj = _obj_for(src, debug)
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hm):
            todo.append((src, obj))
    extra_cu = (["-Xptxas", "-v"] if ptxas_info else []) + (["-DBC_DEBUG"] if debug else [])
    extra_cc = ["-DBC_DEBUG"] if debug else []
    if todo:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            futs = [ex.submit(_compile, s, o, verbose or ptxas_info, extra_cu if s.suffix == ".cu" else extra_cc) for s, o in todo]
            for f in futs:
                f.result()
    if todo or not LIB.exists() or force:
        tmp = LIB.with_suffix(".so.tmp")
        cmd = [NVCC] + ARCH_FLAGS + ["-shared", "-o", str(tmp)] + [str(o) for o in objs] + ["-lpthread", "-ldl", "-lrt"]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
    _stamp(debug).write_text(_fingerprint(debug) + "\n")
    return LIB


def _sanitizer_cxx(sanitizer: str) -> str:
    """First C++ compiler that can link a program with -fsanitize=<sanitizer> (a toolchain may
    ship without the sanitizer run-time libraries)."""
    import tempfile

    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "probe.cc"
        src.write_text("int main() { return 0; }\n")
        for cxx in dict.fromkeys([CXX, "/usr/bin/g++", "g++", "clang++"]):
            try:
                r = subprocess.run([cxx, f"-fsanitize={sanitizer}", str(src), "-o", str(Path(tmp) / "probe")], capture_output=True)
            except OSError:
                continue
            if r.returncode == 0:
                return cxx
    raise RuntimeError(f"no C++ compiler here can link with -fsanitize={sanitizer}")


def build_selftest(sanitizer: str = "thread", verbose: bool = False) -> Path:
    """Build `csrc/selftest/host_selftest.cc` with the host sources compiled under
    `-fsanitize=<sanitizer>` ("thread" or "address"); CUDA objects are reused from the normal build.
    Returns the executable."""
    build()
    cxx = _sanitizer_cxx(sanitizer)
    outdir = LIBDIR / f"selftest_{sanitizer}"
    outdir.mkdir(parents=True, exist_ok=True)
    cc, cu = _sources()
    cc = [p for p in cc if p.name != "capi.cc"] + [CSRC / "selftest" / "host_selftest.cc"]
    flags = [f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", "-O1", "-g"]
    objs = []

    def one(src):
        obj = outdir / ("_".join(src.relative_to(CSRC).parts) + ".o")
        cmd = [cxx] + [f for f in CXX_FLAGS if f not in ("-O2", "-g1")] + flags + ["-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compiling {src} failed:\n{r.stderr}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(one, cc))
    exe = outdir / "host_selftest"
    cmd = [cxx, f"-fsanitize={sanitizer}", "-o", str(exe)] + [str(o) for o in objs] + [str(_obj_for(s)) for s in cu] + [
        f"-L{CUDA_HOME}/lib64", "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking the self-test failed:\n{r.stderr}")
    return exe


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(prog="python -m tensorflow_allreduce_b200.build", description="Build the native library in-tree.")
    ap.add_argument("--force", action="store_true", help="recompile every source")
    ap.add_argument("-v", "--verbose", action="store_true", help="print the compiler commands")
    ap.add_argument("--ptxas", action="store_true", help="print registers, spills and shared memory of every kernel (-Xptxas -v)")
    ap.add_argument("--debug", action="store_true", help="build the bounds-checked variant (-DBC_DEBUG, lib/libbcoll_debug.so)")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, ptxas_info=a.ptxas, debug=a.debug))
