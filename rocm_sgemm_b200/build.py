"""In-tree build of the B200 SGEMM library with nvcc for sm_100a.

Plays the role of the reference's configure-time code generation + static library build
(rocm_sgemm/CMakeLists.txt:9-63): run the generator on config/gemm_config.json, compile the
generated kernel translation units in parallel, link

    rocm_sgemm_b200/libb200_sgemm.so          the C ABI of include/b200_sgemm.h
    rocm_sgemm_b200/libb200_cublas_wrapper.so the vendor-BLAS comparison column (links cuBLAS)
    rocm_sgemm_b200/bin/gemm_test, gemm_bench, cublas_test, cublas_bench   the C++ harnesses (harness/)

Objects are cached under rocm_sgemm_b200/build/ keyed by a hash of the source, the headers it
includes and the flags, so an unchanged kernel is not recompiled.

    python -m rocm_sgemm_b200.build [--config FILE] [--jobs N] [--verbose]
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
REPO = PKG.parent
CSRC = PKG / "csrc"
GEN = CSRC / "generated"
BUILD = PKG / "build"
LIB = PKG / "libb200_sgemm.so"
CUBLAS_LIB = PKG / "libb200_cublas_wrapper.so"
BIN = PKG / "bin"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-O2"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return exe


def _env():
    # the image exports CC/CXX pointing at a compiler wrapper; nvcc should use the system g++
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    return env


def _digest(paths, flags) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(Path(p).read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _compile(src: Path, deps, flags, verbose=False, ptxas_log: Path | None = None, stem: str | None = None) -> Path:
    BUILD.mkdir(exist_ok=True)
    tag = _digest([src] + list(deps), flags)
    stem = stem or src.stem
    obj = BUILD / f"{stem}.{tag}.o"
    if obj.exists():
        return obj
    for old in BUILD.glob(f"{stem}.*.o"):
        old.unlink()
    cmd = [nvcc()] + flags + ["-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True, env=_env())
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr[-4000:]}")
    if ptxas_log is not None:
        with open(ptxas_log, "a") as f:
            f.write(f"== {src.name}\n{r.stderr}\n")
    if verbose:
        print(f"  compiled {src.name}", flush=True)
    return obj


def generate(config: Path, extra_pairs=None):
    sys.path.insert(0, str(PKG / "config"))
    try:
        import generate_config as g
    finally:
        sys.path.pop(0)
    # drop stale generated sources so that removed variants do not linger
    if GEN.exists():
        for f in GEN.glob("kernel_inst_*.cu"):
            f.unlink()
    return g.generate(str(config), str(GEN), extra_pairs=extra_pairs)


def build_library(config: Path | None = None, jobs: int | None = None, verbose=False, extra_pairs=None,
                  out: Path = LIB) -> Path:
    config = Path(config) if config else PKG / "config" / "gemm_config.json"
    generate(config, extra_pairs)
    sources = [GEN / s for s in (GEN / "sources.txt").read_text().split()]
    kernel_hdr = [CSRC / "sgemm_kernel.cuh", CSRC / "sgemm_ws_kernel.cuh"]
    api_deps = kernel_hdr + [CSRC / "transpose.hpp", CSRC / "config_select.hpp", GEN / "config_table.inc", REPO / "include" / "b200_sgemm.h"]
    jobs = jobs or max(1, (os.cpu_count() or 2))
    BUILD.mkdir(exist_ok=True)
    ptxas_log = BUILD / "ptxas.log"
    work = [(s, kernel_hdr if s.name.startswith("kernel_inst") else []) for s in sources]
    work.append((CSRC / "sgemm_api.cu", api_deps))
    work.append((CSRC / "sgemm_static_scratch.cu", [REPO / "include" / "b200_sgemm.h"]))
    work.append((CSRC / "sgemm_host.cu", [REPO / "include" / "b200_sgemm.h"]))
    work.append((CSRC / "sgemm_tf32x3.cu", kernel_hdr + [CSRC / "transpose.hpp", REPO / "include" / "b200_sgemm.h"]))
    work.append((CSRC / "sgemm_blas.cu", [REPO / "include" / "b200_sgemm.h"]))
    work.append((CSRC / "sgemm_selftest.cu", kernel_hdr + [REPO / "include" / "b200_sgemm.h"]))
    objs = []
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        futs = [ex.submit(_compile, s, d, NVCC_FLAGS, verbose, ptxas_log) for s, d in work]
        for f in futs:
            objs.append(f.result())
    cmd = [nvcc()] + ARCH_FLAGS + ["-shared", "-o", str(out)] + [str(o) for o in objs]
    r = subprocess.run(cmd, capture_output=True, text=True, env=_env())
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    return out


def build_cublas_wrapper(verbose=False) -> Path:
    src = CSRC / "cublas_wrapper.cu"
    obj = _compile(src, [REPO / "include" / "b200_cublas_wrapper.h"], NVCC_FLAGS, verbose)
    cmd = [nvcc()] + ARCH_FLAGS + ["-shared", "-o", str(CUBLAS_LIB), str(obj), "-lcublas"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=_env())
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    return CUBLAS_LIB


def build_harness(verbose=False):
    """gemm_test / gemm_bench: C++ programs over the drop-in header include/rocm_sgemm/gemm.hpp."""
    BIN.mkdir(exist_ok=True)
    outs = []
    hdir = PKG / "harness"
    # cublas_test / cublas_bench: the same sources restricted to the vendor column (the reference's
    # test_rocblas / bench_rocblas targets, test/CMakeLists.txt:11, benchmark/CMakeLists.txt:11)
    for name, srcname, defs in (("gemm_test", "gemm_test", []), ("gemm_bench", "gemm_bench", []),
                                ("cublas_test", "gemm_test", ["-DHARNESS_VENDOR_ONLY"]),
                                ("cublas_bench", "gemm_bench", ["-DHARNESS_VENDOR_ONLY"])):
        src = hdir / f"{srcname}.cu"
        if not src.exists():
            continue
        deps = [p for p in hdir.glob("*.hpp")] + [REPO / "include" / "rocm_sgemm" / "gemm.hpp",
                                                  REPO / "include" / "b200_sgemm.h",
                                                  REPO / "include" / "b200_cublas_wrapper.h"]
        flags = NVCC_FLAGS + defs + ["-I", str(REPO / "include"), "-I", str(hdir), "-Xcompiler", "-fopenmp"]
        obj = _compile(src, deps, flags, verbose, stem=name)
        exe = BIN / name
        cmd = [nvcc()] + ARCH_FLAGS + ["-o", str(exe), str(obj), "-L", str(PKG), "-lb200_sgemm",
                                       "-lb200_cublas_wrapper", "-lcublas", "-Xlinker", "-rpath", "-Xlinker",
                                       "$ORIGIN/..", "-Xcompiler", "-fopenmp"]
        r = subprocess.run(cmd, capture_output=True, text=True, env=_env())
        if r.returncode != 0:
            raise RuntimeError(f"link failed for {name}:\n{r.stderr[-4000:]}")
        outs.append(exe)
    # the tuner's one-trial executable (loads a candidate build of the library with dlopen)
    tsrc = PKG / "config" / "tuner.cpp"
    if tsrc.exists():
        exe = BIN / "tuner"
        tag = BIN / f".tuner.{_digest([tsrc, REPO / 'include' / 'b200_sgemm.h'], [])}"
        if not (exe.exists() and tag.exists()):
            for old in BIN.glob(".tuner.*"):
                old.unlink()
            cmd = [nvcc(), "-O2", "-std=c++17", str(tsrc), "-o", str(exe), "-ldl"]
            r = subprocess.run(cmd, capture_output=True, text=True, env=_env())
            if r.returncode != 0:
                raise RuntimeError(f"tuner build failed:\n{r.stderr[-4000:]}")
            tag.touch()
        outs.append(exe)
    return outs


def build_all(config=None, jobs=None, verbose=False):
    lib = build_library(config, jobs, verbose)
    extras = []
    if (CSRC / "cublas_wrapper.cu").exists():
        extras.append(build_cublas_wrapper(verbose))
        extras += build_harness(verbose)
    return [lib] + extras


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=None)
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    for p in build_all(a.config, a.jobs, a.verbose):
        print(p)


if __name__ == "__main__":
    main()
