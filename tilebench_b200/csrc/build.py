"""Builds the native pieces in-tree.

  libtb200.so        the C-ABI library: every .cu in this folder, compiled by nvcc for sm_100a only
  _tb200_torch*.so   the PyTorch C++ extension that unwraps tensors / the current stream and calls
                     the C ABI (no kernels of its own); linked against libtb200.so with an
                     $ORIGIN rpath so the pair loads from wherever the package lies

Both land in tilebench_b200/lib/.  nvcc cross-compiles, so this runs on a machine without a GPU.
Run `python -m tilebench_b200.csrc.build` (add --force to rebuild, --verbose for ptxas -v output).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB_DIR = PKG / "lib"
OBJ_DIR = PKG / "lib" / "obj"
INCLUDE = PKG.parent / "include"

LIB_NAME = "libtb200.so"
EXT_STEM = "_tb200_torch"

CU_SOURCES = ["api.cu", "comm.cu", "dequant.cu", "gemm_fp8.cu", "gemm_i8.cu", "gemm_plain.cu", "gemm_w4a16.cu", "gemv_w4a16.cu", "gemv_w4a16_ring.cu", "quant.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(str(p.name).encode())
        h.update(Path(p).read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _run(cmd, verbose=False):
    if verbose:
        print("+", " ".join(map(str, cmd)), flush=True)
    res = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"command failed ({res.returncode}): {' '.join(map(str, cmd))}\n{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout, res.stderr, sep="\n", flush=True)
    return res


def existing_sources() -> list[Path]:
    return [CSRC / s for s in CU_SOURCES if (CSRC / s).exists()]


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu to an object (in parallel) and link libtb200.so.  Skips when up to date."""
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    srcs = existing_sources()
    deps = srcs + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    stamp = LIB_DIR / (LIB_NAME + ".sha256")
    out = LIB_DIR / LIB_NAME
    want = _digest(deps)
    if not force and out.exists() and stamp.exists() and stamp.read_text().strip() == want:
        return out
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        _run([_nvcc(), *flags, "-I", INCLUDE, "-c", src, "-o", obj], verbose)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(compile_one, srcs))
    _run([_nvcc(), "-shared", "-o", out, *objs], verbose)  # static cudart: no loader dependency
    stamp.write_text(want)
    return out


def build_variant(tag: str, defines: list[str], sources: list[str], verbose: bool = False) -> Path:
    """libtb200_<tag>.so next to the normal library: the normal objects, with `sources` recompiled with -D<defines>.
    For diagnostic builds (e.g. TB200_ROLE_CYCLES); the product library is never replaced."""
    build_library(verbose=verbose)                      # the other objects come from the normal build
    out = LIB_DIR / f"libtb200_{tag}.so"
    stamp = LIB_DIR / f"libtb200_{tag}.sha256"
    want = _digest(existing_sources() + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))) + " " + " ".join(defines + sources)
    if out.exists() and stamp.exists() and stamp.read_text().strip() == want:
        return out
    var_dir = OBJ_DIR / f"variant_{tag}"
    var_dir.mkdir(parents=True, exist_ok=True)
    flags = NVCC_FLAGS + [f"-D{d}" for d in defines]
    objs = []
    for src in existing_sources():
        if src.name in sources:
            obj = var_dir / (src.stem + ".o")
            _run([_nvcc(), *flags, "-I", INCLUDE, "-c", src, "-o", obj], verbose)
        else:
            obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
    _run([_nvcc(), "-shared", "-o", out, *objs], verbose)
    stamp.write_text(want)
    return out


def extension_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return LIB_DIR / (EXT_STEM + suffix)


def build_extension(force: bool = False, verbose: bool = False) -> Path:
    """Compile torch_binding.cpp with g++ against the installed torch headers."""
    import torch
    from torch.utils import cpp_extension as ce

    lib = build_library(force=force, verbose=verbose)
    src = CSRC / "torch_binding.cpp"
    out = extension_path()
    stamp = LIB_DIR / (EXT_STEM + ".sha256")
    want = _digest([src, INCLUDE / "tb200.h"]) + torch.__version__
    if not force and out.exists() and stamp.exists() and stamp.read_text().strip() == want:
        return out
    inc = []
    for p in ce.include_paths("cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(True):
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"], "-I", INCLUDE]
    torch_lib = Path(torch.__file__).parent / "lib"
    cxx11 = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    cmd = [
        os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared",
        f"-D_GLIBCXX_USE_CXX11_ABI={cxx11}", f"-DTORCH_EXTENSION_NAME={EXT_STEM}",
        "-DTORCH_API_INCLUDE_EXTENSION_H",
        *inc, src, "-o", out,
        "-L", torch_lib, "-L", LIB_DIR, "-L", "/usr/local/cuda/lib64",
        "-ltb200", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}",
    ]
    _run(cmd, verbose)
    stamp.write_text(want)
    return out


def build_all(force: bool = False, verbose: bool = False) -> tuple[Path, Path]:
    lib = build_library(force=force, verbose=verbose)
    ext = build_extension(force=force, verbose=verbose)
    return lib, ext


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "--verbose" in sys.argv
    lib, ext = build_all(force=force, verbose=verbose)
    print(lib)
    print(ext)
