"""Loads the compiled pieces: the C-ABI library (ctypes) and the PyTorch C++ extension.

There is no fallback.  If a binary is missing, `load()` / `capi()` raise with the build command;
nothing in the cuda backend computes on the CPU.
"""
from __future__ import annotations

import ctypes
import importlib.util
import sys
import sysconfig
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"
LIB_PATH = LIB_DIR / "libtb200.so"
EXT_STEM = "_tb200_torch"

#: Every symbol include/tb200.h declares; tests check the list against the header and the .so.
ABI_SYMBOLS = (
    "tb200_abi_version", "tb200_last_error", "tb200_check_device",
    "tb200_dequant_int4_group", "tb200_dequant_int8_rowwise", "tb200_weight_dequant_block",
    "tb200_gemm_fp8_blockscaled", "tb200_gemm_w4a16_workspace_bytes", "tb200_gemm_w4a16",
    "tb200_device_status", "tb200_clear_device_status",
    "tb200_gemm_w4a16_static_scratch_bytes", "tb200_gemm_w4a16_static", "tb200_gemm_w4a16_gather",
    "tb200_quantize_fp8_block", "tb200_matmul_int8_packed2", "tb200_matmul_plain", "tb200_quantize_int4_group",
    "tb200_allgather_cols", "tb200_selftest_bounded_wait",
)

DT_F32, DT_F16, DT_BF16, DT_F8E4M3 = 0, 1, 2, 3

_ext = None
_capi = None


class NativeLibraryMissing(RuntimeError):
    pass


def _missing(what: Path) -> NativeLibraryMissing:
    return NativeLibraryMissing(
        f"{what} is not built. Run `python -m tilebench_b200.csrc.build` (or __graft_entry__.build()); "
        "the cuda backend has no CPU fallback.")


def extension_path() -> Path:
    return LIB_DIR / (EXT_STEM + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def load():
    """The PyTorch extension module (functions mirror the C ABI, taking tensors)."""
    global _ext
    if _ext is not None:
        return _ext
    import torch  # noqa: F401  (the extension links against libtorch)
    path = extension_path()
    if not path.exists() or not LIB_PATH.exists():
        raise _missing(path if not path.exists() else LIB_PATH)
    spec = importlib.util.spec_from_file_location(EXT_STEM, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[EXT_STEM] = mod
    import torch
    if torch.cuda.is_available():
        mod.check_device()      # sm_100 only: refuse here, not with a "no kernel image" error at the first launch
    _ext = mod
    return mod


def capi() -> ctypes.CDLL:
    """The C-ABI library with argument types declared, for callers that hold raw device pointers."""
    global _capi
    if _capi is not None:
        return _capi
    if not LIB_PATH.exists():
        raise _missing(LIB_PATH)
    lib = ctypes.CDLL(str(LIB_PATH))
    vp, i64, ci, cf, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    lib.tb200_abi_version.restype = ci
    lib.tb200_last_error.restype = ctypes.c_char_p
    lib.tb200_check_device.restype = ci
    lib.tb200_dequant_int4_group.argtypes = [vp, vp, vp, i64, i64, i64, ci, i64, vp]
    lib.tb200_dequant_int8_rowwise.argtypes = [vp, vp, vp, i64, i64, ci, ci, cf, vp]
    lib.tb200_weight_dequant_block.argtypes = [vp, vp, vp, i64, i64, i64, ci, vp]
    lib.tb200_gemm_fp8_blockscaled.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp]
    lib.tb200_gemm_w4a16_workspace_bytes.argtypes = [i64, i64, i64]
    lib.tb200_gemm_w4a16_workspace_bytes.restype = sz
    lib.tb200_gemm_w4a16.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, ci, i64, i64, vp, sz, vp]
    lib.tb200_gemm_w4a16_static_scratch_bytes.argtypes = []
    lib.tb200_gemm_w4a16_static_scratch_bytes.restype = sz
    lib.tb200_gemm_w4a16_static.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, ci, i64, i64, vp]
    lib.tb200_gemm_w4a16_static.restype = ci
    lib.tb200_gemm_w4a16_gather.argtypes = [vp, vp, vp, ctypes.POINTER(vp), ci, ci, i64, i64, i64, i64, ci, i64, vp]
    lib.tb200_gemm_w4a16_gather.restype = ci
    lib.tb200_quantize_fp8_block.argtypes = [vp, vp, vp, i64, i64, ci, vp]
    lib.tb200_quantize_fp8_block.restype = ci
    lib.tb200_matmul_int8_packed2.argtypes = [vp, vp, vp, i64, i64, i64, i64, vp]
    lib.tb200_matmul_int8_packed2.restype = ci
    lib.tb200_matmul_plain.argtypes = [vp, vp, vp, i64, i64, i64, ci, i64, vp]
    lib.tb200_matmul_plain.restype = ci
    lib.tb200_quantize_int4_group.argtypes = [vp, vp, vp, i64, i64, i64, ci, vp]
    lib.tb200_quantize_int4_group.restype = ci
    lib.tb200_allgather_cols.argtypes = [vp, i64, ctypes.POINTER(vp), ci, ci, i64, i64, i64, i64, vp]
    lib.tb200_allgather_cols.restype = ci
    lib.tb200_selftest_bounded_wait.argtypes = [i64, vp]
    lib.tb200_selftest_bounded_wait.restype = ci
    lib.tb200_device_status.argtypes = [ctypes.POINTER(ci), ctypes.POINTER(ci)]
    lib.tb200_clear_device_status.argtypes = []
    for name in ("tb200_dequant_int4_group", "tb200_dequant_int8_rowwise", "tb200_weight_dequant_block",
                 "tb200_gemm_fp8_blockscaled", "tb200_gemm_w4a16", "tb200_device_status",
                 "tb200_clear_device_status"):
        getattr(lib, name).restype = ci
    _capi = lib
    return lib


def last_error() -> str:
    return capi().tb200_last_error().decode()


def require_b200() -> None:
    """Raise unless the current device is sm_100.  load() makes the same check once when a GPU is present;
    callers that switch devices afterwards call this again."""
    load().check_device()


def device_status() -> tuple[int, int]:
    """(code, detail) of the kernels' bounded-wait status word; synchronises the device."""
    return tuple(load().device_status())


def clear_device_status() -> None:
    load().clear_device_status()
