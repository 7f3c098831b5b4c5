"""The C-ABI library and the PyTorch extension load without a GPU and export every declared symbol."""
import ctypes
import re
from pathlib import Path

import pytest

from tilebench_b200 import native

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "tb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def built():
    from tilebench_b200.csrc import build
    build.build_all()
    return native.capi()


def test_header_and_loader_agree():
    assert declared_symbols() == sorted(native.ABI_SYMBOLS)


def test_library_exports_every_declared_symbol(built):
    for name in declared_symbols():
        assert hasattr(built, name), name


def test_version_and_error_text_without_gpu(built):
    assert built.tb200_abi_version() == 1
    assert built.tb200_last_error() == b"" or isinstance(built.tb200_last_error(), bytes)
    # host-side validation runs before any CUDA call: a null pointer is rejected with a message
    rc = built.tb200_dequant_int4_group(None, None, None, 1, 8, 8, 8, 8, None)
    assert rc == 1 and b"null" in built.tb200_last_error()
    rc = built.tb200_gemm_fp8_blockscaled(None, None, None, None, None, 128, 128, 128, 128, None)
    assert rc == 1
    assert built.tb200_gemm_w4a16_workspace_bytes(4096, 14336, 4096) == 0      # large m: no split-K scratch
    assert built.tb200_gemm_w4a16_workspace_bytes(8, 14336, 4096) == 0         # decode-sized m: never, whatever the group
    # the exchange step and the wait self-test validate on the host too
    assert built.tb200_allgather_cols(None, 8, None, 2, 0, 4, 8, 2, 16, None) == 1
    assert built.tb200_selftest_bounded_wait(0, None) == 1 and b"limit" in built.tb200_last_error()
    assert built.tb200_selftest_bounded_wait(1 << 40, None) == 1


def test_extension_imports_and_mirrors_the_abi(built):
    ext = native.load()
    assert ext.abi_version() == 1
    for fn in ("dequant_int4_group", "dequant_int8_rowwise", "weight_dequant_block", "gemm_fp8_blockscaled",
               "gemm_w4a16", "gemm_w4a16_workspace_bytes", "device_status", "clear_device_status", "check_device"):
        assert hasattr(ext, fn), fn


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(native, "LIB_PATH", tmp_path / "libtb200.so")
    monkeypatch.setattr(native, "_capi", None)
    with pytest.raises(native.NativeLibraryMissing):
        native.capi()


def test_product_code_never_imports_the_oracle():
    for path in (ROOT / "tilebench_b200").rglob("*.py"):
        text = path.read_text()
        assert "import oracle" not in text and "from oracle" not in text, path
