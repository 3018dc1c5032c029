"""CPU-side checks of the C ABI: the library loads and exports every declared entry point."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__
    __graft_entry__.build()
    from heirloom_b200 import _lib
    return _lib.load()


def declared_symbols():
    text = (ROOT / "include" / "heirloom_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hl_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ("hl_ctx_create", "hl_gemm_bf16", "hl_layer_norm_forward", "hl_cross_entropy", "hl_adamw_multi"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing


def test_context_creation_fails_cleanly_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    handle = ctypes.c_void_p()
    rc = lib.hl_ctx_create(0, ctypes.byref(handle))
    assert rc != 0 and not handle.value
    assert b"CUDA" in lib.hl_last_error() or b"device" in lib.hl_last_error()


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    from heirloom_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(_lib.HeirloomError):
        _lib.load()


def test_rust_shim_is_current_and_binds_every_entry_point():
    """`include/heirloom_b200.rs` is generated from the header: regenerating gives the committed file, and its
    `extern "C"` block names every declared entry point (the reference drives this path from Rust)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_rust_shim", ROOT / "include" / "make_rust_shim.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    text = (ROOT / "include" / "heirloom_b200.rs").read_text()
    assert gen.generate() == text
    bound = set(re.findall(r"pub fn (hl_[a-z0-9_]+)\(", text))
    assert bound == set(declared_symbols())
    # the safe layer keeps the names of the reference's wrappers for the ops of the step
    for name in ("layer_norm_forward_f32_buffers", "adamw_update_f32_buffers", "sgd_update_f32_buffer", "concat_i64_buffers",
                 "i64_arange_buffer", "matmul_bf16_tensor_core_rhs_transposed_f32_buffers"):
        assert f"pub fn {name}(" in text
