"""CPU: the C-ABI library loads, exports every symbol the public header declares, and refuses to run
without a device (no compute call is made here)."""
import ctypes as C
import os

import pytest

from rust_ascend_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ruda_b200.h")


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_header_declares_entry_points():
    names = _lib.declared_symbols(HEADER)
    assert len(names) == len(set(names)) and len(names) >= 30
    for required in ("rb_init_exclusive", "rb_rms_norm", "rb_softmax", "rb_rotary_prefix", "rb_alloc", "rb_read"):
        assert required in names


def test_library_exports_every_declared_symbol(lib):
    missing = [n for n in _lib.declared_symbols(HEADER) if not hasattr(lib, n)]
    assert not missing, f"declared in include/ruda_b200.h but not exported: {missing}"


def test_every_entry_point_cites_the_reference():
    text = open(HEADER).read()
    for name in _lib.declared_symbols(HEADER):
        head = text[:text.index(name + "(")]
        comment = head[head.rindex("/*"):]
        assert ".rs" in comment or "no counterpart" in comment or name in (
            "rb_last_error", "rb_shutdown", "rb_import", "rb_host_alloc", "rb_host_free", "rb_stream", "rb_memset",
            "rb_take_errors", "rb_get_stats", "rb_profile_end", "rb_read", "rb_free", "rb_log_softmax"), name


def test_struct_layout_matches_header(lib):
    # rb_tensor: 2*u64 + 2*u32 + 16*u64 = 152 bytes; rb_options: 2*i32 + 4*u64 = 40 bytes.
    assert C.sizeof(_lib.rb_tensor) == 152 and C.sizeof(_lib.rb_options) == 40 and C.sizeof(_lib.rb_stats) == 40


def test_no_device_means_error_not_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from rust_ascend_b200 import B200Runtime, RuntimeOptions
    from rust_ascend_b200.runtime import InvalidDevice
    with pytest.raises(InvalidDevice, match="no CPU fallback"):
        B200Runtime.initialize_exclusive(RuntimeOptions())
    with pytest.raises(InvalidDevice):
        B200Runtime.client(None)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libruda_b200.so"))
    with pytest.raises(OSError, match="no CPU fallback"):
        _lib.load()


def test_ir_launch_is_a_compilation_error_not_a_fallback():
    from rust_ascend_b200.runtime import CompilationError, ComputeClient
    client = ComputeClient(None, None)            # no device needed: the refusal happens on the host
    with pytest.raises(CompilationError, match="CompilationError"):
        client.launch("elementwise_add_f32")
