"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import ctypes


def test_library_exports_every_declared_symbol():
    from nvfp4_training import _native
    handle = _native.lib()
    names = _native.declared_symbols()
    assert "nvfp4_quantize_tile" in names and "nvfp4_dequantize" in names
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in include/nvfp4_b200.h but not exported"
    assert handle.nvfp4_version() >= 1
    assert handle.nvfp4_amax_scratch_bytes() >= 4144


def test_every_bound_signature_is_declared():
    from nvfp4_training import _native
    assert set(_native._SIGNATURES) <= set(_native.declared_symbols())


def test_argument_errors_need_no_gpu():
    from nvfp4_training import _native
    handle = _native.lib()
    rc = handle.nvfp4_amax(None, 0, 4, 4, 4, 1, None, None, None)
    assert rc == 1 and b"null" in handle.nvfp4_last_error()
    buf = ctypes.create_string_buffer(64)
    rc = handle.nvfp4_dequantize(buf, buf, buf, 100, 4, 4, 0, 0, buf, 4, None)
    assert rc == 1
