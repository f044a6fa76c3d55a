"""CPU-side checks of the C-ABI boundary: the library loads without a GPU and exports every symbol that
include/muillm_b200.h declares; the ctypes prototypes cover exactly that set."""
import os
import re

from muillm_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "muillm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"MUI_API\s+[\w\s\*]+?\b(mui_\w+)\s*\(", text))


def test_header_symbols_are_exported_and_bound():
    declared = _declared_symbols()
    assert len(declared) >= 10
    lib = capi.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported by the library"
    assert declared == set(capi.PROTOTYPES), (declared ^ set(capi.PROTOTYPES))


def test_status_strings_and_version():
    lib = capi.lib()
    assert lib.mui_version() >= 100
    assert lib.mui_status_string(capi.MUI_OK) == b"ok"
    for code in range(1, 6):
        assert len(lib.mui_status_string(code)) > 0


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected on the host before any CUDA call."""
    lib = capi.lib()
    s = lib.mui_linear_forward(None, capi.MUI_F16, 1, 8, 8, None, 0.0, None, 0, None, None, None, None, None, 0)
    assert s == capi.MUI_ERR_INVALID_ARG and b"non-null" in lib.mui_last_error()
    s = lib.mui_linear_forward(None, 7, 1, 8, 8, None, 0.0, 1, 0, None, None, None, 1, 1, 0)
    assert s == capi.MUI_ERR_UNSUPPORTED
    s = lib.mui_linear_forward(None, capi.MUI_F16, 9, 8, 8, None, 0.0, 16, 0, None, None, None, 16, 16, 0)
    assert s == capi.MUI_ERR_UNSUPPORTED and b"1..8" in lib.mui_last_error()
    s = lib.mui_flash_decode(None, capi.MUI_F16, 1, 6, 4, 128, 4, None, 1.0, 16, 16, 16, capi.Strides3(8, 8, 8),
                             None, 16, 256, 1 << 20, 0)
    assert s == capi.MUI_ERR_INVALID_ARG  # Hq not a multiple of Hkv
    assert lib.mui_flash_decode_workspace_bytes(1, 32, 8, 128, 4096) == 4096 + 32 * 64 * 130 * 4
