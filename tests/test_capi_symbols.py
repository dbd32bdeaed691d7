"""CPU: libttb.so builds, loads, and exports every function that include/ttb.h declares."""
import os
import re

from turbotransformers_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "ttb.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ttb_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_functions():
    names = declared_functions()
    assert len(names) >= 35 and "ttb_linear" in names and "ttb_attention_fwd" in names


def test_library_exports_every_declared_symbol(built):
    lib = _capi.lib()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in ttb.h but not exported by libttb.so"


def test_binding_table_matches_header(built):
    assert sorted(_capi.SIGNATURES) == declared_functions()


def test_version_string(built):
    assert b"sm_100a" in _capi.lib().ttb_version()


def test_null_context_is_rejected_not_crashed(built):
    lib = _capi.lib()
    assert lib.ttb_ctx_sync(None) == _capi.ERR_INVALID
    assert lib.ttb_layernorm(None, 0, None, None, None, None, 1, 8, 1e-12) == _capi.ERR_INVALID
    assert lib.ttb_linear(None, 1, None, 8, None, None, None, 0, 1, 8, 8, 0, None, 8) == _capi.ERR_INVALID
