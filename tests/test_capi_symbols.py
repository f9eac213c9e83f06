"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from sageattention import _native

HEADER = os.path.join(ROOT, "include", "sage_b200.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sage_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert _declared() == sorted(_native.SIGNATURES)


def test_library_exports_every_symbol():
    lib = _native.load()
    for name in _declared():
        assert hasattr(lib, name), name


def test_host_only_entry_points():
    lib = _native.load()
    assert lib.sage_version() >= 100
    assert lib.sage_pad_len(8771) == 8832
    assert lib.sage_pad_len(128) == 128
    assert lib.sage_workspace_bytes(1, 48, 47520) > 3 * 48 * 47520 * 128
    assert lib.sage_workspace_bytes(0, 1, 1) == 0
    offs = (ctypes.c_size_t * 11)()
    assert lib.sage_workspace_layout(1, 2, 300, offs) == 11
    vals = list(offs)
    assert vals == sorted(vals) and all(v % 256 == 0 for v in vals)
    assert lib.sage_prologue_ctrl_bytes(1, 48, 47520) >= 48 * 12


def test_argument_errors_are_reported_before_any_launch():
    lib = _native.load()
    s3 = _native.strides3(1024, 512, 128)
    # null pointers -> SAGE_E_ARG with a message, no CUDA call made
    rc = lib.sage_attention(None, None, None, None, None, 0, 1, 1, 4, s3, s3, s3, s3, 0, -1, 0, 1, 0.1, None)
    assert rc == _native.SAGE_E_ARG
    assert b"workspace" in lib.sage_last_error()
    rc = lib.sage_prologue(*([None] * 13), 1, 1, 4, 128, s3, s3, s3, 0, 0, 1, None)
    assert rc == _native.SAGE_E_ARG
    rc = lib.sage_attn_fwd(*([None] * 8), 0, 1, 4, 128, s3, 0, 0.1, 0, 0, None, None)
    assert rc == _native.SAGE_E_ARG
    with pytest.raises(ValueError):
        _native.check(rc, "sage_attn_fwd")
