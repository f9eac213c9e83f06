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
    # every segment starts on a 256-byte boundary; the status word (entry 10) is a spare word of
    # the control block (entry 9), cleared by the same kernel
    assert vals == sorted(vals) and all(v % 256 == 0 for i, v in enumerate(vals) if i != 10)
    assert vals[9] < vals[10] < vals[9] + 4096 and vals[10] % 4 == 0
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


def test_extended_entry_points_validate_on_the_host():
    """The `_ex` entry points refuse bad shapes with a code and a message before touching CUDA."""
    lib = _native.load()
    s3 = _native.strides3(1024, 512, 128)
    buf = (ctypes.c_char * 4096)()                       # host memory: every call below must stop at validation
    p = ctypes.c_void_p((ctypes.addressof(buf) + 255) // 256 * 256)
    # sizes: the workspace does not depend on head_dim; bad head counts give 0 / an error
    assert lib.sage_workspace_bytes_ex(1, 8, 2, 300, 500) > lib.sage_workspace_bytes_ex(1, 8, 2, 300, 100)
    assert lib.sage_workspace_bytes_ex(1, 8, 3, 300, 300) == 0          # 8 is not a multiple of 3
    assert lib.sage_workspace_bytes_ex(1, 4, 4, 300, 300) >= lib.sage_workspace_bytes(1, 4, 300)
    offs = (ctypes.c_size_t * 13)()
    assert lib.sage_workspace_layout_ex(2, 4, 2, 70, 200, offs) == 13
    vals = list(offs)
    # every segment starts on a 256-byte boundary; the status word (entry 10) is a spare word of
    # the control block (entry 9), cleared by the same kernel
    assert vals == sorted(vals) and all(v % 256 == 0 for i, v in enumerate(vals) if i != 10)
    assert vals[9] < vals[10] < vals[9] + 4096 and vals[10] % 4 == 0
    assert lib.sage_workspace_layout_ex(2, 4, 3, 70, 200, offs) == _native.SAGE_E_ARG

    def attention(hq, hkv, nq, nk, d, causal=0, ws=p, ws_bytes=1 << 40):
        return lib.sage_attention_ex(p, p, p, p, None, ws, ws_bytes, 1, hq, hkv, nq, nk, d,
                                     s3, s3, s3, s3, 0, -1, causal, 1, 0, 0.1, None)

    for d in (0, 4, 12, 136, 256):
        assert attention(2, 2, 16, 16, d) == _native.SAGE_E_UNSUPPORTED
        assert b"head_dim" in lib.sage_last_error()
    assert attention(3, 2, 16, 16, 128) == _native.SAGE_E_ARG
    assert b"multiple" in lib.sage_last_error()
    assert attention(2, 2, 0, 16, 128) == _native.SAGE_E_ARG
    assert attention(2, 2, 16, 16, 128, ws=None) == _native.SAGE_E_ARG
    assert attention(2, 2, 16, 16, 128, ws_bytes=1024) == _native.SAGE_E_WORKSPACE
    assert b"needs" in lib.sage_last_error()
    assert attention(70000, 70000, 16, 16, 128) == _native.SAGE_E_UNSUPPORTED   # grid limit
    # the two-step forms
    rc = lib.sage_prologue_ex(*([None] * 15), 1, 2, 2, 16, 16, 128, 64, s3, s3, s3, 0, 0, 1, None)
    assert rc == _native.SAGE_E_ARG and b"null" in lib.sage_last_error()
    rc = lib.sage_prologue_ex(*([p] * 15), 1, 2, 2, 16, 16, 256, 64, s3, s3, s3, 0, 0, 1, None)
    assert rc == _native.SAGE_E_ARG and b"padded key length" in lib.sage_last_error()


def test_packed_batch_entry_point_validates_on_the_host():
    """`sage_attention_varlen` refuses bad arguments with a code and a message before touching CUDA."""
    lib = _native.load()
    s2 = _native.strides2(512, 128)
    buf = (ctypes.c_char * 4096)()
    p = ctypes.c_void_p((ctypes.addressof(buf) + 255) // 256 * 256)

    def call(cu_q=p, cu_k=p, n_seq=3, hq=4, hkv=2, tq=600, tk=700, mq=300, mk=400, d=128, causal=0,
             ws=p, ws_bytes=1 << 40, strides=s2, scale=0.1):
        return lib.sage_attention_varlen(p, p, p, p, cu_q, cu_k, ws, ws_bytes, n_seq, hq, hkv, tq, tk, mq, mk, d,
                                         strides, strides, strides, strides, 0, -1, causal, 1, scale, None)

    assert call(cu_q=None) == _native.SAGE_E_ARG and b"cu_seqlens" in lib.sage_last_error()
    assert call(cu_k=ctypes.c_void_p(p.value + 2)) == _native.SAGE_E_ARG
    assert call(tq=0) == _native.SAGE_E_ARG
    assert call(mq=601) == _native.SAGE_E_ARG and b"longest" in lib.sage_last_error()
    assert call(tq=1 << 31, mq=300) == _native.SAGE_E_UNSUPPORTED
    assert call(n_seq=0) == _native.SAGE_E_ARG
    assert call(hq=3) == _native.SAGE_E_ARG and b"multiple" in lib.sage_last_error()
    assert call(d=136) == _native.SAGE_E_UNSUPPORTED
    assert call(strides=_native.strides2(516, 128)) == _native.SAGE_E_ARG          # not a multiple of 8
    assert call(ws=None) == _native.SAGE_E_ARG
    assert call(ws_bytes=4096) == _native.SAGE_E_WORKSPACE
    # the workspace is the fixed-length one for n_seq slots of the longest lengths
    need = lib.sage_workspace_bytes_ex(3, 4, 2, 300, 400)
    assert call(ws_bytes=need - 1) == _native.SAGE_E_WORKSPACE
    assert call(causal=1) == _native.SAGE_E_ARG and b"causal" in lib.sage_last_error()   # 300 != 400


def test_attention_shape_rule_is_host_arithmetic():
    """`sage_attention_tiles_per_cta` needs no GPU.  The cases are call sizes on which both shapes
    were timed on a 148-SM part (one-tile / two-tile ms in the comments)."""
    lib = _native.load()
    f = lambda h, n, causal=0, sms=148: lib.sage_attention_tiles_per_cta(1, h, n, causal, sms)
    assert f(48, 47520) == 2            # the headline shape: 60.5 against 61 rounds (45.4 / 43.9 ms)
    assert f(48, 8771) == 2             # 1.764 / 1.766
    assert f(7, 16384) == 1             # 0.911 / 0.961
    assert f(48, 4096) == 1             # 0.394 / 0.414
    assert f(48, 1024) == 1             # 0.042 / 0.048: 192 two-tile CTAs are two rounds, the second nearly empty
    assert f(48, 2048) == 2             # 0.121 / 0.118
    assert f(12, 6400) == 1             # 0.279 / 0.306
    assert f(36, 6400) == 1             # 0.689 / 0.711
    assert f(8, 4096) == 2              # 0.082 / 0.072: resident at once either way
    assert f(1, 32768) == 2             # 0.568 / 0.475
    assert f(48, 128) == 1              # a single query tile per head
    assert f(48, 47520, causal=1) == 2
    assert f(8, 4096, causal=1) == 1    # fewer two-tile CTAs than SMs
    assert f(0, 128) == 0 and f(4, 0) == 0 and f(4, 128, sms=0) == 0
    # more SMs move the thresholds with them
    assert f(48, 1024, sms=96) == 2 and f(48, 1024, sms=192) == 2


def test_vector_accessed_pointers_must_be_aligned():
    """Every pointer the kernels touch with 16-byte accesses is checked on the host: a pointer that
    is only 4-byte aligned is refused before any launch (so these calls cannot fault a device)."""
    lib = _native.load()
    s3 = _native.strides3(1024, 512, 128)
    buf = (ctypes.c_char * 8192)()
    base = (ctypes.addressof(buf) + 255) // 256 * 256
    ok, off = ctypes.c_void_p(base), ctypes.c_void_p(base + 4)

    def prologue(**bad):
        names = ["q", "k", "v", "q8", "sq", "k8", "sk", "v8t", "sv", "svp", "s_fold", "mean", "qm", "vmean", "ctrl"]
        args = [bad.get(n, ok) for n in names]
        return lib.sage_prologue_ex(*args, 1, 2, 2, 16, 16, 128, 128, s3, s3, s3, 0, 0, 1, None)

    for name in ("q", "k", "v", "q8", "k8", "v8t", "sk", "sv", "svp", "vmean", "ctrl"):
        assert prologue(**{name: off}) == _native.SAGE_E_ARG, name
        assert b"16-byte aligned" in lib.sage_last_error(), name

    def attn(**bad):
        names = ["q8", "sq", "k8", "sk", "v8t", "svp", "s_fold", "out", "lse", "qm", "vmean"]
        args = [bad.get(n, ok) for n in names]
        return lib.sage_attn_fwd_ex(*args, 1, 2, 2, 16, 16, 128, 128, s3, 0, 0.1, 0, 0, ok, None)

    for name in ("q8", "k8", "v8t", "sk", "svp", "out", "vmean"):
        assert attn(**{name: off}) == _native.SAGE_E_ARG, name
        assert b"16-byte aligned" in lib.sage_last_error(), name


@pytest.mark.parametrize("scale", [0.0, -0.1, float("inf"), float("-inf"), float("nan")])
def test_sm_scale_must_be_finite_and_positive(scale):
    lib = _native.load()
    s3 = _native.strides3(1024, 512, 128)
    buf = (ctypes.c_char * 4096)()
    p = ctypes.c_void_p((ctypes.addressof(buf) + 255) // 256 * 256)
    rc = lib.sage_attn_fwd(*([p] * 8), 1, 2, 16, 128, s3, 0, scale, 0, 0, p, None)
    assert rc == _native.SAGE_E_ARG
    assert b"sm_scale" in lib.sage_last_error()


def test_static_scratch_entry_point_checks_its_status_pointer():
    lib = _native.load()
    s3 = _native.strides3(1024, 512, 128)
    buf = (ctypes.c_char * 4096)()
    base = (ctypes.addressof(buf) + 255) // 256 * 256
    # shape too large for the built-in scratch: refused before the status pointer is even looked at
    rc = lib.sage_prologue_static_ctrl(*([ctypes.c_void_p(base)] * 12), 32, 64, 65536, 65536, s3, s3, s3, 0, 0, 1,
                                       ctypes.c_void_p(base + 2), None)
    assert rc == _native.SAGE_E_UNSUPPORTED
