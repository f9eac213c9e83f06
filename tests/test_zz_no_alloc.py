"""The allocation-free prologue entry point, checked against the ordinary one.

`sage_prologue_static_ctrl` exists for hosts that are not allowed to allocate device memory at the
point where they run the prologue (a plugin's enqueue step with pre-assigned buffers, a process
under a hard memory cap, a path that cannot afford cudaMalloc's implicit synchronisation): its
scratch is an array built into the library.  The array is shared by all calls on a device and keeps
what the previous call left in it, so the test makes two calls in a row, with different inputs, and
each must reproduce `sage_prologue` bit for bit.  Both calls go through the C-ABI with ctypes; the
only allocations are this test's own input and output tensors.

The file name sorts last on purpose: a run that stops at the first failure has already run every
other test.
"""
import ctypes

import pytest
import torch

from conftest import bytes_equal
from oracle import ref_numerics as R
from sageattention import _native
from sageattention import b200_backend as be

pytestmark = pytest.mark.gpu

KEYS = ("q8", "sq", "k8", "sk", "v8t", "sv", "svp", "S", "mean")


def _buffers(b, h, n, dev):
    bh, n_pad = b * h, be.pad_len(n)
    u8 = dict(dtype=torch.uint8, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    # sentinel-filled so that an entry point that skipped a tensor cannot pass by accident
    return dict(q8=torch.full((bh, n, 128), 0x5A, **u8), sq=torch.full((bh, n), -7.0, **f32),
                k8=torch.full((bh, n_pad, 128), 0x5A, **u8), sk=torch.full((bh, n_pad), -7.0, **f32),
                v8t=torch.full((bh, 128, n_pad), 0x5A, **u8), sv=torch.full((bh, n_pad), -7.0, **f32),
                svp=torch.full((bh, n_pad), -7.0, **f32), S=torch.full((bh,), -7.0, **f32),
                mean=torch.full((bh, 128), -7.0, **f32))


def _call_static(lib, q, k, v, o, smooth, int8, status=None):
    b, h, n, _ = q.shape
    p = lambda t: ctypes.c_void_p(int(t.data_ptr()))
    s3 = lambda t: _native.strides3(t.stride(0), t.stride(1), t.stride(2))
    stream = ctypes.c_void_p(int(torch.cuda.current_stream(q.device).cuda_stream))
    return lib.sage_prologue_static_ctrl(
        p(q), p(k), p(v), p(o["q8"]), p(o["sq"]), p(o["k8"]), p(o["sk"]), p(o["v8t"]), p(o["sv"]),
        p(o["svp"]), p(o["S"]), p(o["mean"]), b, h, n, be.pad_len(n), s3(q), s3(k), s3(v),
        0 if q.dtype == torch.float16 else 1, 0 if int8 else 1, 1 if smooth else 0,
        None if status is None else p(status), stream)


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    lib = _native.load()
    assert lib.sage_prologue_static_ctrl_capacity() == 1 << 20
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cases = [
        (1, 6, 1000, torch.float16, True, 11),     # int8 codes, mean on, a |V| > 448 token
        (2, 3, 333, torch.bfloat16, True, 12),     # e4m3 codes, different shape: stale scratch contents
    ]
    # The caller cannot look inside the built-in scratch, so a wait that ran out is reported in a
    # word of the caller's own: it must stay zero.
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for i, (b, h, n, dtype, smooth, seed) in enumerate(cases):
        q, k, v = R.make_inputs(b, h, n, 128, dtype, seed=seed, k_bias_std=1.0, device=dev)
        v[0, 1, 5] = 20000.0
        int8 = dtype == torch.float16
        want = be.quant_qkv(q, k, v, smooth_k=smooth, int8=int8)        # sage_prologue, caller-owned scratch
        got = _buffers(b, h, n, dev)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = _call_static(lib, q, k, v, got, smooth, int8, status)
        assert rc == 0, lib.sage_last_error()
        torch.cuda.synchronize()
        if i > 0:
            # "allocates nothing", observed from outside: once the first call on the device has
            # resolved the array's address, a call leaves the device's free memory as it found it
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        for key in KEYS:
            assert bytes_equal(got[key], want[key].view(got[key].dtype)), (key, b, h, n)
        assert want["S"].max().item() > 1.0
        assert status.item() == 0
    # and without a status word, as before
    got = _buffers(b, h, n, dev)
    assert _call_static(lib, q, k, v, got, smooth, int8, None) == 0, lib.sage_last_error()
    torch.cuda.synchronize()
    for key in KEYS:
        assert bytes_equal(got[key], want[key].view(got[key].dtype)), key


def test_oversized_shape_is_refused_before_any_launch():
    lib = _native.load()
    b, h, n = 32, 64, 64 * 1024          # 2048 heads: the mean's partial sums alone exceed 1 MiB
    assert lib.sage_prologue_ctrl_bytes(b, h, n) > lib.sage_prologue_static_ctrl_capacity()
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p = ctypes.c_void_p(int(dummy.data_ptr()))
    s3 = _native.strides3(h * n * 128, n * 128, 128)
    rc = lib.sage_prologue_static_ctrl(p, p, p, p, p, p, p, p, p, p, p, p, b, h, n, be.pad_len(n),
                                       s3, s3, s3, 0, 0, 1, None, None)
    assert rc == _native.SAGE_E_UNSUPPORTED
    assert b"control scratch" in lib.sage_last_error()
