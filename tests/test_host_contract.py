"""Host-side contract of the drop-in package: signatures, acceptance rule, refusals (CPU only)."""
import inspect
import os

import pytest
import torch

import sageattention
from sageattention import b200_backend as be


def _t(*shape, dtype=torch.float16):
    return torch.zeros(*shape, dtype=dtype)


def test_public_names_and_signature():
    for name in ("sageattn", "sageattn_qk_int8_pv_fp8", "sageattn_qk_int8_pv_fp8_cuda",
                 "sageattn_qk_int8_pv_fp8_cuda_sm90"):
        assert callable(getattr(sageattention, name))
    sig = inspect.signature(sageattention.sageattn)
    names = list(sig.parameters)
    assert names[:10] == ["q", "k", "v", "tensor_layout", "is_causal", "sm_scale", "return_lse",
                          "sk1_backend", "sk1_int8", "sk1_bf16"]
    # callers probe for an attn_mask parameter; there must be none
    assert "attn_mask" not in sig.parameters
    assert sig.parameters["tensor_layout"].default == "HND"
    assert sig.parameters["is_causal"].default is False
    up = inspect.signature(sageattention.sageattn_qk_int8_pv_fp8)
    assert up.parameters["smooth_k"].default is True
    assert up.parameters["qk_quant_gran"].default == "per_thread"
    assert up.parameters["pv_accum_dtype"].default == "fp32+fp16"


def test_attn_mask_and_backend_switch_are_refused():
    q = _t(1, 1, 4, 128)
    with pytest.raises(NotImplementedError):
        sageattention.sageattn(q, q, q, attn_mask=torch.ones(4, 4))
    with pytest.raises(ValueError, match="no CPU path"):      # return_lse is served, CPU tensors are not
        sageattention.sageattn(q, q, q, return_lse=True)
    with pytest.raises(ValueError, match="no CPU path"):      # smooth_v is served too
        sageattention.sageattn(q, q, q, smooth_v=True)
    with pytest.raises(NotImplementedError):
        sageattention.sageattn(q, q, q, sk1_backend=False)
    with pytest.warns(UserWarning, match="smooth_v will be ignored"):     # upstream rule for two-level accumulators
        with pytest.raises(ValueError, match="no CPU path"):
            sageattention.sageattn_qk_int8_pv_fp8(q, q, q, smooth_v=True)
    with pytest.raises(ValueError):
        sageattention.sageattn_qk_int8_pv_fp8(q, q, q, qk_quant_gran="per_block")


def test_cpu_tensors_raise_no_fallback():
    q = _t(1, 1, 4, 128)
    with pytest.raises(ValueError, match="no CPU path"):
        sageattention.sageattn(q, q, q)


def test_strided_view_reasons_in_order():
    ok = _t(2, 3, 16, 128)
    assert be.strided_view_reason(ok) is None
    assert be.strided_view_reason(_t(3, 16, 128)) == "rank"
    assert be.strided_view_reason(ok.transpose(2, 3)) == "stride_last"
    assert be.strided_view_reason(_t(1, 1, 16, 128).expand(2, 3, 16, 128)) == "stride_nonpos"
    odd = torch.zeros(2 * 3 * 16 * 132, dtype=torch.float16).as_strided((2, 3, 16, 128), (3 * 16 * 132, 16 * 132, 132, 1))
    assert be.strided_view_reason(odd) == "stride_align"
    off = torch.zeros(2 * 3 * 16 * 128 + 8, dtype=torch.float16)[4:].as_strided((2, 3, 16, 128), (3 * 16 * 128, 16 * 128, 128, 1))
    assert be.strided_view_reason(off) == "ptr_align"
    overlap = torch.zeros(4096, dtype=torch.float16).as_strided((1, 2, 16, 128), (4096, 64 * 8, 128, 1))
    assert be.strided_view_reason(overlap) == "stride_overlap"


def test_accepted_views():
    # physical NHD read as HND, and a fused-QKV view whose row stride is 3*H*D
    nhd = _t(2, 16, 3, 128).transpose(1, 2)
    assert be.strided_view_reason(nhd) is None
    fused = _t(2, 16, 3, 3 * 128)
    qv = fused[..., :128].transpose(1, 2)
    assert be.strided_view_reason(qv) is None
    # unsqueeze(0) gives B=1 a small batch stride; size-1 dims are ignored by the overlap rule
    one = _t(3, 16, 128).unsqueeze(0)
    assert be.strided_view_reason(one) is None


@pytest.mark.parametrize("mutate,reason", [
    (lambda q, k, v: (q, k, v.float()), "dtype"),
    (lambda q, k, v: (q.float(), k.float(), v.float()), "dtype"),
    (lambda q, k, v: (q[..., :64], k[..., :64], v[..., :64]), None),      # head_dim 64 view of wider rows
    (lambda q, k, v: (q[..., :60], k[..., :60], v[..., :60]), "head_dim"),   # not a multiple of 8
    (lambda q, k, v: (q[..., :64], k, v), "head_dim"),
    (lambda q, k, v: (q, k[:, :, :8], v), "seq_len"),                     # K and V lengths differ
    (lambda q, k, v: (q, k[:, :, :8], v[:, :, :8]), None),                # a shorter K/V is served
    (lambda q, k, v: (q, k[:, :1], v[:, :1]), None),                      # 2 query heads per K/V head
    (lambda q, k, v: (q[:, :1], k, v), "heads"),                          # fewer query heads than K/V heads
    (lambda q, k, v: (q, k[:, :1], v), "heads"),
    (lambda q, k, v: (q, k[:1], v[:1]), "batch"),
])
def test_envelope_reasons(mutate, reason):
    q, k, v = _t(2, 2, 16, 128), _t(2, 2, 16, 128), _t(2, 2, 16, 128)
    q, k, v = mutate(q, k, v)
    assert be.envelope_reason(q, k, v, "HND", require_cuda=False) == reason


def test_envelope_layout_and_flags():
    q = _t(1, 1, 4, 128)
    assert be.envelope_reason(q, q, q, "HDN", require_cuda=False) == "layout"
    assert be.envelope_reason(q, q, q, "HND", return_lse=True, require_cuda=False) is None
    assert be.envelope_reason(q, q, q, "HND", attn_mask=q, require_cuda=False) == "attn_mask"
    assert be.envelope_reason(q, q, q, "HND", require_cuda=True) == "device"
    assert be.envelope_reason(q, q, q, "NHD", require_cuda=False) is None
    d64, d136 = _t(1, 1, 4, 64), _t(1, 1, 4, 136)
    assert be.envelope_reason(d64, d64, d64, "HND", require_cuda=False) is None
    assert be.envelope_reason(d136, d136, d136, "HND", require_cuda=False) == "head_dim"


def test_varlen_argument_checks():
    q = _t(10, 2, 128)
    cu = torch.tensor([0, 4, 10], dtype=torch.int32)
    with pytest.raises(ValueError, match="packed"):
        sageattention.sageattn_varlen(q.unsqueeze(0), q, q, cu, cu, 6, 6)
    with pytest.raises(ValueError, match="int32 or int64"):
        sageattention.sageattn_varlen(q, q, q, cu.float(), cu, 6, 6)
    with pytest.raises(ValueError, match="do not match"):
        sageattention.sageattn_varlen(q, q, q, torch.tensor([0, 4, 9]), cu, 6, 6)
    with pytest.raises(ValueError, match="max_seqlen"):
        sageattention.sageattn_varlen(q, q, q, cu, cu, 5, 6)
    with pytest.raises(ValueError, match="no CPU path"):
        sageattention.sageattn_varlen(q, q, q, cu, cu, 6, 6)


def test_packed_batch_host_rules():
    """The two host-side decisions of `sageattn_varlen`: which packed views can be served, and when
    slots of the longest length per sequence are an acceptable workspace."""
    from sageattention import core
    t = _t(10, 2, 128)
    assert be.packed_view_reason(t) is None
    assert be.packed_view_reason(t[:, :, ::2]) == "last_stride"
    assert be.packed_view_reason(t.unsqueeze(0)) == "rank"
    assert be.packed_view_reason(torch.empty(10, 2, 132, dtype=torch.float16)[:, :, :128]) == "stride_range"
    fused = _t(10, 3, 2, 128)
    assert be.packed_view_reason(fused[:, 1]) is None                 # token stride 3 * H * D
    fit = core._varlen_slots_fit
    assert fit(11, 8, 8, 11 * 4096, 11 * 4096, 4096, 4096)            # equal lengths: slots == packed size
    assert fit(4, 8, 8, 1000, 1000, 900, 900)                         # small: below the free allowance
    assert not fit(4096, 32, 32, 4096 * 64 + 65536, 4096 * 64 + 65536, 65536, 65536)   # one long sequence among thousands
    assert not fit(40000, 2, 2, 80000, 80000, 4, 4)                   # more (sequence, head) units than a grid axis takes
    assert fit(3, 2, 2, 10, 10, 10 ** 9, 10 ** 9)                     # bounds above the token count are cut to it


def test_pad_len():
    assert [be.pad_len(n) for n in (1, 127, 128, 129, 8771, 47520)] == [128, 128, 128, 256, 8832, 47616]


def test_environment_switches_are_read_at_import():
    """SAGEATTN_SK1_BACKEND=0 asks for a backend this package does not have; SAGEATTN_SK1_INT8=0 makes
    e4m3 Q.K the default for float16 (both read once, at import, like the reference)."""
    import subprocess
    import sys
    from conftest import ROOT
    code = ("import sys, torch; sys.path.insert(0, %r); import sageattention as s; from sageattention import core; "
            "print(core.SK1_INT8, core.SK1_BACKEND); q = torch.zeros(1, 1, 4, 128, dtype=torch.float16); "
            "s.sageattn(q, q, q)") % os.path.join(ROOT, "sageattention-rdna4_b200")

    def run(env):
        full = dict(os.environ, **env)
        return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=full, timeout=300)

    off = run({"SAGEATTN_SK1_BACKEND": "0"})
    assert off.stdout.split()[:2] == ["True", "False"] and "NotImplementedError" in off.stderr
    fp8 = run({"SAGEATTN_SK1_INT8": "off"})
    assert fp8.stdout.split()[:2] == ["False", "True"] and "no CPU path" in fp8.stderr
    default = run({"SAGEATTN_SK1_INT8": "", "SAGEATTN_SK1_BACKEND": ""})
    assert default.stdout.split()[:2] == ["True", "True"] and "no CPU path" in default.stderr


def test_device_status_codes_become_exceptions():
    """A status word that a finished call left non-zero is turned into RuntimeError by the host
    logic (the word is faked here; no GPU involved) and cleared, so that the report is made once."""
    import ctypes
    word = ctypes.c_int32(0)
    st = be._StreamState(host_word=word)
    st.raise_if_failed("test")                                   # zero: nothing happens
    assert st.pending() == 0
    word.value = 2
    with pytest.raises(RuntimeError, match="MMA issuer"):
        st.raise_if_failed("test")
    assert word.value == 0 and st.pending() == 0
    word.value = 8 | 4
    with pytest.raises(RuntimeError) as exc:
        st.raise_if_failed("the next call on the stream")
    msg = str(exc.value)
    assert "0xc" in msg and "softmax warp" in msg and "prologue" in msg and "undefined" in msg
    assert "unknown role" in be.describe_status(0x40)
    assert be.status()["watch"] in (True, False) and "device_status" in be.status()


def test_strict_and_watch_switches_are_read_from_the_environment():
    import subprocess
    import sys
    code = ("import sys; sys.path.insert(0, %r); from sageattention import b200_backend as be; "
            "print(int(be._STRICT), int(be._WATCH))" % os.path.dirname(os.path.dirname(be.__file__)))
    run = lambda env: subprocess.run([sys.executable, "-c", code], env={**os.environ, **env}, capture_output=True,
                                     text=True, check=True).stdout.split()
    assert run({"SAGEATTN_B200_STRICT": "", "SAGEATTN_B200_WATCH": ""}) == ["0", "1"]
    assert run({"SAGEATTN_B200_STRICT": "1", "SAGEATTN_B200_WATCH": "0"}) == ["1", "1"]     # strict needs the copy
    assert run({"SAGEATTN_B200_STRICT": "0", "SAGEATTN_B200_WATCH": "0"}) == ["0", "0"]



def test_choice_between_the_two_sets_of_attention_kernels():
    """Host logic only: a signature starts with the negligible-tile tests on and one probing call;
    a probe that skipped next to nothing buys PLAIN_CALLS calls on the kernels without the tests,
    then the signature probes again; a probe that skipped a lot keeps the tests on; only one probe
    is outstanding at a time, and a signature that could not probe keeps asking."""
    a = be._Adaptive()
    k1, k2 = ("sig", 1), ("sig", 2)
    assert a.decide(k1) == (False, True)
    a.probe = ("placeholder",)
    assert a.decide(k1) == (False, False) and a.decide(k2) == (False, False)
    a.probe = None
    assert a.decide(k2) == (False, True)                         # k2 never got its probe: it asks again
    assert a.take_result(k1, 3, 1000) < be.PROBE_MIN_SHARE
    for _ in range(be.PLAIN_CALLS):
        assert a.decide(k1) == (True, False)
    assert a.decide(k1) == (False, True)                         # back to the tests, probing
    assert a.take_result(k1, 600, 1000) == 0.6
    assert a.decide(k1) == (False, False)
    for _ in range(be.PROBE_AGAIN_AFTER - 1):
        a.decide(k1)
    assert a.decide(k1) == (False, True)
