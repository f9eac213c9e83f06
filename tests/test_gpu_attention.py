"""Attention parity on the GPU, through the C-ABI.

Tolerances (the output is not a bit target: exp2 is a hardware approximation and the running max
advances per 128 keys here, per 64 in the reference):
  * against the oracle evaluated with the same 128-key tile:  cosine >= 0.9999, rel-L1 <= 5e-3
  * against the oracle with the reference's 64-key tile:       cosine >= 0.9995, rel-L1 <= 2e-2
  * against fp32 SDPA: relative RMS below the reference's bar 0.08, and no worse than 1.03x the
    oracle's own error.
"""
import pytest
import torch

from oracle import ref_numerics as R
from sageattention import b200_backend as be
import sageattention

pytestmark = pytest.mark.gpu

COS_SAME, L1_SAME = 0.9999, 5e-3
COS_REF, L1_REF = 0.9995, 2e-2
MAX_REL_RMS = 0.08


def _run(q, k, v, causal, smooth=True, int8=None, layout="HND"):
    out = be.sage_call(q, k, v, tensor_layout=layout, is_causal=causal, smooth_k=smooth, int8=int8)
    torch.cuda.synchronize()
    ql = q.transpose(1, 2) if layout == "NHD" else q
    b, h, n, _ = ql.shape
    assert be.last_status(q, b, h, n) == 0, "a bounded wait inside the kernel gave up"
    return out


def _check(out, q, k, v, causal, smooth=True, int8=None, tight=True):
    o128 = R.sageattn_oracle(q, k, v, is_causal=causal, smooth_k=smooth, int8=int8, tile=128)
    o64 = R.sageattn_oracle(q, k, v, is_causal=causal, smooth_k=smooth, int8=int8, tile=64)
    ref = R.sdpa_fp32(q, k, v, is_causal=causal)
    assert torch.isfinite(out.float()).all()
    assert R.cosine(out, o128) >= COS_SAME and R.rel_l1(out, o128) <= L1_SAME
    assert R.cosine(out, o64) >= COS_REF and R.rel_l1(out, o64) <= L1_REF
    e_gpu, e_ora = R.rel_rms(out, ref), R.rel_rms(o64, ref)
    assert e_gpu < MAX_REL_RMS
    if tight:
        assert e_gpu <= 1.03 * e_ora + 1e-4


def test_golden_outputs(golden):
    g = golden
    out = _run(g.q.cuda(), g.k.cuda(), g.v.cuda(), g.causal, g.smooth).cpu()
    assert torch.isfinite(out.float()).all()
    assert R.cosine(out, g.out128) >= COS_SAME and R.rel_l1(out, g.out128) <= L1_SAME
    assert R.cosine(out, g.out64) >= COS_REF and R.rel_l1(out, g.out64) <= L1_REF


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
def test_config1_cpu_reference_check(dtype, causal):
    """B=1,H=4,N=512, K channel bias 0.5, smooth_k on."""
    q, k, v = R.make_inputs(1, 4, 512, 128, dtype, seed=0, k_bias_std=0.5)
    out = _run(q.cuda(), k.cuda(), v.cuda(), causal).cpu()
    _check(out, q, k, v, causal)


@pytest.mark.parametrize("n", [1, 15, 63, 64, 65, 127, 128, 129, 300, 1000])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("smooth", [True, False])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_edge_lengths(n, causal, smooth, dtype):
    q, k, v = R.make_inputs(2, 3, n, 128, dtype, seed=100 + n)
    # sentinel-prefilled output: every element must be overwritten
    out = torch.full(q.shape, float("nan"), dtype=dtype, device="cuda")
    be.sage_call(q.cuda(), k.cuda(), v.cuda(), is_causal=causal, smooth_k=smooth, out=out)
    torch.cuda.synchronize()
    assert be.last_status(out, 2, 3, n) == 0
    _check(out.cpu(), q, k, v, causal, smooth, tight=n >= 64)


def test_large_v_stays_finite():
    q, k, v = R.make_inputs(1, 2, 300, seed=7)
    v[0, 0, 11] = 20000.0
    out = _run(q.cuda(), k.cuda(), v.cuda(), False).cpu()
    assert torch.isfinite(out.float()).all()
    # With S > 1 most of P lands in e4m3's subnormal range, so the error depends on where the
    # running max stands when a key is folded: the 64-key and 128-key loops differ by more than
    # the 3 % bar here (0.022 vs 0.026, both far below 0.08); the same-tile comparison still holds.
    _check(out, q, k, v, False, tight=False)


def test_nhd_and_fused_qkv_match_hnd_bitwise():
    b, h, n = 2, 3, 300
    q, k, v = R.make_inputs(b, h, n, seed=9, device="cuda")
    base = _run(q, k, v, True)
    qn, kn, vn = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    out_nhd = _run(qn, kn, vn, True, layout="NHD")
    assert out_nhd.shape == (b, n, h, 128)
    assert torch.equal(out_nhd.transpose(1, 2), base)
    fused = torch.empty(b, n, h, 3 * 128, dtype=q.dtype, device="cuda")
    for i, t in enumerate((q, k, v)):
        fused[..., 128 * i:128 * (i + 1)] = t.transpose(1, 2)
    views = [fused[..., 128 * i:128 * (i + 1)] for i in range(3)]
    out_f = _run(*views, True, layout="NHD")
    assert torch.equal(out_f.transpose(1, 2), base)


def test_int8_is_default_and_not_worse_than_e4m3():
    q, k, v = R.make_inputs(1, 4, 1000, seed=3, k_bias_std=0.5, device="cuda")
    ref = R.sdpa_fp32(q, k, v)
    d = sageattention.sageattn(q, k, v)
    i8 = sageattention.sageattn(q, k, v, sk1_int8=True)
    f8 = sageattention.sageattn(q, k, v, sk1_int8=False)
    assert torch.equal(d, i8)
    assert not torch.equal(d, f8)
    assert R.rel_rms(d, ref) <= 1.05 * R.rel_rms(f8, ref)


def test_public_api_entry_points_agree():
    q, k, v = R.make_inputs(1, 2, 200, seed=4, device="cuda")
    a = sageattention.sageattn(q, k, v, is_causal=True)
    b = sageattention.sageattn_qk_int8_pv_fp8(q, k, v, is_causal=True)
    c = sageattention.sageattn_qk_int8_pv_fp8_cuda(q, k, v, is_causal=True, pv_accum_dtype="fp32")
    assert torch.equal(a, b) and torch.equal(a, c)
    s = sageattention.sageattn(q, k, v, sm_scale=0.05)
    assert not torch.equal(s, sageattention.sageattn(q, k, v))
    with pytest.raises(NotImplementedError):          # head_dim must be a multiple of 8 (up to 128)
        sageattention.sageattn(q[..., :60], k[..., :60], v[..., :60])


def test_separate_launches_equal_the_fused_entry_point():
    """sage_prologue + sage_attn_fwd (the two reference-shaped entry points) == sage_attention."""
    q, k, v = R.make_inputs(1, 3, 400, seed=12, device="cuda")
    pq = be.quant_qkv(q, k, v)
    out = torch.empty_like(q)
    st = be.attn_launch(pq, out, True, 128 ** -0.5)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert torch.equal(out, _run(q, k, v, True))


@pytest.mark.parametrize("dtype,causal", [(torch.float16, False), (torch.bfloat16, True)])
def test_image_size_config(dtype, causal):
    """B=1,H=48,N=8771 with a K channel bias and per-head Q/K multipliers; the oracle is the same
    restatement evaluated by torch on the device (8 heads of it, to bound the run time)."""
    q, k, v = R.make_inputs(1, 48, 8771, 128, dtype, seed=0, k_bias_std=1.0,
                            head_scale=(dtype == torch.float16), device="cuda")
    out = _run(q, k, v, causal)
    assert torch.isfinite(out.float()).all()
    sl = slice(0, 48, 6)
    qs, ks, vs = q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous()
    _check(out[:, sl], qs, ks, vs, causal)


def test_video_length_properties():
    """B=1,H=2 at N=47520 (two of the 48 heads; every head is independent) with 0.1 % of the K
    tokens scaled x50, causal.  The oracle is the same restatement evaluated by torch on the
    device.  Head 1 has a constant V: its output must equal the oracle's, which is NOT the
    constant for every row -- when an outlier key dominates a row, the many small probabilities
    fall below e4m3's smallest subnormal after the fold and drop out of P.V while they stay in the
    row sum; that is a property of the reference's numerics, reproduced here."""
    n = 47520
    q, k, v = R.make_inputs(1, 2, n, seed=0, outlier_frac=0.001, device="cuda")
    v[:, 1] = 0.75
    out = _run(q, k, v, True)
    assert torch.isfinite(out.float()).all()
    o128 = R.sageattn_oracle(q, k, v, is_causal=True, tile=128)
    o64 = R.sageattn_oracle(q, k, v, is_causal=True, tile=64)
    assert R.cosine(out, o128) >= COS_SAME and R.rel_l1(out, o128) <= L1_SAME
    assert R.cosine(out, o64) >= COS_REF and R.rel_l1(out, o64) <= L1_REF
    assert (out[:, 1].float() - o128[:, 1].float()).abs().max().item() < 0.05
    assert out[:, 1].float().max().item() <= 0.75 * 1.0625    # e4m3 rounding of P can add at most one half-ulp (2^-4)
    rows = torch.tensor([0, 1, 127, 128, 5000, 23760, 47519], device="cuda")
    s = torch.matmul(q[0, 0, rows].float(), k[0, 0].float().t()) * 128 ** -0.5
    s = s.masked_fill(torch.arange(n, device="cuda")[None, :] > rows[:, None], float("-inf"))
    ref = torch.matmul(torch.softmax(s, -1), v[0, 0].float())
    e_gpu, e_ora = R.rel_rms(out[0, 0, rows], ref), R.rel_rms(o64[0, 0, rows], ref)
    assert e_gpu <= 1.1 * e_ora + 1e-3


def test_device_status_reaches_the_caller_as_an_exception():
    """The host learns of a device-side failure from a 4-byte copy of the status word that follows
    every call (no synchronisation on the hot path).  No wait is made to run out here: the copy is
    fed a word that already holds a code, and the next call, `check()` and `status()` must report
    it; a healthy call leaves nothing behind."""
    import ctypes
    from sageattention import _native
    lib = _native.load()
    q, k, v = R.make_inputs(1, 2, 300, seed=6, device="cuda")
    out = sageattention.sageattn(q, k, v)
    be.check()                                                       # waits, finds nothing
    assert be.status()["device_status"] == {}
    dev, stream = q.device, torch.cuda.current_stream().cuda_stream
    st = be._state(dev, stream, create=False)
    assert st is not None and st.pending() == 0
    word = torch.tensor([2 | 8], dtype=torch.int32, device="cuda")   # "MMA issuer" and "prologue"
    assert lib.sage_status_mirror(word.data_ptr(), ctypes.addressof(be._host_word(st)), 1, stream) == 0
    torch.cuda.synchronize()
    assert list(be.status()["device_status"].values()) == [10]
    with pytest.raises(RuntimeError, match="MMA issuer"):
        sageattention.sageattn(q, k, v)                              # reported at the next call, before it launches
    again = sageattention.sageattn(q, k, v)                          # reported once; the path works on
    be.check()
    assert torch.equal(out, again)
    # strict mode: every call synchronises and checks
    assert lib.sage_status_mirror(word.data_ptr(), ctypes.addressof(be._host_word(st)), 1, stream) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="prologue"):
        be.check()
    be._STRICT = True
    try:
        assert torch.equal(sageattention.sageattn(q, k, v), out)
    finally:
        be._STRICT = False


@pytest.mark.parametrize("scale", [0.0, -0.5, float("inf"), float("nan")])
def test_sm_scale_must_be_finite_and_positive(scale):
    q, k, v = R.make_inputs(1, 1, 64, seed=1, device="cuda")
    with pytest.raises(ValueError, match="sm_scale"):
        sageattention.sageattn(q, k, v, sm_scale=scale)


def test_last_status_does_not_invent_a_workspace():
    q, k, v = R.make_inputs(1, 2, 200, seed=2, device="cuda")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with pytest.raises(RuntimeError, match="no call has run"):
            be.last_status(q, 1, 2, 200)
    sageattention.sageattn(q, k, v)
    assert be.last_status(q, 1, 2, 200) == 0
    with pytest.raises(RuntimeError, match="had shape"):
        be.last_status(q, 1, 2, 201)
