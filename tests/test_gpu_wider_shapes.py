"""Call shapes the reference's hand-written path refuses (it hands them to its other backends) and
that the upstream API defines: grouped-query attention, a key length different from the query
length, and the log-sum-exp output.  Parity is against the oracle with the same extensions and
against exact attention; everything goes through the C-ABI (`sage_attention_ex`)."""
import pytest
import torch

from oracle import ref_numerics as R
from sageattention import b200_backend as be
import sageattention

pytestmark = pytest.mark.gpu

COS_SAME, L1_SAME = 0.9999, 5e-3
MAX_REL_RMS = 0.08
LSE_ABS = 0.15          # worst row: a causal row with a handful of keys carries one logit's int8 error
LSE_MEAN = 0.02         # typical row: the int8 score error moves the log-sum-exp by about 1e-2


def _inputs(b, hq, hkv, nq, nk, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, hq, nq, 128, generator=g).to(dtype)
    k = (torch.randn(b, hkv, nk, 128, generator=g) + 0.5 * torch.randn(1, hkv, 1, 128, generator=g)).to(dtype)
    v = torch.randn(b, hkv, nk, 128, generator=g).to(dtype)
    return q, k, v


def _status(out, q, k):
    torch.cuda.synchronize()
    b, hq, nq, _ = q.shape
    return be.last_status(out, b, hq, nq, k.shape[1], k.shape[2])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,causal", [(8, 2, False), (6, 3, True), (4, 1, False)])
def test_grouped_query_attention(dtype, hq, hkv, causal):
    q, k, v = _inputs(2, hq, hkv, 300, 300, dtype, 1)
    out = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), is_causal=causal)
    assert _status(out, q, k) == 0
    want = R.sageattn_oracle(q, k, v, is_causal=causal, tile=128)
    ref = R.sdpa_fp32(q, k, v, is_causal=causal)
    assert out.shape == q.shape
    assert R.cosine(out.cpu(), want) >= COS_SAME and R.rel_l1(out.cpu(), want) <= L1_SAME
    assert R.rel_rms(out.cpu(), ref) < MAX_REL_RMS
    # the same call with K/V heads repeated explicitly gives the same bits
    g = hq // hkv
    rep = sageattention.sageattn(q.cuda(), k.repeat_interleave(g, 1).cuda(), v.repeat_interleave(g, 1).cuda(),
                                 is_causal=causal)
    assert torch.equal(rep, out)


@pytest.mark.parametrize("nq,nk", [(1, 300), (130, 64), (257, 1000), (1000, 129)])
def test_key_length_differs_from_query_length(nq, nk):
    q, k, v = _inputs(1, 4, 2, nq, nk, torch.float16, 2)
    out = torch.full(q.shape, float("nan"), dtype=q.dtype, device="cuda")
    be.sage_call(q.cuda(), k.cuda(), v.cuda(), out=out)
    assert _status(out, q, k) == 0
    want = R.sageattn_oracle(q, k, v, tile=128)
    ref = R.sdpa_fp32(q, k, v)
    assert torch.isfinite(out.float()).all()
    assert R.cosine(out.cpu(), want) >= COS_SAME and R.rel_l1(out.cpu(), want) <= L1_SAME
    assert R.rel_rms(out.cpu(), ref) < MAX_REL_RMS
    with pytest.raises(ValueError, match="causal"):
        sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), is_causal=True)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal,smooth", [(False, True), (True, True), (False, False)])
def test_log_sum_exp(dtype, causal, smooth):
    q, k, v = _inputs(1, 4, 2, 333, 333, dtype, 3)
    out, lse = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), is_causal=causal, smooth_k=smooth,
                                      return_lse=True)
    assert _status(out, q, k) == 0
    assert lse.shape == (1, 4, 333) and lse.dtype == torch.float32
    want_o, want_l = R.sageattn_oracle(q, k, v, is_causal=causal, smooth_k=smooth, tile=128, return_lse=True)
    _, exact = R.sdpa_fp32(q, k, v, is_causal=causal, return_lse=True)
    assert (lse.cpu() - want_l).abs().max().item() < 2e-3          # same quantised logits as the oracle
    err = (lse.cpu() - exact).abs()                                 # and close to the exact value
    assert err.max().item() < LSE_ABS and err.mean().item() < LSE_MEAN
    plain = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), is_causal=causal, smooth_k=smooth)
    assert torch.equal(plain, out)                                  # asking for the LSE does not change the output
    out2, lse2 = sageattention.sageattn_qk_int8_pv_fp8(q.cuda(), k.cuda(), v.cuda(), is_causal=causal,
                                                       smooth_k=smooth, return_lse=True)
    assert torch.equal(out2, out) and torch.equal(lse2, lse)


def test_nhd_layout_with_grouped_heads_and_lse():
    q, k, v = _inputs(2, 4, 2, 200, 200, torch.float16, 4)
    out_h, lse_h = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), return_lse=True)
    qn, kn, vn = (t.transpose(1, 2).contiguous().cuda() for t in (q, k, v))
    out_n, lse_n = sageattention.sageattn(qn, kn, vn, tensor_layout="NHD", return_lse=True)
    assert out_n.shape == (2, 200, 4, 128)
    assert torch.equal(out_n.transpose(1, 2), out_h) and torch.equal(lse_n, lse_h)
