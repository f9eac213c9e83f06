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


@pytest.mark.parametrize("d", [64, 96, 8, 120])
@pytest.mark.parametrize("dtype,causal", [(torch.float16, False), (torch.bfloat16, True)])
def test_head_dim_below_128(d, dtype, causal):
    g = torch.Generator().manual_seed(5 + d)
    q = torch.randn(2, 4, 260, d, generator=g).to(dtype)
    k = (torch.randn(2, 2, 260, d, generator=g) + 0.5).to(dtype)
    v = torch.randn(2, 2, 260, d, generator=g).to(dtype)
    out, lse = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), is_causal=causal, return_lse=True)
    assert _status(out, q, k) == 0
    assert out.shape == q.shape and torch.isfinite(out.float()).all()
    want, want_l = R.sageattn_oracle(q, k, v, is_causal=causal, tile=128, return_lse=True)
    ref = R.sdpa_fp32(q, k, v, is_causal=causal)
    assert R.cosine(out.cpu(), want) >= COS_SAME and R.rel_l1(out.cpu(), want) <= L1_SAME
    assert R.rel_rms(out.cpu(), ref) < (MAX_REL_RMS if d >= 64 else 0.2)
    assert (lse.cpu() - want_l).abs().max().item() < 2e-3
    # identical to the same call on rows zero-padded to 128 columns with the same softmax scale
    pad = lambda t: torch.nn.functional.pad(t, (0, 128 - d)).cuda()
    padded = sageattention.sageattn(pad(q), pad(k), pad(v), is_causal=causal, sm_scale=d ** -0.5)
    assert torch.equal(padded[..., :d], out)


def test_head_dim_64_view_of_wider_rows_leaves_neighbours_alone():
    g = torch.Generator().manual_seed(9)
    qkv = torch.randn(1, 200, 3, 4, 128, generator=g).half().cuda()       # fused QKV, NHD, only 64 columns used
    q, k, v = (qkv[:, :, i, :, :64] for i in range(3))
    out = torch.full((1, 200, 4, 128), 7.0, dtype=torch.float16, device="cuda")
    be.sage_call(q, k, v, tensor_layout="NHD", out=out[..., :64])
    torch.cuda.synchronize()
    assert (out[..., 64:] == 7.0).all()
    want = sageattention.sageattn(q.contiguous(), k.contiguous(), v.contiguous(), tensor_layout="NHD")
    assert torch.equal(out[..., :64], want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,nq,nk,causal", [(4, 4, 300, 300, False), (4, 2, 300, 300, True), (4, 2, 100, 515, False)])
def test_smooth_v(dtype, hq, hkv, nq, nk, causal):
    g = torch.Generator().manual_seed(6)
    q = torch.randn(1, hq, nq, 128, generator=g).to(dtype)
    k = torch.randn(1, hkv, nk, 128, generator=g).to(dtype)
    v = (torch.randn(1, hkv, nk, 128, generator=g) + 4.0 * torch.randn(1, hkv, 1, 128, generator=g)).to(dtype)
    out = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), is_causal=causal, smooth_v=True)
    assert _status(out, q, k) == 0
    want = R.sageattn_oracle(q, k, v, is_causal=causal, tile=128, smooth_v=True)
    ref = R.sdpa_fp32(q, k, v, is_causal=causal)
    assert R.cosine(out.cpu(), want) >= COS_SAME and R.rel_l1(out.cpu(), want) <= L1_SAME
    plain = sageattention.sageattn(q.cuda(), k.cuda(), v.cuda(), is_causal=causal)
    # a V with a large per-channel offset is exactly the case smooth_v is for
    assert R.rel_rms(out.cpu(), ref) < 0.6 * R.rel_rms(plain.cpu(), ref)
    up = sageattention.sageattn_qk_int8_pv_fp8(q.cuda(), k.cuda(), v.cuda(), is_causal=causal, smooth_v=True,
                                               pv_accum_dtype="fp32")
    assert torch.equal(up, out)
    with pytest.warns(UserWarning, match="smooth_v will be ignored"):
        ign = sageattention.sageattn_qk_int8_pv_fp8(q.cuda(), k.cuda(), v.cuda(), is_causal=causal, smooth_v=True)
    assert torch.equal(ign, plain)


def test_smooth_v_mean_and_codes_match_the_oracle():
    q, k, v = _inputs(1, 2, 2, 200, 200, torch.float16, 7)
    v = (v.float() + 2.0).half()
    out = be.sage_call(q.cuda(), k.cuda(), v.cuda(), smooth_v=True)
    torch.cuda.synchronize()
    lib = be._native.load()
    import ctypes
    offs = (ctypes.c_size_t * 13)()
    assert lib.sage_workspace_layout_ex(1, 2, 2, 200, 200, offs) == 13
    ws = be._workspace(out.device, int(torch.cuda.current_stream().cuda_stream), 1, 2, 200, 2, 200)
    vmean = ws[offs[12]: offs[12] + 2 * 128 * 4].view(torch.float32).view(1, 2, 128).cpu()
    v8t = ws[offs[4]: offs[4] + 2 * 256 * 128].view(2, 128, 256).cpu()
    sv = ws[offs[5]: offs[5] + 2 * 256 * 4].view(torch.float32).view(1, 2, 256).cpu()
    pq = R.prologue(q, k, v, pad_multiple=128, smooth_v=True)
    assert torch.equal(vmean, pq["vmean"])
    assert torch.equal(sv, pq["sv"])
    want_codes = pq["v8"].to(torch.float8_e4m3fn).view(torch.uint8).view(2, 256, 128).transpose(1, 2)
    assert torch.equal(v8t, want_codes)


@pytest.mark.parametrize("dtype,causal", [(torch.float16, False), (torch.bfloat16, True)])
def test_varlen_matches_per_sequence_calls(dtype, causal):
    g = torch.Generator().manual_seed(8)
    lens_q = [5, 130, 130, 130, 0, 257, 64, 64]            # runs of equal lengths go out as one batched call
    lens_k = lens_q if causal else [40, 130, 130, 130, 0, 64, 200, 200]
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int64).cuda()
    q = torch.randn(sum(lens_q), 4, 128, generator=g).to(dtype).cuda()
    k = torch.randn(sum(lens_k), 2, 128, generator=g).to(dtype).cuda()
    v = torch.randn(sum(lens_k), 2, 128, generator=g).to(dtype).cuda()
    out = sageattention.sageattn_varlen(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), is_causal=causal)
    assert out.shape == q.shape
    for i in range(len(lens_q)):
        a, b = int(cu_q[i]), int(cu_q[i + 1])
        c, d = int(cu_k[i]), int(cu_k[i + 1])
        if a == b:
            continue
        one = sageattention.sageattn(q[a:b].unsqueeze(0).contiguous(), k[c:d].unsqueeze(0).contiguous(),
                                     v[c:d].unsqueeze(0).contiguous(), tensor_layout="NHD", is_causal=causal)
        assert torch.equal(out[a:b], one[0])
        ref = R.sdpa_fp32(q[a:b].transpose(0, 1).unsqueeze(0).cpu(), k[c:d].transpose(0, 1).unsqueeze(0).cpu(),
                          v[c:d].transpose(0, 1).unsqueeze(0).cpu(), is_causal=causal)
        assert R.rel_rms(out[a:b].transpose(0, 1).unsqueeze(0).cpu(), ref) < MAX_REL_RMS


def test_cuda_graph_capture_and_replay():
    """After one warm-up call (library load, shared-memory opt-in, workspace allocation) the whole
    call -- tensor-map encodes on the host, four kernels -- can be captured and replayed."""
    q, k, v = _inputs(1, 8, 8, 300, 300, torch.float16, 11)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    want = sageattention.sageattn(q, k, v, is_causal=True)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        sageattention.sageattn(q, k, v, is_causal=True)          # warm-up on the capture stream
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            got = sageattention.sageattn(q, k, v, is_causal=True)
    torch.cuda.current_stream().wait_stream(s)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    q.copy_(torch.roll(q, 1, dims=2))                              # new data in the captured buffers
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(got, sageattention.sageattn(q, k, v, is_causal=True))


def test_strides_beyond_32_bits():
    """Two batch elements more than 2**31 elements apart (the reference refuses such views; the
    kernels here take 64-bit strides): same bits as the call on compact copies."""
    far = 2 ** 31 + 4096
    n, h = 200, 2
    g = torch.Generator(device="cuda").manual_seed(5)

    def spread():
        buf = torch.empty(far + h * n * 128, dtype=torch.float16, device="cuda")
        view = buf.as_strided((2, h, n, 128), (far, n * 128, 128, 1))
        view.copy_(torch.randn(2, h, n, 128, device="cuda", generator=g).half())
        return view

    q, k, v = spread(), spread(), spread()
    assert q.stride(0) > 2 ** 31
    out = sageattention.sageattn(q, k, v, is_causal=True)
    want = sageattention.sageattn(q.contiguous(), k.contiguous(), v.contiguous(), is_causal=True)
    assert torch.equal(out, want)
    out_far = torch.empty(far + h * n * 128, dtype=torch.float16, device="cuda").as_strided(
        (2, h, n, 128), (far, n * 128, 128, 1))
    be.sage_call(q, k, v, is_causal=True, out=out_far)
    assert torch.equal(out_far, want)


def test_int8_environment_switch_selects_the_e4m3_kernel(tmp_path):
    """SAGEATTN_SK1_INT8=0 in a fresh interpreter gives the e4m3 Q.K path bit for bit (the reference's
    tests/test_sk1_backend.py:121-130)."""
    import os
    import subprocess
    import sys
    from conftest import ROOT
    out_file = tmp_path / "o.pt"
    code = ("import sys, torch; sys.path.insert(0, %r); sys.path.insert(0, %r); import sageattention as s; "
            "from oracle import ref_numerics as R; q, k, v = R.make_inputs(1, 2, 300, seed=31, device='cuda'); "
            "torch.save(s.sageattn(q, k, v).cpu(), %r)"
            % (os.path.join(ROOT, "sageattention-rdna4_b200"), ROOT, str(out_file)))
    res = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, SAGEATTN_SK1_INT8="0"),
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    q, k, v = R.make_inputs(1, 2, 300, seed=31, device="cuda")
    assert torch.equal(torch.load(out_file), sageattention.sageattn(q, k, v, sk1_int8=False).cpu())
    assert not torch.equal(torch.load(out_file), sageattention.sageattn(q, k, v).cpu())


def test_caller_that_probes_for_attn_mask_and_passes_nhd():
    """The way ComfyUI's `--use-sage-attention` drives the package: it inspects `sageattn` for an
    `attn_mask` parameter (none, so masked calls stay with its own attention), reshapes to
    (batch, tokens, heads, head_dim), and calls with `tensor_layout="NHD"`, `is_causal=False` and,
    through its generic wrapper, `attn_mask=None`.  No ComfyUI here: this is the call pattern."""
    import inspect
    assert "attn_mask" not in inspect.signature(sageattention.sageattn).parameters
    b, heads, dim_head, n = 2, 6, 128, 333
    g = torch.Generator().manual_seed(12)
    q, k, v = (torch.randn(b, n, heads * dim_head, generator=g).half().cuda() for _ in range(3))
    q4, k4, v4 = (t.view(b, -1, heads, dim_head) for t in (q, k, v))
    out = sageattention.sageattn(q4, k4, v4, attn_mask=None, is_causal=False, tensor_layout="NHD")
    out = out.reshape(b, -1, heads * dim_head)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q4.transpose(1, 2).float(), k4.transpose(1, 2).float(), v4.transpose(1, 2).float()).transpose(1, 2)
    assert R.rel_rms(out.view(b, n, heads, dim_head).cpu(), ref.cpu()) < MAX_REL_RMS
    with pytest.raises(NotImplementedError):
        sageattention.sageattn(q4, k4, v4, attn_mask=torch.ones(n, n, device="cuda", dtype=torch.bool),
                               tensor_layout="NHD")
