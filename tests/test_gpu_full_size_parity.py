"""Parity at the full sizes of the benchmark configurations, through the C-ABI.

The video-length configuration (B=1, H=48, N=47520, 0.1 % of the K tokens scaled x50; fp16 and
bf16, causal and not) and the scaling configuration (B=4, H=48, N=47520, bf16) are run as the real
calls -- all 48 (or 192) heads, so the kernel instantiation and grid are the benchmark's -- and a
few heads are compared with the oracle, which torch evaluates on the device in row chunks.  The
prologue's codes and scales are compared bit for bit for every head.  One test pins the
device-side evaluation of the oracle itself: it must give the CPU evaluation's bytes.

Inputs are generated on the device head by head (a host-side generator would need minutes for
3 x 48 x 47520 x 128 normal deviates).
"""
import pytest
import torch

from oracle import ref_numerics as R
from sageattention import b200_backend as be

pytestmark = pytest.mark.gpu

N_VIDEO = 47520
COS_SAME, L1_SAME = 0.9999, 5e-3          # against the oracle with the kernel's 128-key tile
COS_REF, L1_REF = 0.9995, 2e-2            # against the oracle with the reference's 64-key tile


def _device_inputs(b, h, n, dtype, seed, outlier_frac=0.001):
    """Q, K, V ~ N(0,1), a seeded `outlier_frac` of the key tokens (one index set for all heads)
    scaled x50: the value distribution of the video-length configuration, drawn on the device."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = [torch.empty(b, h, n, 128, dtype=dtype, device="cuda") for _ in range(3)]
    idx = torch.randperm(n, generator=g, device="cuda")[: int(round(outlier_frac * n))]
    for bi in range(b):
        for hi in range(h):
            for t, dst in enumerate(out):
                x = torch.randn(n, 128, generator=g, device="cuda")
                if t == 1:
                    x[idx] *= 50.0
                dst[bi, hi] = x.to(dtype)
    return out


def _compare_heads(out, q, k, v, units, causal, tiles=(128, 64), wide_scores=False):
    """`wide_scores`: e4m3 Q.K^T with x50 keys.  The tensor core does not carry the sum of the 128
    e4m3 products of a score at full fp32 precision; with ordinary scores the difference from the
    oracle's fp32 sum is invisible, but the x50 keys put the row maxima near 2^8 in the exponent
    domain, where a relative error of 2^-13 is 0.03 in the exponent.  The pair of bounds the
    north star states (cosine 0.9995, relative L1 2e-2) is applied for both tilings then, and the
    error against exact attention must stay within 5 % of the oracle's own."""
    for bi, hi in units:
        sl = (slice(bi, bi + 1), slice(hi, hi + 1))
        qs, ks, vs = q[sl], k[sl], v[sl]
        for tile in tiles:
            want = R.sageattn_oracle(qs, ks, vs, is_causal=causal, tile=tile)
            cos, l1 = R.cosine(out[sl], want), R.rel_l1(out[sl], want)
            lim = (COS_SAME, L1_SAME) if (tile == 128 and not wide_scores) else (COS_REF, L1_REF)
            assert cos >= lim[0] and l1 <= lim[1], (bi, hi, tile, cos, l1)
        if wide_scores:
            ref = R.sdpa_fp32(qs, ks, vs, is_causal=causal)
            assert R.rel_rms(out[sl], ref) <= 1.05 * R.rel_rms(want, ref) + 1e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
def test_video_length_all_heads(dtype, causal):
    """B=1, H=48, N=47520: the headline call (fp16, non-causal: int8 Q.K, two query tiles per
    CTA, 372 query tiles per head) and its three siblings.  Heads 0, 29 and 47 against the oracle
    with both tilings."""
    q, k, v = _device_inputs(1, 48, N_VIDEO, dtype, seed=3)
    out = be.sage_call(q, k, v, is_causal=causal)
    torch.cuda.synchronize()
    assert be.last_status(out, 1, 48, N_VIDEO) == 0
    assert torch.isfinite(out.float()).all()
    wide = dtype == torch.bfloat16
    _compare_heads(out, q, k, v, [(0, 0), (0, 29)], causal, wide_scores=wide)
    _compare_heads(out, q, k, v, [(0, 47)], causal, tiles=(128,), wide_scores=wide)


def _assert_prologue_bits(pq, ref, bh0, bh1):
    """Codes and scales of heads bh0..bh1-1 of a prologue result against the oracle's, on the
    device, bit for bit."""
    n_pad = pq["n_pad"]
    u8 = lambda t: t.contiguous().view(torch.uint8)
    flat = lambda t: t.reshape(bh1 - bh0, *t.shape[2:])
    order = be.k8_row_order(n_pad, device="cuda")
    assert torch.equal(u8(pq["q8"][bh0:bh1]), u8(flat(ref["q8"]))), "q8"
    assert torch.equal(pq["sq"][bh0:bh1], flat(ref["sq"])), "sq"
    assert torch.equal(u8(pq["k8"][bh0:bh1])[:, order], u8(flat(ref["k8"]))), "k8"
    assert torch.equal(pq["sk"][bh0:bh1], flat(ref["sk"])), "sk"
    assert torch.equal(u8(pq["v8t"][bh0:bh1]), u8(flat(ref["v8"]).transpose(1, 2))), "v8t"
    assert torch.equal(pq["sv"][bh0:bh1], flat(ref["sv"])), "sv"
    assert torch.equal(pq["S"][bh0:bh1], flat(ref["S"])), "S"
    assert torch.equal(pq["svp"][bh0:bh1], flat(R.stage_sv(ref["svp"]))), "svp"
    assert torch.equal(pq["mean"][bh0:bh1], flat(ref["mean"])), "mean"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_video_length_prologue_bits(dtype):
    """Q8/SQ/K8/SK/V8T/SV/S/SVP/mean of all 48 heads at N=47520 with the x50 outlier tokens (the
    case per-token scales exist for): int8 codes for fp16 inputs, e4m3 for bf16."""
    q, k, v = _device_inputs(1, 48, N_VIDEO, dtype, seed=5)
    pq = be.quant_qkv(q, k, v)
    torch.cuda.synchronize()
    assert int(pq["ctrl"].view(torch.int32)[4 * 48].item()) == 0
    for h0 in range(0, 48, 8):                                  # the oracle, eight heads at a time
        ref = R.prologue(q[:, h0:h0 + 8], k[:, h0:h0 + 8], v[:, h0:h0 + 8], pad_multiple=128)
        _assert_prologue_bits(pq, ref, h0, h0 + 8)
    # an outlier token's scale is about 50 times its neighbours': per-token scales are in use
    sk = pq["sk"][0, :N_VIDEO]
    assert sk.max().item() > 20 * sk.median().item()


def test_scaling_configuration_b4():
    """B=4, H=48, N=47520, bf16, non-causal: the 192 (batch, head) units of the multi-GPU
    configuration in one call.  Prologue bits for every unit, attention for three of them."""
    b, h = 4, 48
    q, k, v = _device_inputs(b, h, N_VIDEO, torch.bfloat16, seed=9)
    pq = be.quant_qkv(q, k, v)
    torch.cuda.synchronize()
    assert int(pq["ctrl"].view(torch.int32)[4 * b * h].item()) == 0
    for bi in range(b):
        for h0 in range(0, h, 16):
            ref = R.prologue(q[bi:bi + 1, h0:h0 + 16], k[bi:bi + 1, h0:h0 + 16], v[bi:bi + 1, h0:h0 + 16],
                             pad_multiple=128)
            _assert_prologue_bits(pq, ref, bi * h + h0, bi * h + h0 + 16)
    del pq
    out = be.sage_call(q, k, v, is_causal=False)
    torch.cuda.synchronize()
    assert be.last_status(out, b, h, N_VIDEO) == 0
    assert torch.isfinite(out.float()).all()
    _compare_heads(out, q, k, v, [(0, 0), (3, 47)], False, tiles=(128,), wide_scores=True)
    _compare_heads(out, q, k, v, [(2, 17)], False, tiles=(64,), wide_scores=True)


def test_oracle_gives_the_same_bytes_on_cpu_and_on_the_device():
    """The comparisons above evaluate the oracle with torch on the device.  On the first
    configuration (B=1, H=4, N=512, fp16, K channel bias 0.5) that evaluation must reproduce the
    CPU evaluation: every prologue tensor bit for bit (all of its operations are correctly
    rounded or exact), and the attention output up to the last bits of exp2 and the fp32 summation
    order of P.V (the integer Q.K^T sums are exact in either order)."""
    q, k, v = R.make_inputs(1, 4, 512, 128, torch.float16, seed=0, k_bias_std=0.5)
    for dtype in (torch.float16, torch.bfloat16):
        qc, kc, vc = q.to(dtype), k.to(dtype), v.to(dtype)
        cpu = R.prologue(qc, kc, vc, pad_multiple=128)
        gpu = R.prologue(qc.cuda(), kc.cuda(), vc.cuda(), pad_multiple=128)
        for key in ("q8", "sq", "k8", "sk", "v8", "sv", "svp", "S", "mean"):
            a, b = cpu[key], gpu[key].cpu()
            assert a.dtype == b.dtype and a.shape == b.shape, key
            assert torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8)), (key, dtype)
        for causal in (False, True):
            o_cpu = R.sageattn_oracle(qc, kc, vc, is_causal=causal, tile=128).float()
            o_gpu = R.sageattn_oracle(qc.cuda(), kc.cuda(), vc.cuda(), is_causal=causal, tile=128).cpu().float()
            # exp2 and the fp32 sums differ in their last bits between the two evaluations; once in
            # a while that moves an e4m3 rounding of P, so single outputs may differ by more than an
            # ulp while the tensors agree to about 1e-5
            assert R.rel_l1(o_gpu, o_cpu) <= 2e-4
            assert (o_cpu - o_gpu).abs().max().item() <= 2.0 ** -6 * o_cpu.abs().max().item()
            assert R.cosine(o_gpu, o_cpu) >= 0.999999
