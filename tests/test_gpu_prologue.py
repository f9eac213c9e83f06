"""Prologue parity on the GPU: codes and scales bit-exact against the oracle and the golden file.
All calls go through the C-ABI (ctypes)."""
import pytest
import torch

from conftest import bytes_equal
from oracle import ref_numerics as R
from sageattention import b200_backend as be

pytestmark = pytest.mark.gpu


def _check_against(pq_gpu, pq_ref, n, smooth):
    bh = pq_gpu["B"] * pq_gpu["H"]
    n_pad = pq_gpu["n_pad"]
    flat = lambda t: t.reshape(bh, *t.shape[2:]).cpu()
    assert bytes_equal(pq_gpu["q8"], flat(pq_ref["q8"])), "q8"
    assert torch.equal(pq_gpu["sq"].cpu(), flat(pq_ref["sq"])), "sq"
    k8_key_order = pq_gpu["k8"].cpu()[:, be.k8_row_order(n_pad)]       # stored permuted inside 16-key blocks
    assert bytes_equal(k8_key_order, flat(pq_ref["k8"])), "k8"
    assert torch.equal(pq_gpu["sk"].cpu(), flat(pq_ref["sk"])), "sk"
    v8t_ref = flat(pq_ref["v8"]).transpose(1, 2).contiguous()
    assert bytes_equal(pq_gpu["v8t"], v8t_ref), "v8t"
    assert torch.equal(pq_gpu["sv"].cpu(), flat(pq_ref["sv"])), "sv"
    assert torch.equal(pq_gpu["S"].cpu(), flat(pq_ref["S"])), "S"
    assert torch.equal(pq_gpu["svp"].cpu(), flat(R.stage_sv(pq_ref["svp"]))), "svp"
    if smooth:
        assert torch.equal(pq_gpu["mean"].cpu(), flat(pq_ref["mean"])), "mean"
    assert n_pad % 128 == 0


def test_golden_vectors(golden):
    g = golden
    q, k, v = g.q.cuda(), g.k.cuda(), g.v.cuda()
    pq = be.quant_qkv(q, k, v, smooth_k=g.smooth, int8=g.int8)
    ref = dict(g.ora)
    _check_against(pq, ref, g.N, g.smooth)


@pytest.mark.parametrize("n", [1, 15, 63, 64, 65, 127, 128, 129, 300, 1000])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("smooth", [True, False])
def test_edge_lengths(n, dtype, smooth):
    q, k, v = R.make_inputs(2, 3, n, 128, dtype, seed=n, k_bias_std=1.0)
    ref = R.prologue(q, k, v, smooth_k=smooth, pad_multiple=128)
    pq = be.quant_qkv(q.cuda(), k.cuda(), v.cuda(), smooth_k=smooth)
    _check_against(pq, ref, n, smooth)


def test_fp16_with_e4m3_codes():
    q, k, v = R.make_inputs(1, 2, 200, seed=8, k_bias_std=0.5)
    k[0, 1, 8, ::5] = -0.0
    q[0, 0, 3, ::2] = -0.0
    ref = R.prologue(q, k, v, smooth_k=True, int8=False, pad_multiple=128)
    pq = be.quant_qkv(q.cuda(), k.cuda(), v.cuda(), smooth_k=True, int8=False)
    _check_against(pq, ref, 200, True)


def test_outliers_zero_rows_and_large_v():
    q, k, v = R.make_inputs(1, 4, 500, seed=21, k_bias_std=1.0, outlier_frac=0.01)
    v[0, 1, 17] = 20000.0          # the reference's |V| = 20000 case: S > 1
    k[0, 2, 5] = 0
    q[0, 3, 9] = 0
    v[0, 0, 400] = 0
    v[0, 2, 7, ::3] = -0.0         # signed zeros must keep their sign bit in the e4m3 codes
    k[0, 1, 8, ::5] = -0.0
    q[0, 0, 3, ::2] = -0.0
    ref = R.prologue(q, k, v, pad_multiple=128)
    pq = be.quant_qkv(q.cuda(), k.cuda(), v.cuda())
    _check_against(pq, ref, 500, True)
    assert pq["S"].max().item() > 1.0


def test_strided_views_give_the_same_bytes():
    """NHD storage and a fused-QKV buffer read through strides equal the contiguous call."""
    b, h, n = 2, 3, 260
    q, k, v = R.make_inputs(b, h, n, seed=5, k_bias_std=0.7, device="cuda")
    base = be.quant_qkv(q, k, v)
    nhd = [t.transpose(1, 2).contiguous().transpose(1, 2) for t in (q, k, v)]
    fused = torch.empty(b, n, h, 3 * 128, dtype=q.dtype, device="cuda")
    views = []
    for i, t in enumerate((q, k, v)):
        fused[..., 128 * i:128 * (i + 1)] = t.transpose(1, 2)
        views.append(fused[..., 128 * i:128 * (i + 1)].transpose(1, 2))
    for alt in (nhd, views):
        got = be.quant_qkv(*alt)
        for key in ("q8", "sq", "k8", "sk", "v8t", "sv", "svp", "S", "mean"):
            assert bytes_equal(got[key], base[key]), key


def test_full_size_properties():
    """B=1,H=48,N=8771: size-independent checks (pad rows, code range, scale consistency) plus a
    bit-exact comparison with the same restatement evaluated by torch on the GPU."""
    q, k, v = R.make_inputs(1, 48, 8771, seed=0, k_bias_std=1.0, head_scale=True, device="cuda")
    pq = be.quant_qkv(q, k, v)
    n, n_pad = 8771, 8832
    assert pq["n_pad"] == n_pad
    k8 = pq["k8"][:, be.k8_row_order(n_pad, device="cuda")]           # key order
    assert torch.all(k8[:, n:] == 0) and torch.all(pq["sk"][:, n:] == 1.0)
    assert torch.all(pq["v8t"].view(torch.uint8)[:, :, n:] == 0) and torch.all(pq["sv"][:, n:] == 0)
    assert k8.abs().amax(dim=2)[:, :n].min().item() == 127            # every live row uses the range
    assert pq["q8"].abs().amax(dim=2).min().item() == 127
    ref = R.prologue(q, k, v, pad_multiple=128)                       # torch ops on the device
    _check_against(pq, ref, n, True)


@pytest.mark.parametrize("b,h,n", [(16, 40, 70), (3, 200, 129), (1, 1, 5000)])
def test_many_units_and_the_work_counter(b, h, n):
    """More (tensor, head, tile) items than persistent CTAs, and fewer: every item is quantised
    exactly once whatever order the CTAs draw them in, and the status word stays clear."""
    q, k, v = R.make_inputs(b, h, n, 128, torch.float16, seed=b + h + n, k_bias_std=0.3)
    ref = R.prologue(q, k, v, smooth_k=True, pad_multiple=128)
    pq = be.quant_qkv(q.cuda(), k.cuda(), v.cuda(), smooth_k=True)
    again = be.quant_qkv(q.cuda(), k.cuda(), v.cuda(), smooth_k=True, reuse=pq)     # same buffers, second run
    _check_against(again, ref, n, True)
    words = pq["ctrl"].view(torch.int32)
    assert int(words[4 * b * h].item()) == 0                                          # the quantiser's status word
    items = 2 * b * h * ((n + 127) // 128) + b * h * ((n + 127) // 128)
    counter = int(pq["ctrl"][4 * (4 * b * h + 2): 4 * (4 * b * h + 2) + 8].view(torch.int64).item())
    assert counter >= items                                                            # every item was drawn


def test_prologue_is_deterministic_across_runs():
    q, k, v = R.make_inputs(2, 6, 1500, 128, torch.bfloat16, seed=77, k_bias_std=0.5, device="cuda")
    a = be.quant_qkv(q, k, v)
    b = be.quant_qkv(q, k, v)
    for key in ("q8", "k8", "v8t"):
        assert bytes_equal(a[key], b[key].cpu()), key
    for key in ("sq", "sk", "sv", "svp", "S", "mean"):
        assert torch.equal(a[key], b[key]), key
