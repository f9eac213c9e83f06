"""`sageattn_varlen` as one call of the kernels (`sage_attention_varlen`).

The kernels read the cumulative lengths on the device; every sequence is quantised and attended
exactly as if it were passed alone, so the packed result must equal the per-sequence calls bit for
bit.  With the lengths on the device the call reads nothing back: it can be captured into a CUDA
graph, and a replay follows lengths written into the captured arrays afterwards.
"""
import pytest
import torch

import sageattention
from oracle import ref_numerics as R
from sageattention import b200_backend as be
from sageattention import core

pytestmark = pytest.mark.gpu

MAX_REL_RMS = 0.06


def _cu(lens, device="cuda", dtype=torch.int32):
    return torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=dtype).to(device)


def _packed(lens_q, lens_k, hq, hkv, dtype, seed, d=128):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(sum(lens_q), hq, d, generator=g).to(dtype).cuda()
    k = (torch.randn(sum(lens_k), hkv, d, generator=g) + 0.5 * torch.randn(1, hkv, d, generator=g)).to(dtype).cuda()
    v = torch.randn(sum(lens_k), hkv, d, generator=g).to(dtype).cuda()
    return q, k, v


def _per_sequence(q, k, v, lens_q, lens_k, causal, **kw):
    out = torch.full_like(q, float("nan"))
    a = c = 0
    for nq, nk in zip(lens_q, lens_k):
        if nq:
            one = sageattention.sageattn(q[a:a + nq].unsqueeze(0).contiguous(), k[c:c + nk].unsqueeze(0).contiguous(),
                                         v[c:c + nk].unsqueeze(0).contiguous(), tensor_layout="NHD",
                                         is_causal=causal, **kw)
            out[a:a + nq] = one[0]
        a, c = a + nq, c + nk
    return out


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
def test_device_lengths_match_per_sequence_calls(dtype, causal):
    lens_q = [1, 127, 128, 129, 0, 300, 1000, 64, 257]
    lens_k = lens_q if causal else [77, 128, 1, 300, 0, 129, 513, 1000, 256]
    q, k, v = _packed(lens_q, lens_k, 4, 2, dtype, seed=21)
    out = sageattention.sageattn_varlen(q, k, v, _cu(lens_q), _cu(lens_k, dtype=torch.int64),
                                        max(lens_q), max(lens_k), is_causal=causal)
    torch.cuda.synchronize()
    n_seq = len(lens_q)
    assert be.last_status(q, n_seq, 4, max(lens_q), 2, max(lens_k)) == 0
    want = _per_sequence(q, k, v, lens_q, lens_k, causal)
    assert torch.equal(out, want)
    a = c = 0
    for nq, nk in zip(lens_q, lens_k):                     # and each sequence is the right attention
        if nq:
            ref = R.sdpa_fp32(q[a:a + nq].transpose(0, 1).unsqueeze(0).cpu(),
                              k[c:c + nk].transpose(0, 1).unsqueeze(0).cpu().repeat_interleave(2, 1),
                              v[c:c + nk].transpose(0, 1).unsqueeze(0).cpu().repeat_interleave(2, 1),
                              is_causal=causal)
            assert R.rel_rms(out[a:a + nq].transpose(0, 1).unsqueeze(0).cpu(), ref) < MAX_REL_RMS
        a, c = a + nq, c + nk


def test_generous_length_bounds_change_nothing():
    """`max_seqlen` only sizes slots and grids: any bound at or above the longest sequence gives
    the same bits."""
    lens = [200, 31, 450]
    q, k, v = _packed(lens, lens, 2, 2, torch.float16, seed=4)
    cu = _cu(lens)
    tight = sageattention.sageattn_varlen(q, k, v, cu, cu, 450, 450, is_causal=True).clone()
    loose = sageattention.sageattn_varlen(q, k, v, cu, cu, 681, 681, is_causal=True)
    assert torch.equal(tight, loose)


def test_no_smoothing_and_scale_and_strided_inputs():
    lens_q, lens_k = [150, 20, 333], [90, 400, 128]
    q, k, v = _packed(lens_q, lens_k, 2, 2, torch.float16, seed=9)
    fused = torch.randn(sum(lens_k), 2, 2, 128, generator=torch.Generator().manual_seed(1)).half().cuda()
    k, v = fused[:, 0], fused[:, 1]                        # views with a token stride of 2 * H * D
    assert not k.is_contiguous()
    out = sageattention.sageattn_varlen(q, k, v, _cu(lens_q), _cu(lens_k), 333, 400, sm_scale=0.05, smooth_k=False)
    want = _per_sequence(q, k, v, lens_q, lens_k, False, sm_scale=0.05, smooth_k=False)
    assert torch.equal(out, want)


def test_a_sequence_does_not_see_its_neighbours():
    """The rows behind a sequence's last token belong to the next sequence.  Non-finite values
    there must not reach the sequence before (its padded key rows are zeroed by the prologue and
    masked by the kernel)."""
    lens = [100, 60, 200]
    q, k, v = _packed(lens, lens, 2, 2, torch.bfloat16, seed=13)
    cu = _cu(lens)
    clean = sageattention.sageattn_varlen(q, k, v, cu, cu, 200, 200).clone()
    k2, v2, q2 = k.clone(), v.clone(), q.clone()
    k2[100:160] = float("inf")
    v2[100:160] = float("nan")
    q2[100:160] = float("nan")
    dirty = sageattention.sageattn_varlen(q2, k2, v2, cu, cu, 200, 200)
    assert torch.equal(dirty[:100], clean[:100])
    assert torch.equal(dirty[160:], clean[160:])


def test_capture_once_replay_with_other_lengths():
    """Nothing is read back from the device: the call is capturable, and the captured kernels take
    whatever lengths the arrays hold at replay."""
    total, hq = 900, 2
    q, k, v = _packed([total], [total], hq, hq, torch.float16, seed=17)
    lens_a, lens_b = [300, 500, 100], [128, 129, 643]
    cu = _cu(lens_a)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        sageattention.sageattn_varlen(q, k, v, cu, cu, 700, 700, is_causal=True)      # warm-up
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            got = sageattention.sageattn_varlen(q, k, v, cu, cu, 700, 700, is_causal=True)
    torch.cuda.current_stream().wait_stream(s)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(got, _per_sequence(q, k, v, lens_a, lens_a, True))
    cu.copy_(_cu(lens_b))
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(got, _per_sequence(q, k, v, lens_b, lens_b, True))


def test_host_lengths_and_the_run_by_run_form_agree(monkeypatch):
    """Lengths given on the host are validated and then take the same single call; a batch too
    ragged for slots of the longest length is split into runs of equal lengths instead.  All three
    forms give the same bits."""
    lens_q, lens_k = [40, 40, 40, 700, 3], [64, 64, 64, 300, 900]
    q, k, v = _packed(lens_q, lens_k, 2, 1, torch.float16, seed=23)
    dev = sageattention.sageattn_varlen(q, k, v, _cu(lens_q), _cu(lens_k), 700, 900).clone()
    host = sageattention.sageattn_varlen(q, k, v, _cu(lens_q, "cpu"), _cu(lens_k, "cpu", torch.int64), 700, 900).clone()
    monkeypatch.setattr(core, "_VARLEN_SLOT_FACTOR", 0)
    monkeypatch.setattr(core, "_VARLEN_SLOT_FREE_BYTES", 0)
    runs = sageattention.sageattn_varlen(q, k, v, _cu(lens_q), _cu(lens_k), 700, 900)
    assert torch.equal(dev, host) and torch.equal(dev, runs)
    with pytest.raises(ValueError):
        sageattention.sageattn_varlen(q, k, v, _cu(lens_q, "cpu"), _cu(lens_k, "cpu"), 699, 900)


def test_queries_without_keys_get_zeros_and_long_sequences_are_cut():
    """What the device-side form does with lengths the host-side checks would have refused."""
    lens_q, lens_k = [50, 70], [0, 90]
    q, k, v = _packed(lens_q, lens_k, 2, 2, torch.float16, seed=29)
    out = be.sage_call_varlen(q, k, v, _cu(lens_q), _cu(lens_k), 70, 90)
    assert torch.count_nonzero(out[:50]).item() == 0
    one = sageattention.sageattn(q[50:].unsqueeze(0).contiguous(), k.unsqueeze(0).contiguous(),
                                 v.unsqueeze(0).contiguous(), tensor_layout="NHD")
    assert torch.equal(out[50:], one[0])
    # a bound below the longest sequence: its first `max` rows see its first `max` keys
    lens = [300]
    q, k, v = _packed(lens, lens, 1, 1, torch.float16, seed=31)
    out = torch.full_like(q, 7.0)
    be.sage_call_varlen(q, k, v, _cu(lens), _cu(lens), 200, 200, out=out)
    want = sageattention.sageattn(q[:200].unsqueeze(0).contiguous(), k[:200].unsqueeze(0).contiguous(),
                                  v[:200].unsqueeze(0).contiguous(), tensor_layout="NHD")
    assert torch.equal(out[:200], want[0])
    assert (out[200:] == 7.0).all()


def test_lengths_that_point_outside_the_packed_tensors_are_clamped():
    """The device-side lengths are the caller's promise, but the kernels keep every access inside
    the packed tensors whatever the arrays hold: starts and ends are clamped to the token counts.
    The output sits in the middle of a guarded buffer; the guards must stay untouched, and the
    sequences that are described correctly come out as usual."""
    lens = [120, 200, 80]
    q, k, v = _packed(lens, lens, 2, 2, torch.float16, seed=37)
    total = sum(lens)
    guard = 4096
    buf = torch.full((guard + total * 2 * 128 + guard,), 3.0, dtype=torch.float16, device="cuda")
    out = buf[guard: guard + total * 2 * 128].view(total, 2, 128)
    good = _cu(lens)
    want = sageattention.sageattn_varlen(q, k, v, good, good, 200, 200).clone()
    for bad in ([0, 120, 10 ** 9, 400],          # an end far beyond the tensor
                [0, -50, 320, 400],              # a negative entry
                [0, 500, 320, 400],              # a start beyond the tensor, then a decreasing entry
                [2 ** 31 - 1, 2 ** 31 - 1, 2 ** 31 - 1, 2 ** 31 - 1]):
        buf.fill_(3.0)
        cu = torch.tensor(bad, dtype=torch.int32, device="cuda")
        be.sage_call_varlen(q, k, v, cu, cu, 200, 200, out=out)
        torch.cuda.synchronize()
        assert (buf[:guard] == 3.0).all() and (buf[-guard:] == 3.0).all()
    # a batch whose last sequence is described wrongly still serves the first two
    buf.fill_(3.0)
    cu = torch.tensor([0, 120, 320, 10 ** 9], dtype=torch.int32, device="cuda")
    be.sage_call_varlen(q, k, v, cu, cu, 200, 200, out=out)
    torch.cuda.synchronize()
    assert torch.equal(out[:320], want[:320])
    assert (buf[:guard] == 3.0).all() and (buf[-guard:] == 3.0).all()
