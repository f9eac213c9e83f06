"""Seeded random call shapes through the public API against the oracle and exact attention: every
combination of layout, dtype, code type, masking, grouped heads, lengths, head_dim and options that
the envelope admits can come up."""
import random

import pytest
import torch

from oracle import ref_numerics as R
from sageattention import b200_backend as be
import sageattention

pytestmark = pytest.mark.gpu


def _case(seed):
    rng = random.Random(seed)
    b = rng.choice([1, 1, 2, 3])
    hkv = rng.choice([1, 2, 3, 5])
    grp = rng.choice([1, 1, 2, 4])
    d = rng.choice([128, 128, 128, 64, 96, 32])
    causal = rng.random() < 0.4
    nq = rng.choice([1, 7, 64, 127, 128, 129, 200, 333, 511, 700])
    nk = nq if causal or rng.random() < 0.5 else rng.choice([1, 40, 128, 257, 600, 900])
    dtype = rng.choice([torch.float16, torch.bfloat16])
    layout = rng.choice(["HND", "NHD"])
    return dict(b=b, hq=hkv * grp, hkv=hkv, d=d, causal=causal, nq=nq, nk=nk, dtype=dtype, layout=layout,
                smooth_k=rng.random() < 0.8, smooth_v=rng.random() < 0.3, lse=rng.random() < 0.4,
                int8=(rng.random() < 0.7) if dtype == torch.float16 else None,
                sm_scale=rng.choice([None, None, 0.07]))


@pytest.mark.parametrize("seed", range(48))
def test_random_call(seed):
    c = _case(seed)
    g = torch.Generator().manual_seed(1000 + seed)
    q = torch.randn(c["b"], c["hq"], c["nq"], c["d"], generator=g).to(c["dtype"])
    k = (torch.randn(c["b"], c["hkv"], c["nk"], c["d"], generator=g)
         + 0.5 * torch.randn(1, c["hkv"], 1, c["d"], generator=g)).to(c["dtype"])
    v = (torch.randn(c["b"], c["hkv"], c["nk"], c["d"], generator=g)
         + (1.5 if c["smooth_v"] else 0.0) * torch.randn(1, c["hkv"], 1, c["d"], generator=g)).to(c["dtype"])
    dev = lambda t: (t.transpose(1, 2).contiguous() if c["layout"] == "NHD" else t).cuda()
    kwargs = dict(tensor_layout=c["layout"], is_causal=c["causal"], sm_scale=c["sm_scale"], smooth_k=c["smooth_k"],
                  smooth_v=c["smooth_v"], return_lse=c["lse"])
    if c["int8"] is not None:
        kwargs["sk1_int8"] = c["int8"]
    res = sageattention.sageattn(dev(q), dev(k), dev(v), **kwargs)
    out, lse = res if c["lse"] else (res, None)
    torch.cuda.synchronize()
    assert be.last_status(out, c["b"], c["hq"], c["nq"], c["hkv"], c["nk"]) == 0
    if c["layout"] == "NHD":
        out = out.transpose(1, 2)
    assert out.shape == q.shape and out.dtype == q.dtype
    want = R.sageattn_oracle(q, k, v, is_causal=c["causal"], sm_scale=c["sm_scale"], smooth_k=c["smooth_k"],
                             int8=c["int8"], tile=128, return_lse=c["lse"], smooth_v=c["smooth_v"])
    want_o, want_l = want if c["lse"] else (want, None)
    ref = R.sdpa_fp32(q, k, v, is_causal=c["causal"], sm_scale=c["sm_scale"])
    o = out.cpu()
    assert torch.isfinite(o.float()).all()
    # same numerics as the oracle: hardware exp2 and accumulation order differ in the last bits,
    # which flips a few e4m3 roundings of P; over a handful of output rows those flips are not
    # averaged out, so small outputs get the stated tolerance and large ones a tighter one
    big = o.numel() >= 32768
    assert R.cosine(o, want_o) >= (0.9999 if big else 0.9995), c
    assert R.rel_l1(o, want_o) <= (6e-3 if big else 2e-2), c
    # and no further from exact attention than the restated reference is
    assert R.rel_rms(o, ref) <= 1.05 * R.rel_rms(want_o, ref) + 2e-3, c
    if lse is not None:
        assert (lse.cpu() - want_l).abs().max().item() < 3e-3, c
