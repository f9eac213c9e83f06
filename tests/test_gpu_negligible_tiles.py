"""The attention kernels with the negligible-tile tests against the ones without.

A key tile is not exponentiated when, for all 16 query rows of a warp, every score of the tile lies
at least 40 (base-2 exponent units) below the row's running maximum: P is exactly zero for such a
tile either way, and the row sum loses at most 128 * 2^-40 of its largest term per tile.  The
tests select the kernels without the tests through `sage_debug_skip_threshold(0)` and compare:
  * on inputs with a few dominant keys (where most tiles are skipped) the outputs agree to the
    last bit of fp16/bf16 on all but a vanishing share of elements, and both are within the usual
    bounds of the oracle, which exponentiates everything;
  * on inputs without dominant keys nothing is skipped and the outputs are bit-identical.
"""
import pytest
import torch

from oracle import ref_numerics as R
from sageattention import _native
from sageattention import b200_backend as be

pytestmark = pytest.mark.gpu

COS_SAME, L1_SAME = 0.9999, 5e-3


@pytest.fixture
def threshold():
    """The threshold hook; while a test runs, every call keeps the tests on (no switching to the
    plain kernels from the counts of earlier calls)."""
    lib = _native.load()
    adaptive, be._ADAPTIVE = be._ADAPTIVE, False
    yield lib.sage_debug_skip_threshold
    lib.sage_debug_skip_threshold(-1.0)          # back to the default
    be._ADAPTIVE = adaptive


def _both(threshold, q, k, v, causal, **kw):
    threshold(0.0)
    off = be.sage_call(q, k, v, is_causal=causal, **kw)
    off = (off[0].clone(), off[1].clone()) if isinstance(off, tuple) else off.clone()
    threshold(-1.0)
    on = be.sage_call(q, k, v, is_causal=causal, **kw)
    torch.cuda.synchronize()
    b, h, n = q.shape[0], q.shape[1], q.shape[2]
    assert be.last_status(q, b, h, n, k.shape[1], k.shape[2]) == 0
    return on, off


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("n", [1000, 4096])
def test_dominant_keys(threshold, dtype, causal, n):
    """1 % of the keys scaled x50: after the first of them most tiles are far below the maxima."""
    q, k, v = R.make_inputs(2, 3, n, 128, dtype, seed=n, outlier_frac=0.01, device="cuda")
    on, off = _both(threshold, q, k, v, causal)
    diff = (on.float() - off.float()).abs()
    ulp = (2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7) * off.float().abs().clamp_min(2.0 ** -14)
    assert (diff <= ulp).all()                                   # never more than the last bit
    assert (on != off).float().mean().item() < 1e-3
    want = R.sageattn_oracle(q, k, v, is_causal=causal, tile=128)
    for got in (on, off):
        assert R.rel_l1(got, want) <= L1_SAME * (1 if dtype == torch.float16 else 4)
    assert abs(R.rel_l1(on, want) - R.rel_l1(off, want)) < 1e-5


@pytest.mark.parametrize("shape", [1, 2])
@pytest.mark.parametrize("dtype,causal", [(torch.float16, False), (torch.float16, True), (torch.bfloat16, False)])
def test_both_kernel_shapes_skip_alike(threshold, shape, dtype, causal):
    """The one-tile and the two-tile shape of the kernel carry the same tests: each, forced, agrees
    with its own plain instantiation on inputs where most tiles are skipped."""
    lib = _native.load()
    q, k, v = R.make_inputs(1, 4, 3000, 128, dtype, seed=77, outlier_frac=0.01, device="cuda")
    lib.sage_debug_tiles_per_cta(shape)
    try:
        on, off = _both(threshold, q, k, v, causal)
    finally:
        lib.sage_debug_tiles_per_cta(0)
    ulp = (2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7) * off.float().abs().clamp_min(2.0 ** -14)
    assert ((on.float() - off.float()).abs() <= ulp).all()
    assert (on != off).float().mean().item() < 1e-3


def test_nothing_is_skipped_without_dominant_keys(threshold):
    q, k, v = R.make_inputs(1, 4, 3000, 128, torch.float16, seed=5, k_bias_std=0.5, device="cuda")
    on, off = _both(threshold, q, k, v, False)
    assert torch.equal(on, off)
    on, off = _both(threshold, q, k, v, True)
    assert torch.equal(on, off)


def test_one_row_that_is_not_dominated_keeps_the_tile(threshold):
    """Fifteen rows of a warp see a huge key, the sixteenth is orthogonal to it: the tiles after
    that key hold that row's largest scores, so none of them may be dropped for the warp."""
    n = 1024
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 1, n, 128, generator=g)
    k = torch.randn(1, 1, n, 128, generator=g)
    v = torch.randn(1, 1, n, 128, generator=g)
    k[0, 0, 5] = 60.0 * q[0, 0, 0] / q[0, 0, 0].norm() * 11.3       # a key every row like q[0] loves
    q[0, 0, :16] = q[0, 0, 0] + 0.01 * q[0, 0, :16]
    kd = k[0, 0, 5] / k[0, 0, 5].norm()
    q[0, 0, 7] = q[0, 0, 7] - (q[0, 0, 7] @ kd) * kd - 0.5 * kd      # row 7 dislikes that key
    q, k, v = q.half().cuda(), k.half().cuda(), v.half().cuda()
    on, off = _both(threshold, q, k, v, False, smooth_k=False)
    want = R.sageattn_oracle(q, k, v, smooth_k=False, tile=128)
    assert (on.float() - off.float()).abs().max().item() <= 2e-3
    assert R.cosine(on[0, 0, 7], want[0, 0, 7]) >= 0.99 and R.cosine(off[0, 0, 7], want[0, 0, 7]) >= 0.99
    assert R.cosine(on, want) >= 0.999


def test_log_sum_exp_and_grouped_heads_with_skipped_tiles(threshold):
    q, k, v = R.make_inputs(1, 4, 2500, 128, torch.float16, seed=8, outlier_frac=0.01, device="cuda")
    k, v = k[:, :2].contiguous(), v[:, :2].contiguous()
    (on, lse_on), (off, lse_off) = _both(threshold, q, k, v, False, return_lse=True)
    assert (on.float() - off.float()).abs().max().item() <= 2e-3
    assert (lse_on - lse_off).abs().max().item() <= 1e-5 * lse_off.abs().max().item() + 1e-5


def test_threshold_hook_round_trip(threshold):
    """A large threshold skips nothing (bit-identical to off); the default is restored by -1."""
    q, k, v = R.make_inputs(1, 2, 1500, 128, torch.float16, seed=2, outlier_frac=0.02, device="cuda")
    threshold(0.0)
    off = be.sage_call(q, k, v).clone()
    threshold(1.0e30)
    huge = be.sage_call(q, k, v).clone()
    torch.cuda.synchronize()
    assert torch.equal(off, huge)


def test_skipped_pairs_are_counted_and_steer_the_choice_of_kernels():
    """The kernels with the tests count the (warp, key tile) pairs they skip; the host reads the
    count of a probing call without synchronising and sends a signature that skips nothing to
    the kernels without the tests.  Outputs are identical either way when nothing is skipped."""
    lib = _native.load()
    saved = be._ADAPTIVE
    be._ADAPTIVE = True
    try:
        be.clear_workspaces()
        dense = R.make_inputs(1, 4, 2048, 128, torch.float16, seed=31, device="cuda")
        # every query likes key 0 far more than any other key: all later key tiles are negligible
        g = torch.Generator().manual_seed(32)
        u = torch.randn(128, generator=g)
        qp = u + 0.5 * torch.randn(1, 4, 2304, 128, generator=g)
        kp = torch.randn(1, 4, 2304, 128, generator=g)
        kp[:, :, 0] = 4.0 * u
        peaky = tuple(t.half().cuda() for t in (qp, kp, torch.randn(1, 4, 2304, 128, generator=g)))
        first = be.sage_call(*dense).clone()                      # the probe for this signature
        torch.cuda.synchronize()
        outs = [be.sage_call(*dense).clone() for _ in range(3)]   # picks the result up, then plain kernels
        torch.cuda.synchronize()
        st = be._state(dense[0].device, torch.cuda.current_stream().cuda_stream, create=False)
        assert st.last_share == 0.0
        assert sum(1 for v in st.adaptive.plain_left.values() if v > 0) == 1
        assert all(torch.equal(first, o) for o in outs)
        a = be.sage_call(*peaky).clone()
        torch.cuda.synchronize()
        b = be.sage_call(*peaky).clone()
        torch.cuda.synchronize()
        assert st.last_share is not None and st.last_share > 0.5          # most pairs were skipped
        assert sum(1 for v in st.adaptive.plain_left.values() if v > 0) == 1   # still only the dense signature
        assert torch.equal(a, b)
    finally:
        be._ADAPTIVE = saved
        be.clear_workspaces()
