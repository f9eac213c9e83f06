"""The attention kernel's two shapes -- one or two 128-query tiles per CTA -- must agree bit for bit:
both compute a row with the same instructions in the same order, only the scheduling differs.  The
automatic choice takes two tiles only for large calls, so the small cases here force
each shape through `sage_debug_tiles_per_cta` and compare; the forced two-tile result is also held
against the oracle."""
import pytest
import torch

from oracle import ref_numerics as R
from sageattention import _native
from sageattention import b200_backend as be

pytestmark = pytest.mark.gpu


@pytest.fixture
def force_shape():
    lib = _native.load()
    yield lib.sage_debug_tiles_per_cta
    lib.sage_debug_tiles_per_cta(0)


def _inputs(b, hq, hkv, nq, nk, d, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, hq, nq, d, generator=g).to(dtype)
    k = (torch.randn(b, hkv, nk, d, generator=g) + 0.5 * torch.randn(1, hkv, 1, d, generator=g)).to(dtype)
    v = torch.randn(b, hkv, nk, d, generator=g).to(dtype)
    return q, k, v


CASES = [
    # b, hq, hkv, nq, nk, d, dtype, int8, smooth_v
    (1, 4, 4, 300, 300, 128, torch.float16, True, False),     # 3 query tiles: the last CTA's second tile is empty
    (2, 8, 2, 513, 1000, 128, torch.bfloat16, True, False),   # grouped heads, ragged last tile on both sides
    (1, 2, 2, 256, 129, 64, torch.float16, True, False),      # exactly two tiles, head_dim 64
    (1, 3, 3, 1024, 1024, 128, torch.bfloat16, False, False), # e4m3 Q/K codes
    (1, 4, 2, 700, 515, 128, torch.float16, True, True),      # smooth_v
    (3, 1, 1, 129, 4096, 128, torch.float16, True, False),    # one row in the second tile, many key tiles
]


@pytest.mark.parametrize("b,hq,hkv,nq,nk,d,dtype,int8,smooth_v", CASES)
def test_both_shapes_agree_bit_for_bit(force_shape, b, hq, hkv, nq, nk, d, dtype, int8, smooth_v):
    q, k, v = (t.cuda() for t in _inputs(b, hq, hkv, nq, nk, d, dtype, nq + nk))
    results = []
    for n in (1, 2):
        force_shape(n)
        out, lse = be.sage_call(q, k, v, is_causal=False, int8=int8, return_lse=True, smooth_v=smooth_v)
        torch.cuda.synchronize()
        assert be.last_status(out, b, hq, nq, hkv, nk) == 0
        results.append((out.clone(), lse.clone()))
    assert torch.equal(results[0][0], results[1][0])
    assert torch.equal(results[0][1], results[1][1])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_two_tile_shape_against_the_oracle(force_shape, dtype):
    q, k, v = _inputs(2, 3, 3, 640, 640, 128, dtype, 7)
    force_shape(2)
    out = be.sage_call(q.cuda(), k.cuda(), v.cuda(), is_causal=False)
    torch.cuda.synchronize()
    assert be.last_status(out, 2, 3, 640) == 0
    want = R.sageattn_oracle(q, k, v, is_causal=False, tile=128)
    # same tolerances as the one-tile parity tests: same quantised operands, fp32 order differs
    assert R.cosine(out.cpu(), want) >= 0.9999
    assert R.rel_l1(out.cpu(), want) <= 5e-3


@pytest.mark.parametrize("b,hq,hkv,n,d,dtype,int8", [
    (1, 2, 2, 400, 128, torch.float16, True),      # 4 query tiles, ragged diagonal tile
    (2, 6, 3, 641, 128, torch.bfloat16, True),     # 6 tiles, one row in the last; grouped heads
    (1, 3, 3, 300, 64, torch.float16, True),       # 3 tiles: the longest CTA's second tile does not exist
    (1, 2, 2, 1280, 128, torch.bfloat16, False),   # e4m3 Q/K codes
    (1, 1, 1, 129, 128, torch.float16, True),      # 2 tiles, one row in the second
])
def test_both_shapes_agree_bit_for_bit_when_causal(force_shape, b, hq, hkv, n, d, dtype, int8):
    q, k, v = (t.cuda() for t in _inputs(b, hq, hkv, n, n, d, dtype, n))
    results = []
    for shape in (1, 2):
        force_shape(shape)
        out, lse = be.sage_call(q, k, v, is_causal=True, int8=int8, return_lse=True)
        torch.cuda.synchronize()
        assert be.last_status(out, b, hq, n, hkv, n) == 0
        results.append((out.clone(), lse.clone()))
    assert torch.equal(results[0][0], results[1][0])
    assert torch.equal(results[0][1], results[1][1])


def test_two_tile_shape_against_the_oracle_when_causal(force_shape):
    q, k, v = _inputs(1, 3, 3, 700, 700, 128, torch.float16, 5)
    force_shape(2)
    out = be.sage_call(q.cuda(), k.cuda(), v.cuda(), is_causal=True)
    torch.cuda.synchronize()
    assert be.last_status(out, 1, 3, 700) == 0
    want = R.sageattn_oracle(q, k, v, is_causal=True, tile=128)
    assert R.cosine(out.cpu(), want) >= 0.9999
    assert R.rel_l1(out.cpu(), want) <= 5e-3


def test_automatic_choice_serves_a_call_large_enough_for_two_tiles():
    # 8 heads x 40 query tiles: 160 two-tile CTAs >= the SM count, so this runs the two-tile shape
    # without being forced; parity as everywhere else
    q, k, v = _inputs(1, 8, 8, 5120, 512, 128, torch.float16, 11)
    out = be.sage_call(q.cuda(), k.cuda(), v.cuda(), is_causal=False)
    torch.cuda.synchronize()
    assert be.last_status(out, 1, 8, 5120, 8, 512) == 0
    want = R.sageattn_oracle(q, k, v, is_causal=False, tile=128)
    assert R.cosine(out.cpu(), want) >= 0.9999
    assert R.rel_l1(out.cpu(), want) <= 5e-3


@pytest.mark.parametrize("seed", range(24))
def test_shapes_agree_on_random_calls(force_shape, seed):
    """Seeded random call shapes (lengths, head counts, grouping, head_dim, dtype, causal, code type,
    smooth_v): the two kernel shapes must return the same bits."""
    g = torch.Generator().manual_seed(1000 + seed)
    ri = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g).item())
    causal = bool(ri(0, 1))
    hkv = ri(1, 3)
    hq = hkv * ri(1, 3)
    nq = ri(129, 1100)
    nk = nq if causal else ri(1, 1100)
    d = (128, 128, 64, 96, 40)[ri(0, 4)]
    dtype = (torch.float16, torch.bfloat16)[ri(0, 1)]
    int8 = bool(ri(0, 3))
    smooth_v = bool(ri(0, 1))
    b = ri(1, 2)
    q, k, v = (t.cuda() for t in _inputs(b, hq, hkv, nq, nk, d, dtype, seed))
    results = []
    for shape in (1, 2):
        force_shape(shape)
        out, lse = be.sage_call(q, k, v, is_causal=causal, int8=int8, return_lse=True, smooth_v=smooth_v)
        torch.cuda.synchronize()
        assert be.last_status(out, b, hq, nq, hkv, nk) == 0
        results.append((out.clone(), lse.clone()))
    assert torch.isfinite(results[0][0].float()).all()
    assert torch.equal(results[0][0], results[1][0])
    assert torch.equal(results[0][1], results[1][1])


@pytest.mark.parametrize("shape", [1, 2])
def test_a_failure_already_reported_makes_every_cta_return_at_once(force_shape, shape):
    """The status word is how a CTA whose bounded wait gave up tells the others; CTAs that start
    with it non-zero must leave without touching the output (and release their TMEM, so that the
    next launch runs).  Nothing waits here: the word is simply set by the host before the launch."""
    q, k, v = (t.cuda() for t in _inputs(1, 2, 2, 512, 512, 128, torch.float16, 9))
    pq = be.quant_qkv(q, k, v)
    out = torch.full_like(q, 7.0)
    status = torch.full((1,), 4, dtype=torch.int32, device="cuda")
    force_shape(shape)
    be.attn_launch(pq, out, False, 128 ** -0.5, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 4
    assert bool((out == 7.0).all())
    status.zero_()
    be.attn_launch(pq, out, False, 128 ** -0.5, status=status)      # the same SMs serve the next launch
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    force_shape(0)
    want = be.sage_call(q, k, v, is_causal=False)
    assert torch.equal(out, want)
