"""CPU restatement of the reference's quantize-then-attend numerics.  TEST INFRASTRUCTURE ONLY.

This file is the checker, never the product: only the test-suite, the smoke check and the
benchmark's CPU-baseline leg may import it.  The shipped `sageattention` package never does and
fails loudly when its CUDA library is missing.

Every function restates, operation by operation, one piece of the reference (citations are paths
inside the reference project):

  kseq_mean        kernels/hip/h34_prologue.hip:259-282   fp64 sequence mean of K (smooth_k)
  quant_k          kernels/hip/h34_prologue.hip:116-166   per-token int8 / e4m3 K, pad rows
  quant_v          kernels/hip/h34_prologue.hip:168-211   per-token e4m3 V, pad rows
  fold_v_scale     sageattention/sk1_backend/__init__.py:561-579   S = max(max sv, 1), sv /= S
  quant_q          kernels/hip/sk1_t6i.hip:91-117 (int8), kernels/hip/sk1_t4a1sb.hip:73-100 (e4m3)
  attend           kernels/hip/sk1_t6i.hip:151-299        64-key tiles, running max, e4m3 P fold
  sageattn_oracle  sageattention/sk1_backend/__init__.py:982-1284   the whole call

Parity status: the reference ships no golden vectors for this path (its tests compare against fp32
SDPA with a tolerance).  The K/V row quantisers here are pinned against the reference's own
PyTorch checkers `ref_quant_row_i8` / `ref_quant_row_fp8`
(sageattention/sk1_backend/quant_triton.py:1128-1156), imported from the reference when the
fixtures under tests/golden/ were generated; the S fold and the padded length are pinned against
the reference's own `fold_v_scale` and `n_pad_for`, whose source was executed at the same time.
The Q quantiser, the mean and the attention loop have no runnable counterpart outside AMD
hardware: for those parity is pinned by the source-level arithmetic only ("parity unpinned" by any
reference-produced vector).

All arithmetic is separate, correctly rounded fp32 operations unless stated; the code is plain
torch so it runs on CPU (the oracle proper) and, unchanged, on a CUDA device when a test needs the
same restatement at sizes eight host cores cannot finish.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

LOG2E = 1.4426950408889634  # the reference's constant, rounded to fp32 at use (sk1_t6i.hip:109)
I8_MAX = 127.0
F8_MAX = 448.0              # e4m3 maximum and the reference's P_SCALE
FLOOR = 1e-12               # scale floor (hip_prologue.py:188, h34_prologue.hip:147,185)
REF_BN = 64                 # keys per tile of the reference's loop (sk1_t6i.hip:162)
E4M3 = torch.float8_e4m3fn


def _f32(x: float, device) -> torch.Tensor:
    return torch.tensor(x, dtype=torch.float32, device=device)


def pad_len(n: int, multiple: int = REF_BN) -> int:
    """Padded key length.  The reference pads to 64 (hip_prologue.py:93-95)."""
    return (n + multiple - 1) // multiple * multiple


def e4m3_rne(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3, round to nearest even.  Callers clamp first; torch's cast then agrees with
    both the AMD pack instruction and NVIDIA's saturating convert for every finite |x| <= 448."""
    return x.to(E4M3)


def kseq_mean(k: torch.Tensor) -> torch.Tensor:
    """mean[b,h,d] = f32( (sum_n f64(K[b,h,n,d])) / f64(N) ), summed the reference's way: eight
    partial sums over n = y, y+8, ... (each in increasing n), combined in index order
    (h34_prologue.hip:272-281).  `k` is logical (B,H,N,D)."""
    n = k.shape[2]
    kd = k.double()
    total = torch.zeros(k.shape[0], k.shape[1], k.shape[3], dtype=torch.float64, device=k.device)
    for y in range(8):
        part = kd[:, :, y::8, :]
        if part.shape[2] == 0:
            continue
        # cumsum is a sequential left-to-right sum, like the kernel's loop
        total = total + part.cumsum(dim=2)[:, :, -1, :]
    return (total / float(n)).float()


def _pad_rows(x: torch.Tensor, n_pad: int) -> torch.Tensor:
    b, h, n, d = x.shape
    if n_pad == n:
        return x
    out = torch.zeros(b, h, n_pad, d, dtype=x.dtype, device=x.device)
    out[:, :, :n] = x
    return out


def quant_k(k: torch.Tensor, mean: Optional[torch.Tensor], n_pad: int, int8: bool
            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """K -> (K8 (B,H,n_pad,D) int8|e4m3, SK (B,H,n_pad) f32).

    x = f32(k) - mean (live rows), amax = max_d|x|, sk = max(amax/127, 1e-12) [int8] or
    max(amax/448, 1e-12) [e4m3]; int8 code = clamp(RNE(x / sk), -128, 127) with a true division;
    e4m3 code = e4m3(min(x / sk, 448)) (upper clamp only).  Pad rows: code 0, SK = 1.0
    (h34_prologue.hip:116-166)."""
    b, h, n, d = k.shape
    x = k.float()
    if mean is not None:
        x = x - mean[:, :, None, :]
    amax = x.abs().amax(dim=3)
    qmax = I8_MAX if int8 else F8_MAX
    sk = torch.maximum(amax / _f32(qmax, k.device), _f32(FLOOR, k.device))
    y = x / sk[..., None]
    if int8:
        codes = torch.round(y).clamp_(-128.0, 127.0).to(torch.int8)
    else:
        codes = e4m3_rne(torch.minimum(y, _f32(F8_MAX, k.device)))
    k8 = _pad_rows(codes, n_pad)
    sk_out = torch.ones(b, h, n_pad, dtype=torch.float32, device=k.device)
    sk_out[:, :, :n] = sk
    return k8, sk_out


def quant_v(v: torch.Tensor, n_pad: int, mean: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """V -> (V8 (B,H,n_pad,D) e4m3 in token-major order, SV (B,H,n_pad) f32).  With `mean`
    (B,H,D), upstream's smooth_v (sageattention/quant.py:297-301), f32(V) - mean is quantised.

    sv = max(max_d|v| / 448, 1e-12); code = e4m3(min(v / sv, 448)); pad rows: code 0, SV = 0.0
    (h34_prologue.hip:168-211).  The reference stores the codes transposed, (B*H, D, n_pad);
    `v8.transpose(2, 3)` gives that view."""
    b, h, n, d = v.shape
    x = v.float()
    if mean is not None:
        x = x - mean[:, :, None, :]
    amax = x.abs().amax(dim=3)
    sv = torch.maximum(amax / _f32(F8_MAX, v.device), _f32(FLOOR, v.device))
    codes = e4m3_rne(torch.minimum(x / sv[..., None], _f32(F8_MAX, v.device)))
    v8 = _pad_rows(codes, n_pad)
    sv_out = torch.zeros(b, h, n_pad, dtype=torch.float32, device=v.device)
    sv_out[:, :, :n] = sv
    return v8, sv_out


def fold_v_scale(sv: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(SV' = SV / S, S) with S[b,h] = max(max_n SV[b,h,n], 1.0)
    (sageattention/sk1_backend/__init__.py:577-579).  Returns new tensors."""
    s = sv.amax(dim=2).clamp_min(1.0)
    return sv / s[..., None], s


def stage_sv(svp: torch.Tensor) -> torch.Tensor:
    """The factor the kernel multiplies P by: f32(SV' * 448) (sk1_t6i.hip:132)."""
    return svp * _f32(F8_MAX, svp.device)


def quant_q(q: torch.Tensor, int8: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Q -> (Q8 (B,H,N,D), SQ (B,H,N) f32).  Unlike K this multiplies by a reciprocal:
    amax = max(max_d|q|, 1e-12); qinv = 127/amax; code = clamp(rint(f32(q) * qinv), -128, 127);
    the dequant scale is amax/127 (sk1_t6i.hip:104-117).  e4m3 arm: qinv = 448/amax,
    code = e4m3(clamp(q * qinv, -448, 448)), scale amax/448 (sk1_t4a1sb.hip:89-100)."""
    x = q.float()
    amax = torch.maximum(x.abs().amax(dim=3), _f32(FLOOR, q.device))
    qmax = _f32(I8_MAX if int8 else F8_MAX, q.device)
    qinv = qmax / amax
    y = x * qinv[..., None]
    if int8:
        codes = torch.round(y).clamp_(-128.0, 127.0).to(torch.int8)
    else:
        codes = e4m3_rne(y.clamp_(-F8_MAX, F8_MAX))
    return codes, amax / qmax


def row_score_scale(sq: torch.Tensor, sm_scale: float) -> torch.Tensor:
    """c_q = f32( f32(sm_scale * LOG2E) * sq ), evaluated left to right (sk1_t6i.hip:109)."""
    c = _f32(sm_scale, sq.device) * _f32(LOG2E, sq.device)
    return c * sq


def attend(q8: torch.Tensor, sq: torch.Tensor, k8: torch.Tensor, sk: torch.Tensor,
           v8: torch.Tensor, svp: torch.Tensor, s_fold: torch.Tensor, n: int, causal: bool,
           sm_scale: float, out_dtype: torch.dtype, tile: int = REF_BN,
           row_chunk: int = 2048, row0: int = 0, return_lse: bool = False,
           vmean: Optional[torch.Tensor] = None):
    """The attention loop of sk1_t6i.hip:151-299 on already-quantised operands.

    q8 (B,H,R,D), sq (B,H,R) hold the query rows row0 .. row0+R-1 (all N rows by default); k8, v8
    (B,H,n_pad,D) with n_pad a multiple of `tile`; sk, svp (B,H,n_pad) where svp = SV / S;
    s_fold (B,H); `n` is the number of live keys.  Per query row, tiles of `tile` keys in
    increasing order: integer (or fp32 for e4m3 codes) dot products, s = f32(t) * f32(c_q * sk),
    mask, one running-max update per tile, p = exp2(s - m), l = l*alpha + sum(p) taken BEFORE
    the fold, p8 = e4m3(p * f32(svp*448)), acc = acc*alpha + p8 @ v8 in fp32; epilogue
    acc * (S / (l*448)).  `exp2` here is torch's, the kernels use hardware approximations: the
    output is a tolerance target, not a bit target.

    Beyond the reference's hand-written path (which refuses these shapes): k8/v8 may have fewer
    heads than q8 (grouped-query attention; every group of Hq/Hkv query heads shares a K/V head),
    the number of keys may differ from the number of queries when not causal, and with
    `return_lse` the function also returns ln2 * (m + log2 l), the log-sum-exp of the
    mean-subtracted logits (callers add sm_scale * q.mean(K) for the caller's K).  `vmean`
    (B,Hkv,D), the mean that smooth_v subtracted from V, is added to every output row in fp32
    before the cast (sk1_t6i.hip:297 `acc*inv + vm`)."""
    prev_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        b, h, nq, d = q8.shape
        n_pad = k8.shape[2]
        assert n_pad % tile == 0 and (not causal or row0 + nq <= n)
        if k8.shape[1] != h:                                  # grouped-query attention
            g = h // k8.shape[1]
            k8, v8 = k8.repeat_interleave(g, dim=1), v8.repeat_interleave(g, dim=1)
            sk, svp = sk.repeat_interleave(g, dim=1), svp.repeat_interleave(g, dim=1)
            s_fold = s_fold.repeat_interleave(g, dim=1)
            vmean = vmean.repeat_interleave(g, dim=1) if vmean is not None else None
        dev = q8.device
        kf = k8.float()
        vf = v8.float()
        stage = stage_sv(svp)
        cq_all = row_score_scale(sq, sm_scale)
        out = torch.empty(b, h, nq, d, dtype=out_dtype, device=dev)
        lse = torch.empty(b, h, nq, dtype=torch.float32, device=dev)
        neg_inf = _f32(float("-inf"), dev)
        for r0 in range(0, nq, row_chunk):
            r1 = min(nq, r0 + row_chunk)
            qf = q8[:, :, r0:r1].float()
            cq = cq_all[:, :, r0:r1]
            rows = torch.arange(row0 + r0, row0 + r1, device=dev)
            m = torch.full((b, h, r1 - r0), float("-inf"), dtype=torch.float32, device=dev)
            l = torch.zeros(b, h, r1 - r0, dtype=torch.float32, device=dev)
            acc = torch.zeros(b, h, r1 - r0, d, dtype=torch.float32, device=dev)
            # the reference visits tiles j < min(n_tiles, 2c+2) for the CTA owning 128 queries
            # (sk1_t6i.hip:88); tiles past the last query of the chunk are fully masked anyway
            last_key = (row0 + r1 - 1) if causal else (n - 1)
            for j in range(0, last_key // tile + 1):
                c0, c1 = j * tile, (j + 1) * tile
                t = torch.matmul(qf, kf[:, :, c0:c1].transpose(2, 3))
                s = t * (cq[..., None] * sk[:, :, None, c0:c1])
                keys = torch.arange(c0, c1, device=dev)
                if causal:
                    s = torch.where(keys[None, :] > rows[:, None], neg_inf, s)
                elif c1 > n:
                    s = torch.where((keys >= n)[None, :], neg_inf, s)
                m_new = torch.maximum(m, s.amax(dim=3))
                m_use = torch.where(torch.isinf(m_new) & (m_new < 0), torch.zeros_like(m_new), m_new)
                alpha = torch.exp2(m - m_use)
                m = m_new
                p = torch.exp2(s - m_use[..., None])
                l = l * alpha + p.sum(dim=3)
                p8 = e4m3_rne(p * stage[:, :, None, c0:c1]).float()
                acc = acc * alpha[..., None] + torch.matmul(p8, vf[:, :, c0:c1])
            inv = torch.where(l > 0, s_fold[..., None] / (l * _f32(F8_MAX, dev)), torch.zeros_like(l))
            res = acc * inv[..., None]
            if vmean is not None:
                res = res + vmean[:, :, None, :]
            out[:, :, r0:r1] = res.to(out_dtype)
            lse[:, :, r0:r1] = math.log(2.0) * (m + torch.log2(l))
        return (out, lse) if return_lse else out
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev_tf32


def prologue(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, smooth_k: bool = True,
             int8: Optional[bool] = None, pad_multiple: int = REF_BN, smooth_v: bool = False) -> dict:
    """The whole quantisation prologue on logical (B,H,N,D) tensors.  `int8=None` picks the
    reference's default: int8 Q.K for fp16 inputs, e4m3 Q.K for bf16
    (sageattention/sk1_backend/__init__.py:1045-1060)."""
    if int8 is None:
        int8 = q.dtype == torch.float16
    n = k.shape[2]
    n_pad = pad_len(n, pad_multiple)
    mean = kseq_mean(k) if smooth_k else None
    q8, sq = quant_q(q, int8)
    k8, sk = quant_k(k, mean, n_pad, int8)
    vmean = kseq_mean(v) if smooth_v else None      # same fp64 accumulation as the K mean
    v8, sv = quant_v(v, n_pad, vmean)
    svp, s_fold = fold_v_scale(sv)
    return dict(q8=q8, sq=sq, k8=k8, sk=sk, v8=v8, sv=sv, svp=svp, S=s_fold, mean=mean, vmean=vmean,
                n=n, n_pad=n_pad, int8=int8)


def sageattn_oracle(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                    is_causal: bool = False, sm_scale: Optional[float] = None,
                    smooth_k: bool = True, int8: Optional[bool] = None,
                    tile: int = REF_BN, return_lse: bool = False, smooth_v: bool = False):
    """The reference call end to end (sageattention/sk1_backend/__init__.py:982-1284): output has
    q's shape, dtype and layout; sm_scale defaults to D**-0.5 (:1165)."""
    if tensor_layout == "NHD":
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
    elif tensor_layout != "HND":
        raise ValueError("tensor_layout must be HND or NHD")
    d = q.shape[3]
    if sm_scale is None:
        sm_scale = d ** -0.5
    pq = prologue(q, k, v, smooth_k=smooth_k, int8=int8, pad_multiple=tile, smooth_v=smooth_v)
    res = attend(pq["q8"], pq["sq"], pq["k8"], pq["sk"], pq["v8"], pq["svp"], pq["S"], pq["n"],
                 is_causal, float(sm_scale), q.dtype, tile=tile, return_lse=return_lse, vmean=pq["vmean"])
    out = res[0] if return_lse else res
    if tensor_layout == "NHD":
        out = out.transpose(1, 2)
    if not return_lse:
        return out
    lse = res[1]
    if smooth_k:   # the logits of the caller's K differ from the mean-subtracted ones by q.mean per row
        g = q.shape[1] // k.shape[1]
        mean = pq["mean"].repeat_interleave(g, dim=1) if g > 1 else pq["mean"]
        lse = lse + float(sm_scale) * torch.einsum("bhnd,bhd->bhn", q.float(), mean)
    return out, lse


def sdpa_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False,
              sm_scale: Optional[float] = None, row_chunk: int = 4096, return_lse: bool = False):
    """Exact-attention comparator, the reference's own oracle (tests/test_sk1_backend.py:51-52),
    evaluated in query-row chunks so that no N x N matrix beyond `row_chunk` rows exists."""
    b, h, n, d = q.shape
    scale = d ** -0.5 if sm_scale is None else sm_scale
    qf, kf, vf = q.float(), k.float(), v.float()
    if kf.shape[1] != h:
        kf, vf = kf.repeat_interleave(h // kf.shape[1], dim=1), vf.repeat_interleave(h // vf.shape[1], dim=1)
    out = torch.empty(b, h, n, d, dtype=torch.float32, device=q.device)
    lse = torch.empty(b, h, n, dtype=torch.float32, device=q.device)
    keys = torch.arange(kf.shape[2], device=q.device)
    for r0 in range(0, n, row_chunk):
        r1 = min(n, r0 + row_chunk)
        s = torch.matmul(qf[:, :, r0:r1], kf.transpose(2, 3)) * scale
        if is_causal:
            rows = torch.arange(r0, r1, device=q.device)
            s = s.masked_fill(keys[None, :] > rows[:, None], float("-inf"))
        out[:, :, r0:r1] = torch.matmul(torch.softmax(s, dim=-1), vf)
        lse[:, :, r0:r1] = torch.logsumexp(s, dim=-1)
    return (out, lse) if return_lse else out


# ---- error metrics used by the tests and the reports -------------------------------------------
def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-300))


def rel_l1(a: torch.Tensor, ref: torch.Tensor) -> float:
    a, ref = a.double(), ref.double()
    return float((a - ref).abs().sum() / ref.abs().sum().clamp_min(1e-300))


def rel_rms(a: torch.Tensor, ref: torch.Tensor) -> float:
    """The reference's metric (tests/test_sk1_backend.py:46-48)."""
    a, ref = a.double(), ref.double()
    return float(((a - ref).pow(2).mean().sqrt()) / ref.pow(2).mean().sqrt().clamp_min(1e-300))


# ---- synthetic inputs of the benchmark configurations ------------------------------------------
def make_inputs(b: int, h: int, n: int, d: int = 128, dtype=torch.float16, seed: int = 0,
                k_bias_std: float = 0.0, head_scale: bool = False, outlier_frac: float = 0.0,
                outlier_mult: float = 50.0, device="cpu"):
    """Seeded Q, K, V ~ N(0,1) in fp32 then cast, with the options the benchmark configurations
    name: a per-(head, channel) K bias shared across tokens, per-head Q/K multipliers from
    U(0.5, 2), and a seeded fraction of K tokens (one index set shared by all heads) scaled up."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, h, n, d, generator=g)
    k = torch.randn(b, h, n, d, generator=g)
    v = torch.randn(b, h, n, d, generator=g)
    if k_bias_std > 0:
        k = k + k_bias_std * torch.randn(1, h, 1, d, generator=g)
    if head_scale:
        q = q * (0.5 + 1.5 * torch.rand(1, h, 1, 1, generator=g))
        k = k * (0.5 + 1.5 * torch.rand(1, h, 1, 1, generator=g))
    if outlier_frac > 0:
        cnt = int(round(outlier_frac * n))
        idx = torch.randperm(n, generator=g)[:cnt]
        k[:, :, idx] = k[:, :, idx] * outlier_mult
    return q.to(dtype).to(device), k.to(dtype).to(device), v.to(dtype).to(device)


def attention_flops(b: int, h: int, n: int, d: int, causal: bool) -> float:
    """4*B*H*N^2*D, halved when causal (bench/bench_attention.py:140)."""
    return 4.0 * b * h * n * n * d * (0.5 if causal else 1.0)


__all__ = [name for name in dir() if not name.startswith("_")]
