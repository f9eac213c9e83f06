"""Public entry points of the drop-in `sageattention` package for B200.

Same names, arguments and error behaviour as the reference's dispatcher for the path this package
serves (sageattention/core.py:1037-1252 `sageattn`, :1747-1760 `sageattn_qk_int8_pv_fp8_cuda`):
fp16 / bf16 inputs, head_dim up to 128, HND or NHD layout, `is_causal`, `sm_scale`, `smooth_k`,
`smooth_v`, `return_lse`, grouped-query heads; plus `sageattn_varlen` (:1444-1558).
Anything else raises -- there is no second backend to fall back to.
"""
from __future__ import annotations

import os
import warnings
from typing import Any, Optional

import torch

from . import b200_backend as _be


def _env_switch(name: str) -> Optional[bool]:
    """`1/true/yes/on` -> True, `0/false/no/off` -> False, anything else -> None; the reference's
    reading of its `SAGEATTN_SK1_*` switches (sageattention/sk1_backend/__init__.py:284-297)."""
    val = os.environ.get(name, "").strip().lower()
    if val in ("1", "true", "yes", "on"):
        return True
    if val in ("0", "false", "no", "off"):
        return False
    return None


# The reference's environment switches that still mean something here, read once at import like
# there (sageattention/sk1_backend/__init__.py:48-57):
#   SAGEATTN_SK1_INT8=0     float16 calls use e4m3 Q.K codes unless `sk1_int8` says otherwise
#   SAGEATTN_SK1_BACKEND=0  asks for the other backends, which this package does not have: calls raise
# (SAGEATTN_SK1_BF16, _PROLOGUE and _GFX1200 select AMD-side objects and have no meaning here.)
SK1_INT8 = _env_switch("SAGEATTN_SK1_INT8") is not False
SK1_BACKEND = _env_switch("SAGEATTN_SK1_BACKEND") is not False


def _reject_common(return_lse: bool, kwargs: dict):
    # `sageattn` does not advertise an attn_mask parameter (callers probe for it); a mask that
    # arrives anyway must not be silently ignored (reference: sageattention/core.py:1156-1161).
    if kwargs.get("attn_mask", None) is not None:
        raise NotImplementedError(
            "sageattention (B200 path) does not implement attn_mask; refusing to ignore it. "
            "Pass mask=None or use a backend that supports masking.")


def sageattn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    tensor_layout: str = "HND",
    is_causal: bool = False,
    sm_scale: Optional[float] = None,
    return_lse: bool = False,
    sk1_backend: Optional[bool] = None,
    sk1_int8: Optional[bool] = None,
    sk1_bf16: Optional[bool] = None,
    **kwargs: Any,
) -> torch.Tensor:
    """Quantised attention: per-token int8 Q.K (e4m3 for bf16 inputs), e4m3 P.V, fp32 softmax.

    q : ``[B, Hq, Nq, D]`` (``tensor_layout="HND"``) or ``[B, Nq, Hq, D]`` (``"NHD"``), ``D`` a
        multiple of 8 up to 128;
    k, v : the same with ``Hkv`` heads and ``Nk`` rows; ``Hq`` a multiple of ``Hkv`` (grouped-query
        attention), ``Nk`` may differ from ``Nq`` when the call is not causal.  float16 or
        bfloat16, one CUDA device; strided views are accepted when the last axis is contiguous and
        every other stride is a multiple of 8 elements.
    return_lse : also return the fp32 log-sum-exp ``[B, Hq, Nq]`` of ``sm_scale * q.k``.
    is_causal : causal mask (query i sees keys <= i).
    sm_scale : softmax scale, default ``D ** -0.5``.
    smooth_k (kwarg, default True) : subtract the per-channel sequence mean of K before
        quantising it.
    smooth_v (kwarg, default False) : quantise V minus its per-channel sequence mean and add the
        mean back to the output.
    sk1_int8 : ``False`` selects e4m3 Q.K codes for float16 inputs; ``None``/``True`` keep the
        default (int8 for float16).  bfloat16 inputs always use e4m3 codes.
    sk1_backend, sk1_bf16 : accepted for call compatibility; ``False`` asks for a path this
        package does not have and raises.
    Returns a tensor with q's shape, dtype and layout (and the LSE when asked for).
    """
    _reject_common(return_lse, kwargs)
    if sk1_backend is False or (sk1_backend is None and not SK1_BACKEND) \
            or sk1_bf16 is False and q.dtype == torch.bfloat16:
        raise NotImplementedError("sageattention (B200 path) has no alternative backend to switch to")
    int8 = None
    if q.dtype == torch.float16:
        if sk1_int8 is not None:
            int8 = bool(sk1_int8)
        elif not SK1_INT8:
            int8 = False
    return _be.sage_call(q, k, v, tensor_layout=tensor_layout, is_causal=bool(is_causal),
                         sm_scale=sm_scale, smooth_k=bool(kwargs.get("smooth_k", True)), int8=int8,
                         return_lse=bool(return_lse), smooth_v=bool(kwargs.get("smooth_v", False)))


def sageattn_qk_int8_pv_fp8(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    tensor_layout: str = "HND",
    is_causal: bool = False,
    qk_quant_gran: str = "per_thread",
    sm_scale: Optional[float] = None,
    pv_accum_dtype: str = "fp32+fp16",
    smooth_k: bool = True,
    smooth_v: bool = False,
    return_lse: bool = False,
    **kwargs: Any,
) -> torch.Tensor:
    """The upstream-named entry point (sageattention/core.py:1747-1760 of the reference).  Served
    by the same kernels as `sageattn`: Q and K always get one scale per token (finer than the
    `per_warp` / `per_thread` granularities the argument names), and P.V always accumulates in
    fp32, so every accepted `pv_accum_dtype` value yields the fp32 behaviour.  As upstream
    (:1910-1916), `smooth_v` only takes effect with ``pv_accum_dtype="fp32"`` and is ignored, with
    a warning, for the two-level accumulators."""
    if qk_quant_gran not in ("per_warp", "per_thread"):
        raise ValueError("qk_quant_gran must be 'per_warp' or 'per_thread'")
    if pv_accum_dtype not in ("fp32", "fp32+fp32", "fp32+fp16"):
        raise ValueError("pv_accum_dtype must be 'fp32', 'fp32+fp32' or 'fp32+fp16'")
    _reject_common(return_lse, kwargs)
    if smooth_v and pv_accum_dtype != "fp32":
        warnings.warn("pv_accum_dtype is '%s', smooth_v will be ignored." % pv_accum_dtype)
        smooth_v = False
    return _be.sage_call(q, k, v, tensor_layout=tensor_layout, is_causal=bool(is_causal),
                         sm_scale=sm_scale, smooth_k=bool(smooth_k), int8=None, return_lse=bool(return_lse),
                         smooth_v=bool(smooth_v))


def sageattn_varlen(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    is_causal: bool = False,
    sm_scale: Optional[float] = None,
    smooth_k: bool = True,
    **kwargs: Any,
) -> torch.Tensor:
    """Packed variable-length batch (sageattention/core.py:1444-1558 of the reference).

    q : ``[cu_seqlens_q[-1], Hq, D]``; k, v : ``[cu_seqlens_k[-1], Hkv, D]``; ``cu_seqlens_*`` are
    int32 / int64 prefix sums of the sequence lengths (``[batch + 1]``).  Returns
    ``[cu_seqlens_q[-1], Hq, D]``.

    The batch goes out as ONE call of the kernels, which read the cumulative lengths on the device:
    with `cu_seqlens_*` on the GPU nothing is read back and the call does not synchronise (the
    lengths are then the caller's promise; `max_seqlen_q` / `max_seqlen_k` bound them and size the
    workspace, a longer sequence is cut off at the bound).  Lengths given on the host are checked
    first, and a batch of equal lengths takes the fixed-length kernels on a strided view.  Only a
    batch so ragged that slots of the longest length would take more than `_VARLEN_SLOT_FACTOR`
    times the packed size (and more than `_VARLEN_SLOT_FREE_BYTES`) is split into runs of equal
    lengths, one call each; that path needs the lengths on the host and copies them if necessary.
    `smooth_k` subtracts each sequence's own K mean (the reference subtracts the mean over the
    whole packed batch; softmax is invariant to either shift, only rounding differs).
    """
    _reject_common(False, kwargs)
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("sageattn_varlen takes packed [tokens, heads, head_dim] tensors")
    if cu_seqlens_q.dim() != 1 or cu_seqlens_k.dim() != 1 or cu_seqlens_q.numel() != cu_seqlens_k.numel() \
            or cu_seqlens_q.numel() < 2:
        raise ValueError("cu_seqlens_q and cu_seqlens_k must be 1-D with batch + 1 entries each")
    if cu_seqlens_q.dtype not in (torch.int32, torch.int64) or cu_seqlens_k.dtype not in (torch.int32, torch.int64):
        raise ValueError("cu_seqlens_q and cu_seqlens_k must be int32 or int64")
    if k.size(0) != v.size(0):
        raise ValueError("cu_seqlens do not match the packed tensors")
    n_seq = cu_seqlens_q.numel() - 1
    max_q, max_k = int(max_seqlen_q), int(max_seqlen_k)
    if q.size(0) == 0:
        return torch.empty_like(q)
    on_device = cu_seqlens_q.is_cuda and cu_seqlens_k.is_cuda
    one_call = _varlen_slots_fit(n_seq, q.size(1), k.size(1), q.size(0), k.size(0), max_q, max_k)
    if on_device and one_call:
        if max_q < 1 or max_k < 1:
            raise ValueError("max_seqlen_q and max_seqlen_k must be positive")
        return _be.sage_call_varlen(q, k, v, cu_seqlens_q.to(torch.int32), cu_seqlens_k.to(torch.int32),
                                    min(max_q, q.size(0)), min(max_k, k.size(0)), is_causal=bool(is_causal),
                                    sm_scale=sm_scale, smooth_k=bool(smooth_k))
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    ck = [int(x) for x in cu_seqlens_k.tolist()]
    if cq[0] != 0 or ck[0] != 0 or cq[-1] != q.size(0) or ck[-1] != k.size(0):
        raise ValueError("cu_seqlens do not match the packed tensors")
    for i in range(n_seq):                            # every sequence is checked before anything is launched
        nq, nk = cq[i + 1] - cq[i], ck[i + 1] - ck[i]
        if nq < 0 or nk < 0 or nq > max_q or nk > max_k:
            raise ValueError("sequence %d has lengths (%d, %d) outside 0..max_seqlen" % (i, nq, nk))
        if nq > 0 and nk == 0:
            raise ValueError("sequence %d has queries but no keys" % i)
        if is_causal and nq != nk:
            raise ValueError("sequence %d: a causal call needs q_len == kv_len" % i)
    out = torch.empty_like(q)
    uniform = all(cq[i + 1] - cq[i] == cq[1] and ck[i + 1] - ck[i] == ck[1] for i in range(n_seq))
    if one_call and not uniform:
        dev = q.device
        return _be.sage_call_varlen(q, k, v, torch.tensor(cq, dtype=torch.int32).to(dev, non_blocking=True),
                                    torch.tensor(ck, dtype=torch.int32).to(dev, non_blocking=True),
                                    max(cq[i + 1] - cq[i] for i in range(n_seq)),
                                    max(ck[i + 1] - ck[i] for i in range(n_seq)), is_causal=bool(is_causal),
                                    sm_scale=sm_scale, smooth_k=bool(smooth_k), out=out)
    i = 0
    while i < n_seq:
        nq, nk = cq[i + 1] - cq[i], ck[i + 1] - ck[i]
        j = i + 1                      # consecutive sequences of the same lengths go out as one batched call
        while j < n_seq and cq[j + 1] - cq[j] == nq and ck[j + 1] - ck[j] == nk:
            j += 1
        if nq > 0:
            run = j - i
            _be.sage_call(q[cq[i]:cq[j]].unflatten(0, (run, nq)), k[ck[i]:ck[j]].unflatten(0, (run, nk)),
                          v[ck[i]:ck[j]].unflatten(0, (run, nk)), tensor_layout="NHD", is_causal=bool(is_causal),
                          sm_scale=sm_scale, smooth_k=bool(smooth_k), out=out[cq[i]:cq[j]].unflatten(0, (run, nq)))
        i = j
    return out


#: A packed batch goes out as one call when slots of the longest length for every sequence take at
#: most this many times the packed token count, or less than the byte figure below in any case.
_VARLEN_SLOT_FACTOR = 4
_VARLEN_SLOT_FREE_BYTES = 1 << 30


def _varlen_slots_fit(n_seq: int, hq: int, hkv: int, total_q: int, total_k: int, max_q: int, max_k: int) -> bool:
    """Whether the one-call form's workspace (a slot of the longest length per sequence) is acceptable."""
    max_q, max_k = max(1, min(max_q, total_q)), max(1, min(max_k, total_k))
    slots = n_seq * (hq * max_q + 2 * hkv * max_k)
    packed = hq * total_q + 2 * hkv * total_k
    if n_seq * hq > 65535:                            # the grid's (batch, head) axis
        return False
    return slots <= _VARLEN_SLOT_FACTOR * packed or slots * 132 <= _VARLEN_SLOT_FREE_BYTES


# upstream aliases kept so that existing call sites import unchanged
sageattn_qk_int8_pv_fp8_cuda = sageattn_qk_int8_pv_fp8
sageattn_qk_int8_pv_fp8_cuda_sm90 = sageattn_qk_int8_pv_fp8
