"""Public entry points of the drop-in `sageattention` package for B200.

Same names, arguments and error behaviour as the reference's dispatcher for the path this package
serves (sageattention/core.py:1037-1252 `sageattn`, :1747-1760 `sageattn_qk_int8_pv_fp8_cuda`):
fp16 / bf16 inputs, head_dim 128, HND or NHD layout, `is_causal`, `sm_scale`, `smooth_k`.
Anything else raises -- there is no second backend to fall back to.
"""
from __future__ import annotations

from typing import Any, Optional

import torch

from . import b200_backend as _be


def _reject_common(return_lse: bool, kwargs: dict):
    # `sageattn` does not advertise an attn_mask parameter (callers probe for it); a mask that
    # arrives anyway must not be silently ignored (reference: sageattention/core.py:1156-1161).
    if kwargs.get("attn_mask", None) is not None:
        raise NotImplementedError(
            "sageattention (B200 path) does not implement attn_mask; refusing to ignore it. "
            "Pass mask=None or use a backend that supports masking.")
    if kwargs.get("smooth_v", False):
        raise NotImplementedError("sageattention (B200 path) does not implement smooth_v")


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

    q : ``[B, Hq, Nq, 128]`` (``tensor_layout="HND"``) or ``[B, Nq, Hq, 128]`` (``"NHD"``);
    k, v : the same with ``Hkv`` heads and ``Nk`` rows; ``Hq`` a multiple of ``Hkv`` (grouped-query
        attention), ``Nk`` may differ from ``Nq`` when the call is not causal.  float16 or
        bfloat16, one CUDA device; strided views are accepted when the last axis is contiguous and
        every other stride is a multiple of 8 elements.
    return_lse : also return the fp32 log-sum-exp ``[B, Hq, Nq]`` of ``sm_scale * q.k``.
    is_causal : causal mask (query i sees keys <= i).
    sm_scale : softmax scale, default ``128 ** -0.5``.
    smooth_k (kwarg, default True) : subtract the per-channel sequence mean of K before
        quantising it.
    sk1_int8 : ``False`` selects e4m3 Q.K codes for float16 inputs; ``None``/``True`` keep the
        default (int8 for float16).  bfloat16 inputs always use e4m3 codes.
    sk1_backend, sk1_bf16 : accepted for call compatibility; ``False`` asks for a path this
        package does not have and raises.
    Returns a tensor with q's shape, dtype and layout (and the LSE when asked for).
    """
    _reject_common(return_lse, kwargs)
    if sk1_backend is False or sk1_bf16 is False and q.dtype == torch.bfloat16:
        raise NotImplementedError("sageattention (B200 path) has no alternative backend to switch to")
    int8 = None
    if q.dtype == torch.float16 and sk1_int8 is not None:
        int8 = bool(sk1_int8)
    return _be.sage_call(q, k, v, tensor_layout=tensor_layout, is_causal=bool(is_causal),
                         sm_scale=sm_scale, smooth_k=bool(kwargs.get("smooth_k", True)), int8=int8,
                         return_lse=bool(return_lse))


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
    fp32, so every accepted `pv_accum_dtype` value yields the fp32 behaviour."""
    if qk_quant_gran not in ("per_warp", "per_thread"):
        raise ValueError("qk_quant_gran must be 'per_warp' or 'per_thread'")
    if pv_accum_dtype not in ("fp32", "fp32+fp32", "fp32+fp16"):
        raise ValueError("pv_accum_dtype must be 'fp32', 'fp32+fp32' or 'fp32+fp16'")
    kwargs = dict(kwargs, smooth_v=smooth_v)
    _reject_common(return_lse, kwargs)
    return _be.sage_call(q, k, v, tensor_layout=tensor_layout, is_causal=bool(is_causal),
                         sm_scale=sm_scale, smooth_k=bool(smooth_k), int8=None, return_lse=bool(return_lse))


# upstream aliases kept so that existing call sites import unchanged
sageattn_qk_int8_pv_fp8_cuda = sageattn_qk_int8_pv_fp8
sageattn_qk_int8_pv_fp8_cuda_sm90 = sageattn_qk_int8_pv_fp8
