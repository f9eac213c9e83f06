"""`sageattention` for NVIDIA B200 (sm_100a): a drop-in for the quantize-then-attend path of
SageAttention-RDNA4.

    from sageattention import sageattn
    out = sageattn(q, k, v, tensor_layout="HND", is_causal=False)

`sageattn` deliberately has no `attn_mask` parameter, like the reference
(sageattention/__init__.py:4-8 there): callers that probe for one route masked calls elsewhere.
The CUDA kernels live in libsage_b200.so next to this file and are reached through ctypes; without
that library every call raises (no CPU or PyTorch fallback exists).
"""
from .core import (  # noqa: F401
    sageattn,
    sageattn_qk_int8_pv_fp8,
    sageattn_qk_int8_pv_fp8_cuda,
    sageattn_qk_int8_pv_fp8_cuda_sm90,
    sageattn_varlen,
)
from .b200_backend import status  # noqa: F401
from .sharding import partition_units, sageattn_sharded, gather_units  # noqa: F401

__version__ = "0.1.0+b200"

__all__ = [
    "sageattn",
    "sageattn_qk_int8_pv_fp8",
    "sageattn_qk_int8_pv_fp8_cuda",
    "sageattn_qk_int8_pv_fp8_cuda_sm90",
    "sageattn_varlen",
    "partition_units",
    "sageattn_sharded",
    "gather_units",
    "status",
    "__version__",
]
