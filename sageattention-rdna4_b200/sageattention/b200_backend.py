"""Host side of the B200 quantize-then-attend path: acceptance rules, buffer ownership, launches.

Mirrors, for this one path, the reference's router `try_sk1_t1`
(sageattention/sk1_backend/__init__.py:982-1284), its acceptance rule `strided_view_reason`
(sageattention/sk1_backend/sk1_loader.py:313-369) and `_envelope_ok`
(sageattention/sk1_backend/__init__.py:920-979), its prologue wrapper `HipPrologue.quant_kv`
(sageattention/sk1_backend/hip_prologue.py:188-244) and its launcher `Sk1Attn.launch`
(sageattention/sk1_backend/sk1_loader.py:628-688).  Differences that are deliberate: a request
outside the envelope raises (there is no fallback path), Q is quantised in the prologue and its
codes are materialised, keys are padded to 128, and the fold S is computed inside the prologue.
"""
from __future__ import annotations

import ctypes
import os
import threading
from collections import OrderedDict
from typing import Dict, Optional, Tuple

import torch

from . import _native

HEAD_DIM = 128
TILE = 128
_STRIDE_MAX = 2 ** 39 - 1          # elements: a tensor map takes byte strides below 2**40

#: Every reason `strided_view_reason` can return, in evaluation order (the reference's strings, but
#: "stride_range" where the reference has "stride_int32": its kernels index with 32-bit strides,
#: these take 64-bit ones, so that a batch of long sequences does not have to be split).
STRIDED_REFUSALS = ("rank", "stride_last", "stride_nonpos", "stride_align", "ptr_align",
                    "stride_overlap", "stride_range")

_counters = {"calls": 0, "refusals": 0}


def pad_len(n: int) -> int:
    return (int(n) + TILE - 1) // TILE * TILE


def strided_view_reason(t: torch.Tensor) -> Optional[str]:
    """None if `t` is a servable logical (B,H,N,D) view, else the reason.  Same rule and order as
    the reference: rank 4; last stride 1; strides positive; outer strides multiples of 8 elements;
    16-byte aligned pointer; injective index map (dims of size > 1 sorted by stride must satisfy
    stride[k+1] >= stride[k]*size[k]); strides below 2**39 elements (the reference: 2**31)."""
    if t.dim() != 4:
        return "rank"
    strides = tuple(int(x) for x in t.stride())
    extents = tuple(int(x) for x in t.shape)
    if strides[3] != 1:
        return "stride_last"
    if min(strides) <= 0:
        return "stride_nonpos"
    if any(x % 8 for x in strides[:3]):
        return "stride_align"
    if t.data_ptr() % 16:
        return "ptr_align"
    # Walk the axes that have more than one element from the smallest stride up: each must step
    # over everything the axes below it can reach, or two index tuples share an address.
    reach = 0
    for stride, extent in sorted(zip(strides, extents)):
        if extent <= 1:
            continue
        if stride < reach:
            return "stride_overlap"
        reach = stride * extent
    if max(strides) > _STRIDE_MAX:
        return "stride_range"
    return None


def envelope_reason(q, k, v, tensor_layout, return_lse=False, attn_mask=None,
                    require_cuda=True) -> Optional[str]:
    """None if the call is inside the envelope, else a short reason (the reference's strings:
    layout, attn_mask, device, dtype, rank, stride_*, ptr_align, head_dim, batch, heads,
    seq_len).  Wider than the reference's hand-written path in four places, following the upstream
    contract (sageattention/core.py:1081-1101, :1524-1533): `return_lse` is served, the query heads
    may be a multiple of the key/value heads, the key length may differ from the query length, and
    head_dim may be any multiple of 8 up to 128 (the quantised codes are zero-filled to 128
    columns, which is what upstream's host-side padding amounts to)."""
    if tensor_layout not in ("HND", "NHD"):
        return "layout"
    if attn_mask is not None:
        return "attn_mask"
    if require_cuda and not (q.is_cuda and k.is_cuda and v.is_cuda):
        return "device"
    if q.device != k.device or q.device != v.device:
        return "device"
    if not (q.dtype == k.dtype == v.dtype):
        return "dtype"
    if q.dtype not in (torch.float16, torch.bfloat16):
        return "dtype"
    if not (q.dim() == 4 and k.dim() == 4 and v.dim() == 4):
        return "rank"
    if tensor_layout == "NHD":
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    for t in (q, k, v):
        r = strided_view_reason(t)
        if r is not None:
            return r
    if q.size(3) < 8 or q.size(3) > HEAD_DIM or q.size(3) % 8 or k.size(3) != q.size(3) or v.size(3) != q.size(3):
        return "head_dim"
    if q.size(0) != k.size(0) or q.size(0) != v.size(0):
        return "batch"
    if k.size(1) != v.size(1) or k.size(1) < 1 or q.size(1) % k.size(1):
        return "heads"
    if k.size(2) != v.size(2):
        return "seq_len"
    if q.size(2) < 1 or k.size(2) < 1:
        return "seq_len"
    return None


def _dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return _native.SAGE_F16
    if dt == torch.bfloat16:
        return _native.SAGE_BF16
    raise ValueError("dtype must be float16 or bfloat16, got %s" % dt)


def _bhr(t: torch.Tensor):
    """(batch, head, row) element strides of a logical (B,H,N,D) view."""
    return _native.strides3(t.stride(0), t.stride(1), t.stride(2))


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(int(torch.cuda.current_stream(device).cuda_stream))


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else int(t.data_ptr()))


def _require_cuda(*ts):
    for t in ts:
        if not t.is_cuda:
            raise ValueError("the B200 path serves CUDA tensors only (got a %s tensor); there is no CPU path"
                             % t.device.type)


def k8_row_order(n_pad: int, device="cpu") -> torch.Tensor:
    """Where the prologue stores the K codes of each key: `k8[:, k8_row_order(n_pad)]` is K8 in
    key order.  Inside every block of 16 keys, key 4c + j sits in row 2c + j (j < 2) or
    8 + 2c + j - 2 (j >= 2): the order in which the attention kernel's 16-lane TMEM loads hand a
    thread four consecutive keys of a score row.  Scales (sk, sv, svp) are in key order."""
    key = torch.arange(int(n_pad), device=device)
    o = key & 15
    c, j = o >> 2, o & 3
    return (key & ~15) | torch.where(j < 2, 2 * c + j, 8 + 2 * c + j - 2)


def quant_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, smooth_k: bool = True,
              int8: Optional[bool] = None, reuse: Optional[dict] = None) -> Dict[str, torch.Tensor]:
    """Run the prologue on logical (B,H,N,D) views and return every tensor it writes:
    q8 (BH,N,D), sq (BH,N), k8 (BH,N_pad,D; rows in `k8_row_order`), sk (BH,N_pad), v8t (BH,D,N_pad), sv, svp (BH,N_pad),
    S (BH,), mean (BH,D) or None.  `int8=None` follows the reference's default: int8 codes for
    fp16 inputs, e4m3 for bf16.  Code tensors are torch.int8 or torch.float8_e4m3fn.  `reuse` is a
    previous result for the same shapes whose buffers are written again instead of allocating."""
    _require_cuda(q, k, v)
    lib = _native.load()
    b, h, n, d = q.shape
    if d != HEAD_DIM:
        raise ValueError("the two-step entry points take head_dim 128; use sage_call for smaller heads")
    if int8 is None:
        int8 = q.dtype == torch.float16
    n_pad, bh, dev = pad_len(n), b * h, q.device
    code_dt = torch.int8 if int8 else torch.float8_e4m3fn
    u8 = dict(dtype=torch.uint8, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    if reuse is not None and (reuse["B"], reuse["H"], reuse["n"], reuse["int8"]) == (b, h, n, bool(int8)) \
            and (reuse["mean"] is not None) == bool(smooth_k):
        out = dict(reuse)
        for key in ("q8", "k8", "v8t"):
            out[key] = out[key].view(torch.uint8)
    else:
        out = dict(
            q8=torch.empty((bh, n, d), **u8), sq=torch.empty((bh, n), **f32),
            k8=torch.empty((bh, n_pad, d), **u8), sk=torch.empty((bh, n_pad), **f32),
            v8t=torch.empty((bh, d, n_pad), **u8), sv=torch.empty((bh, n_pad), **f32),
            svp=torch.empty((bh, n_pad), **f32), S=torch.empty((bh,), **f32),
            mean=torch.empty((bh, d), **f32) if smooth_k else None,
            ctrl=torch.empty((lib.sage_prologue_ctrl_bytes(b, h, n),), **u8))
    with torch.cuda.device(dev):
        rc = lib.sage_prologue(
            _ptr(q), _ptr(k), _ptr(v), _ptr(out["q8"]), _ptr(out["sq"]), _ptr(out["k8"]),
            _ptr(out["sk"]), _ptr(out["v8t"]), _ptr(out["sv"]), _ptr(out["svp"]), _ptr(out["S"]),
            _ptr(out["mean"]), _ptr(out["ctrl"]), b, h, n, n_pad, _bhr(q), _bhr(k), _bhr(v),
            _dtype_code(q.dtype), _native.SAGE_QK_INT8 if int8 else _native.SAGE_QK_E4M3,
            1 if smooth_k else 0, _stream(dev))
    _native.check(rc, "sage_prologue")
    out["q8"] = out["q8"].view(code_dt)
    out["k8"] = out["k8"].view(code_dt)
    out["v8t"] = out["v8t"].view(torch.float8_e4m3fn)
    out.update(n=n, n_pad=n_pad, int8=bool(int8), B=b, H=h)
    return out


def attn_launch(pq: Dict[str, torch.Tensor], out: torch.Tensor, is_causal: bool, sm_scale: float,
                status: Optional[torch.Tensor] = None, plain: bool = False) -> torch.Tensor:
    """Launch the attention kernel on a prologue result; `out` is a logical (B,H,N,D) view that
    is written in place.  Returns the int32 status tensor (zero unless a bounded wait gave up).
    `plain` selects the kernels without the negligible-tile tests."""
    lib = _native.load()
    dev = out.device
    b, h, n, n_pad = pq["B"], pq["H"], pq["n"], pq["n_pad"]
    if status is None:
        status = torch.zeros((1,), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.sage_attn_fwd(
            _ptr(pq["q8"]), _ptr(pq["sq"]), _ptr(pq["k8"]), _ptr(pq["sk"]), _ptr(pq["v8t"]),
            _ptr(pq["svp"]), _ptr(pq["S"]), _ptr(out), b, h, n, n_pad, _bhr(out),
            1 if is_causal else 0, float(sm_scale), _dtype_code(out.dtype),
            (_native.SAGE_QK_INT8 if pq["int8"] else _native.SAGE_QK_E4M3) |
            (_native.SAGE_QK_NO_FAST_PATH if plain else 0), _ptr(status), _stream(dev))
    _native.check(rc, "sage_attn_fwd")
    return status


# ---- the whole call ------------------------------------------------------------------------------
# Device-side failures.  Every wait inside the kernels is bounded; a wait that runs out leaves a
# code in the call's status word (a word of the workspace) and the output of that call is
# undefined.  The reference raises in such a case only in its strict mode and otherwise falls back
# (sageattention/sk1_backend/__init__.py:1022-1027,1114-1123); this path has no fallback, so the
# failure must reach the caller.  After every call a 4-byte copy of the status word into pinned
# host memory is enqueued behind it (no synchronisation); the next call on that stream, `check()`
# or `status()` looks at the host word and raises RuntimeError when it is non-zero.
# SAGEATTN_B200_STRICT=1 synchronises after every call and checks at once;
# SAGEATTN_B200_WATCH=0 switches the copy off.
STATUS_BITS = ((1, "the TMA producer of the attention kernel"), (2, "the MMA issuer of the attention kernel"),
               (4, "a softmax warp of the attention kernel"), (8, "a tile load of the quantisation prologue"))


def describe_status(code: int) -> str:
    who = [name for bit, name in STATUS_BITS if code & bit]
    return "status 0x%x: a bounded wait ran out in %s; the output of that call is undefined" % (
        code & 0xFFFFFFFF, " and ".join(who) if who else "an unknown role")


def _env_flag(name: str, default: bool) -> bool:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return v.strip().lower() not in ("0", "false", "off", "no")


# ---- which attention kernels a call takes ---------------------------------------------------------
# The attention kernel exists with and without its negligible-tile tests (include/sage_b200.h,
# SAGE_QK_NO_FAST_PATH).  With them, key tiles far below the running row maxima are not
# exponentiated, which on inputs with a few dominant keys removes most of the softmax work; on
# inputs without such keys the tests only cost (3 to 6 %).  The kernels count what they skip, so
# the choice is made from evidence: a call signature (shape, mask, dtype) starts with the tests
# on; one such call is a probe whose count comes back to the host with the status mirror (no
# synchronisation: the result is picked up by a later call once its event has completed); a probe
# that skipped less than PROBE_MIN_SHARE of the (warp, key tile) pairs sends the next PLAIN_CALLS
# calls of that signature to the kernels without the tests, after which the next call probes
# again.  Both sets of kernels give identical bits whenever no tile is skipped.  (Break-even,
# measured at H=16, N=16384: with 23 % of the pairs skipped the two sets take the same time.)
PROBE_MIN_SHARE = 0.2
PLAIN_CALLS = 255
PROBE_AGAIN_AFTER = 256       # calls with the tests on between two probes


class _Adaptive:
    """Per (device, stream): the decision per call signature and the one outstanding probe."""

    __slots__ = ("plain_left", "since_probe", "probe")

    def __init__(self):
        self.plain_left: Dict[Tuple, int] = {}     # signature -> calls left without the tests
        self.since_probe: Dict[Tuple, int] = {}    # signature -> calls with the tests on since its last probe
        self.probe = None                          # (signature, pairs, event, pinned tensor, ctypes words) or None

    def decide(self, key: Tuple) -> Tuple[bool, bool]:
        """(use the plain kernels, make this call a probe)."""
        left = self.plain_left.get(key, 0)
        if left > 0:
            self.plain_left[key] = left - 1
            return True, False
        n = self.since_probe.get(key)
        want_probe = n is None or n >= PROBE_AGAIN_AFTER
        if want_probe and self.probe is None:
            self.since_probe[key] = 0
            return False, True
        if n is not None:                       # (a signature that never got its probe keeps asking)
            self.since_probe[key] = n + 1
        return False, False

    def take_result(self, key: Tuple, skipped: int, pairs: int) -> float:
        share = float(skipped) / float(max(pairs, 1))
        if share < PROBE_MIN_SHARE:
            self.plain_left[key] = PLAIN_CALLS
            self.since_probe.pop(key, None)
        return share


class _StreamState:
    """What the path keeps per (device, stream): one grow-only workspace (intermediates of a call
    live only until its attention kernel has run, and calls on one stream are ordered) and the
    pinned host word that mirrors the status word of the most recent call."""

    __slots__ = ("ws", "host", "host_word", "status_off", "shape", "adaptive", "probe_host", "last_share")

    def __init__(self, host_word=None):
        self.adaptive = _Adaptive()
        self.probe_host = None              # pinned (4,) int32 the probe's words land in
        self.last_share = None              # share of skipped pairs in the most recent finished probe
        self.ws = None
        self.host = None                    # pinned tensor that owns the memory behind host_word
        self.host_word = host_word          # ctypes.c_int32 view of it (tests pass a plain c_int32)
        self.status_off = None
        self.shape = None

    def pending(self) -> int:
        return 0 if self.host_word is None else int(self.host_word.value)

    def raise_if_failed(self, where: str):
        code = self.pending()
        if code:
            self.host_word.value = 0
            raise RuntimeError("sageattn (B200 path), reported at %s: %s" % (where, describe_status(code)))


_STRICT = _env_flag("SAGEATTN_B200_STRICT", False)
_WATCH = _env_flag("SAGEATTN_B200_WATCH", True) or _STRICT
_ADAPTIVE = _env_flag("SAGEATTN_B200_ADAPTIVE", True)      # 0: every call keeps the negligible-tile tests

_ws_lock = threading.Lock()
_states: "OrderedDict[Tuple[int, int], _StreamState]" = OrderedDict()
_STATE_ENTRIES = 8
_WS_GRANULE = 1 << 20


def _state(dev, stream_id: int, create: bool = True) -> Optional[_StreamState]:
    key = (dev.index, int(stream_id))
    with _ws_lock:
        st = _states.get(key)
        if st is not None:
            _states.move_to_end(key)
            return st
        if not create:
            return None
        st = _states[key] = _StreamState()
        while len(_states) > _STATE_ENTRIES:
            _states.popitem(last=False)
    return st


def _workspace(dev, stream_id: int, b: int, h: int, n: int, hkv: Optional[int] = None,
               nk: Optional[int] = None) -> torch.Tensor:
    """The workspace of (device, stream), grown if this shape needs more than it holds."""
    hkv = h if hkv is None else hkv
    nk = n if nk is None else nk
    nbytes = _native.load().sage_workspace_bytes_ex(b, h, hkv, n, nk)
    return _grow(_state(dev, stream_id), dev, nbytes)


def _grow(st: _StreamState, dev, nbytes: int) -> torch.Tensor:
    if st.ws is None or st.ws.numel() < nbytes:
        st.ws = None                         # release first: the two need not be resident together
        st.ws = torch.empty(((nbytes + _WS_GRANULE - 1) // _WS_GRANULE * _WS_GRANULE,), dtype=torch.uint8, device=dev)
    return st.ws


def _host_word(st: _StreamState):
    if st.host_word is None:
        st.host = torch.zeros((1,), dtype=torch.int32).pin_memory()
        st.host_word = ctypes.c_int32.from_address(st.host.data_ptr())
    return st.host_word


def clear_workspaces():
    with _ws_lock:
        _states.clear()


def reset_adaptive():
    """Forget what earlier calls taught about which call signatures skip key tiles (every
    signature probes again).  For callers whose data changes character under an unchanged shape."""
    with _ws_lock:
        for st in _states.values():
            st.adaptive = _Adaptive()
            st.last_share = None


def check(device=None):
    """Wait for the current stream of `device` and raise RuntimeError if a call on it reported a
    device-side failure (see STATUS_BITS)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    stream = torch.cuda.current_stream(dev)
    st = _state(dev, stream.cuda_stream, create=False)
    if st is None:
        return
    stream.synchronize()
    st.raise_if_failed("check()")


# Calls repeat with the same shapes and strides (a diffusion transformer issues the same attention
# call thousands of times), and for sequences of a few hundred tokens the GPU work is shorter than
# a careless host path.  A call signature that has passed `envelope_reason` once is remembered with
# everything derived from it (logical dims, stride triples for the C call), so the hot path is a
# handful of attribute reads, one dictionary lookup and the C call.
_sig_cache: Dict[Tuple, Tuple] = {}
_SIG_CACHE_ENTRIES = 256


def _logical_strides(t: torch.Tensor, nhd: bool):
    st = t.stride()
    return (st[0], st[2], st[1]) if nhd else (st[0], st[1], st[2])


def _validated(q, k, v, tensor_layout):
    """(b, hq, hkv, nq, nk, d, nhd, stride triples of q, k, v and of a fresh output, dtype code,
    workspace bytes, offset of the status word in the workspace) for a call inside the envelope;
    raises the documented exception otherwise.  Pointer alignment is part of the signature."""
    key = (tensor_layout, q.shape, q.stride(), k.shape, k.stride(), v.shape, v.stride(), q.dtype, k.dtype,
           v.dtype, q.device, k.device, v.device,
           (q.data_ptr() | k.data_ptr() | v.data_ptr()) & 15)
    hit = _sig_cache.get(key)
    if hit is not None:
        return hit
    reason = envelope_reason(q, k, v, tensor_layout)
    if reason is not None:
        _counters["refusals"] += 1
        if reason == "device" and not (q.is_cuda and k.is_cuda and v.is_cuda):
            raise ValueError("sageattn (B200 path) needs CUDA tensors; there is no CPU path")
        if reason == "head_dim":
            raise NotImplementedError("sageattn (B200 path) serves head_dim 8..128 in multiples of 8")
        raise ValueError("sageattn (B200 path) cannot serve this call: %s" % reason)
    nhd = tensor_layout == "NHD"
    qs, ks = q.shape, k.shape
    if nhd:
        b, nq, hq, d = qs
        nk, hkv = ks[1], ks[2]
    else:
        b, hq, nq, d = qs
        hkv, nk = ks[1], ks[2]
    b, hq, hkv, nq, nk, d = int(b), int(hq), int(hkv), int(nq), int(nk), int(d)
    # (batch, head, row) strides of a freshly allocated output with q's shape
    o3 = _native.strides3(nq * hq * d, d, hq * d) if nhd else _native.strides3(hq * nq * d, nq * d, d)
    lib = _native.load()
    offs = (ctypes.c_size_t * 13)()
    if lib.sage_workspace_layout_ex(b, hq, hkv, nq, nk, offs) != 13:
        raise _native.SageNativeError("sage_workspace_layout_ex failed")
    val = (b, hq, hkv, nq, nk, d, nhd,
           _native.strides3(*_logical_strides(q, nhd)), _native.strides3(*_logical_strides(k, nhd)),
           _native.strides3(*_logical_strides(v, nhd)), o3, _dtype_code(q.dtype),
           int(lib.sage_workspace_bytes_ex(b, hq, hkv, nq, nk)), int(offs[10]))
    if len(_sig_cache) >= _SIG_CACHE_ENTRIES:
        _sig_cache.clear()
    _sig_cache[key] = val
    return val


def sage_call(q, k, v, tensor_layout="HND", is_causal=False, sm_scale=None, smooth_k=True,
              int8: Optional[bool] = None, out: Optional[torch.Tensor] = None, return_lse: bool = False,
              smooth_v: bool = False):
    """Prologue + attention through the single C entry point `sage_attention_ex`.  Returns a tensor
    with q's shape, dtype and layout -- and, with `return_lse`, also the fp32 log-sum-exp
    (B, Hq, Nq).  `smooth_v` quantises V minus its sequence mean and adds the mean back to the
    output.  Raises ValueError for a call outside the envelope."""
    _counters["calls"] += 1
    b, h, hkv, n, nk, d, nhd, q3, k3, v3, o3, dt, ws_bytes, status_off = _validated(q, k, v, tensor_layout)
    if is_causal and nk != n:
        raise ValueError("sageattn (B200 path): a causal call needs q_len == kv_len")
    scale = d ** -0.5 if sm_scale is None else float(sm_scale)
    if not (0.0 < scale < float("inf")):
        raise ValueError("sageattn (B200 path): sm_scale must be finite and positive, got %r" % (sm_scale,))
    lib = _native.load()
    dev = q.device
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=dev)
    else:
        ol = out.transpose(1, 2) if nhd else out
        if tuple(ol.shape) != (b, h, n, d) or out.dtype != q.dtype or strided_view_reason(ol) is not None:
            raise ValueError("out must have q's shape and dtype and be a servable view")
        o3 = _native.strides3(*_logical_strides(out, nhd))
    if out.data_ptr() & 15:
        raise ValueError("out must be 16-byte aligned")
    if int8 is None:
        qk_mode = -1
    else:
        qk_mode = _native.SAGE_QK_INT8 if int8 else _native.SAGE_QK_E4M3
    stream_id = torch.cuda.current_stream(dev).cuda_stream
    st = _state(dev, stream_id)
    if st.host_word is not None and st.host_word.value:
        st.raise_if_failed("the next call on the stream")        # an earlier call's failure, seen without a sync
    ws = st.ws
    if ws is None or ws.numel() < ws_bytes:
        ws = _grow(st, dev, ws_bytes)
    st.status_off, st.shape = status_off, (b, h, hkv, n, nk)
    lse = torch.empty((b, h, n), dtype=torch.float32, device=dev) if return_lse else None
    ws_ptr = ws.data_ptr()
    # with or without the negligible-tile tests (see _Adaptive)
    # (while the stream is being captured into a CUDA graph nothing here may allocate, record or
    # query an event: the call then takes the kernels the signature is on, without probing)
    capturing = torch.cuda.is_current_stream_capturing()
    ad = st.adaptive
    if not capturing and ad.probe is not None and ad.probe[2].query():
        pkey, pairs, _ev, words = ad.probe
        ad.probe = None
        st.last_share = ad.take_result(pkey, int(words[3]) & 0xFFFFFFFF, pairs)
    key = (b, h, hkv, n, nk, d, bool(is_causal), dt, qk_mode)
    if capturing:
        plain, probe = ad.plain_left.get(key, 0) > 0, False
    else:
        plain, probe = ad.decide(key) if _ADAPTIVE else (False, False)
    if plain:
        qk_mode = -_native.SAGE_QK_NO_FAST_PATH if qk_mode < 0 else (qk_mode | _native.SAGE_QK_NO_FAST_PATH)
    args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 0 if lse is None else lse.data_ptr(),
            ws_ptr, ws.numel(), b, h, hkv, n, nk, d, q3, k3, v3, o3, dt, qk_mode,
            1 if is_causal else 0, 1 if smooth_k else 0, 1 if smooth_v else 0, scale, stream_id)
    watch = _WATCH and not (capturing and st.host_word is None)
    same_dev = torch.cuda.current_device() == dev.index
    if not same_dev:
        prev_dev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        rc = lib.sage_attention_ex(*args)
        if watch and not rc:
            rc = lib.sage_status_mirror(ws_ptr + status_off, ctypes.addressof(_host_word(st)), 1, stream_id)
        if probe and not rc:
            if st.probe_host is None:
                st.probe_host = torch.zeros((4,), dtype=torch.int32).pin_memory()
            words = (ctypes.c_int32 * 4).from_address(st.probe_host.data_ptr())
            rc = lib.sage_status_mirror(ws_ptr + status_off, ctypes.addressof(words), 4, stream_id)
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(dev))
            q_tiles, k_tiles = (n + TILE - 1) // TILE, (nk + TILE - 1) // TILE
            pairs = 8 * b * h * q_tiles * k_tiles // (2 if is_causal else 1)
            ad.probe = (key, pairs, ev, words)
    finally:
        if not same_dev:
            torch.cuda.set_device(prev_dev)
    if rc:
        _native.check(rc, "sage_attention_ex")
    if _STRICT:
        torch.cuda.current_stream(dev).synchronize()
        st.raise_if_failed("this call (strict mode)")
    if return_lse:
        return out, lse
    return out


def packed_view_reason(t: torch.Tensor) -> Optional[str]:
    """Why a packed (tokens, heads, head_dim) tensor cannot be served as it is, or None: the rule of
    `strided_view_reason` for the two strides a packed tensor has."""
    if t.dim() != 3:
        return "rank"
    if t.stride(2) != 1:
        return "last_stride"
    if t.data_ptr() & 15:
        return "alignment"
    for s in (t.stride(0), t.stride(1)):
        if s <= 0 or s % 8 or s > _STRIDE_MAX:
            return "stride_range"
    return None


def varlen_workspace_bytes(n_seq: int, hq: int, hkv: int, max_q: int, max_k: int) -> int:
    """Bytes of workspace `sage_call_varlen` takes: every sequence gets a slot sized for the longest."""
    return int(_native.load().sage_workspace_bytes_ex(n_seq, hq, hkv, max_q, max_k))


def sage_call_varlen(q, k, v, cu_q, cu_k, max_q: int, max_k: int, is_causal=False, sm_scale=None,
                     smooth_k=True, out: Optional[torch.Tensor] = None):
    """A packed variable-length batch through the single C entry point `sage_attention_varlen`.

    q (total_q, Hq, D), k and v (total_k, Hkv, D); `cu_q` / `cu_k` int32 DEVICE tensors of
    batch + 1 cumulative lengths, never read on the host: the call does not synchronise.
    `max_q` / `max_k` bound the sequence lengths and size the workspace.  Returns (total_q, Hq, D).
    """
    _counters["calls"] += 1
    for name, t in (("q", q), ("k", k), ("v", v)):
        reason = packed_view_reason(t)
        if reason is not None:
            _counters["refusals"] += 1
            raise ValueError("sageattn_varlen (B200 path) cannot serve %s: %s" % (name, reason))
    if not (q.is_cuda and k.is_cuda and v.is_cuda and cu_q.is_cuda and cu_k.is_cuda):
        raise ValueError("sageattn_varlen (B200 path) needs CUDA tensors; there is no CPU path")
    if not (q.device == k.device == v.device == cu_q.device == cu_k.device):
        raise ValueError("sageattn_varlen (B200 path): tensors on different devices")
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("sageattn_varlen (B200 path): q, k, v must share one dtype, fp16 or bf16")
    if cu_q.dtype != torch.int32 or cu_k.dtype != torch.int32 or not cu_q.is_contiguous() or not cu_k.is_contiguous():
        raise ValueError("sageattn_varlen (B200 path): cumulative lengths must be contiguous int32")
    tq, hq, d = (int(x) for x in q.shape)
    tk, hkv, dk = (int(x) for x in k.shape)
    if tuple(v.shape) != (tk, hkv, dk) or dk != d or hq % hkv:
        raise ValueError("sageattn_varlen (B200 path): q, k, v shapes do not fit together")
    if d % 8 or not (8 <= d <= HEAD_DIM):
        raise NotImplementedError("sageattn (B200 path) serves head_dim 8..128 in multiples of 8")
    n_seq = cu_q.numel() - 1
    if n_seq < 1 or cu_k.numel() != n_seq + 1:
        raise ValueError("sageattn_varlen (B200 path): cumulative lengths need batch + 1 entries each")
    max_q, max_k = int(max_q), int(max_k)
    if not (1 <= max_q <= tq and 1 <= max_k <= tk):
        raise ValueError("sageattn_varlen (B200 path): max_seqlen outside 1..total tokens")
    if is_causal and max_q != max_k:
        raise ValueError("sageattn_varlen (B200 path): a causal call needs q_len == kv_len")
    scale = d ** -0.5 if sm_scale is None else float(sm_scale)
    if not (0.0 < scale < float("inf")):
        raise ValueError("sageattn (B200 path): sm_scale must be finite and positive, got %r" % (sm_scale,))
    lib = _native.load()
    dev = q.device
    if out is None:
        out = torch.empty((tq, hq, d), dtype=q.dtype, device=dev)
    elif tuple(out.shape) != (tq, hq, d) or out.dtype != q.dtype or packed_view_reason(out) is not None:
        raise ValueError("out must have q's shape and dtype and be a servable view")
    offs = (ctypes.c_size_t * 13)()
    if lib.sage_workspace_layout_ex(n_seq, hq, hkv, max_q, max_k, offs) != 13:
        _native.check(-1, "sage_workspace_layout_ex")
    ws_bytes, status_off = varlen_workspace_bytes(n_seq, hq, hkv, max_q, max_k), int(offs[10])
    stream_id = torch.cuda.current_stream(dev).cuda_stream
    st = _state(dev, stream_id)
    if st.host_word is not None and st.host_word.value:
        st.raise_if_failed("the next call on the stream")
    ws = st.ws
    if ws is None or ws.numel() < ws_bytes:
        ws = _grow(st, dev, ws_bytes)
    st.status_off, st.shape = status_off, (n_seq, hq, hkv, max_q, max_k)
    capturing = torch.cuda.is_current_stream_capturing()
    watch = _WATCH and not (capturing and st.host_word is None)
    args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), cu_q.data_ptr(), cu_k.data_ptr(),
            ws.data_ptr(), ws.numel(), n_seq, hq, hkv, tq, tk, max_q, max_k, d,
            _native.strides2(q.stride(0), q.stride(1)), _native.strides2(k.stride(0), k.stride(1)),
            _native.strides2(v.stride(0), v.stride(1)), _native.strides2(out.stride(0), out.stride(1)),
            _dtype_code(q.dtype), -1, 1 if is_causal else 0, 1 if smooth_k else 0, scale, stream_id)
    with torch.cuda.device(dev):
        rc = lib.sage_attention_varlen(*args)
        if watch and not rc:
            rc = lib.sage_status_mirror(ws.data_ptr() + status_off, ctypes.addressof(_host_word(st)), 1, stream_id)
    if rc:
        _native.check(rc, "sage_attention_varlen")
    if _STRICT:
        torch.cuda.current_stream(dev).synchronize()
        st.raise_if_failed("this call (strict mode)")
    return out


def workspace_views(b: int, h: int, n: int, ws: torch.Tensor, int8: bool) -> Dict[str, torch.Tensor]:
    """Typed views of the intermediates inside a `sage_attention` workspace (for tests/tools)."""
    lib = _native.load()
    offs = (ctypes.c_size_t * 11)()
    if lib.sage_workspace_layout(b, h, n, offs) != 11:
        raise _native.SageNativeError("sage_workspace_layout failed")
    bh, n_pad, d = b * h, pad_len(n), HEAD_DIM
    code_dt = torch.int8 if int8 else torch.float8_e4m3fn

    def seg(i, nbytes):
        return ws[offs[i]: offs[i] + nbytes]
    return dict(
        q8=seg(0, bh * n * d).view(code_dt).view(bh, n, d),
        sq=seg(1, bh * n * 4).view(torch.float32).view(bh, n),
        k8=seg(2, bh * n_pad * d).view(code_dt).view(bh, n_pad, d),
        sk=seg(3, bh * n_pad * 4).view(torch.float32).view(bh, n_pad),
        v8t=seg(4, bh * n_pad * d).view(torch.float8_e4m3fn).view(bh, d, n_pad),
        sv=seg(5, bh * n_pad * 4).view(torch.float32).view(bh, n_pad),
        svp=seg(6, bh * n_pad * 4).view(torch.float32).view(bh, n_pad),
        S=seg(7, bh * 4).view(torch.float32),
        mean=seg(8, bh * d * 4).view(torch.float32).view(bh, d),
        status=seg(10, 4).view(torch.int32))


def last_status(q_like: torch.Tensor, b: int, h: int, n: int, hkv: Optional[int] = None,
                nk: Optional[int] = None) -> int:
    """Status word of the most recent `sage_call` on the current stream of q_like's device, read
    from that call's workspace (synchronises).  The shape must be that call's shape; raises
    RuntimeError if no call has run on the stream or the last one had another shape."""
    dev = q_like.device
    stream = torch.cuda.current_stream(dev)
    st = _state(dev, stream.cuda_stream, create=False)
    want = (b, h, h if hkv is None else hkv, n, n if nk is None else nk)
    if st is None or st.ws is None or st.shape is None:
        raise RuntimeError("last_status: no call has run on this stream")
    if st.shape != want:
        raise RuntimeError("last_status: the last call on this stream had shape %r, not %r" % (st.shape, want))
    stream.synchronize()
    return int(st.ws[st.status_off: st.status_off + 4].view(torch.int32).item())


def status() -> dict:
    """Small status record in the spirit of the reference's int8_status()/bf16_status()
    (sageattention/sk1_backend/__init__.py:529-558).  `device_status` lists the non-zero status
    words already copied back from finished calls, per (device, stream); nothing is synchronised."""
    info = dict(library=_native.LIB_PATH, loaded=_native._lib is not None, calls=_counters["calls"],
                refusals=_counters["refusals"], arch="sm_100a", tile=TILE, head_dim=HEAD_DIM,
                strict=_STRICT, watch=_WATCH)
    with _ws_lock:
        info["device_status"] = {key: st.pending() for key, st in _states.items() if st.pending()}
        info["fast_path"] = {key: dict(last_probe_share=st.last_share,
                                       signatures_on_plain_kernels=sum(1 for v in st.adaptive.plain_left.values() if v > 0))
                             for key, st in _states.items()}
    info["adaptive"] = _ADAPTIVE
    try:
        info["version"] = _native.load().sage_version()
    except _native.SageNativeError as exc:
        info["error"] = str(exc)
    return info
