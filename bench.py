"""Benchmark of the quantize-then-attend call on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--causal]

One step = one full `sageattn` call (quantisation prologue + attention kernel) on the video-length
configuration the headline metric is quoted on: B=1, H=48, N=47520, D=128, fp16, smooth_k on,
Q, K, V ~ N(0,1) with a seeded 0.1 % of the K tokens scaled x50 (seeded synthetic data stands in
for the reference's activation captures).  With N > 1 GPUs (launched with torch.distributed.run,
one rank per GPU) every rank runs that workload on its own batch element: the path shards over
(batch, head) with no collective, so the per-GPU work is fixed and the scaling is "weak".

Printed: ONE JSON line with whole-job TFLOPS (4*B*H*N^2*D flops per call, halved when causal),
the attention kernel's tensor roofline, the prologue's HBM figure, an end-to-end number measured
through the public API from pinned host buffers, and a bounded CPU baseline (the oracle, i.e. a
PyTorch port of the reference's numerics, on the host cores).

Beside the headline line the same JSON object carries: `roofline.peak_8bit_measured` (dense int8
and e4m3 matrix products of 8192^3 through torch's library calls, burst and sustained, with the SM
clock each was taken at: the yardstick the attention kernel's fraction is quoted against),
`config5` (the strong-scaling configuration: B=4, H=48, N=47520, bf16, non-causal, its 192
(batch, head) units partitioned over the ranks), `other_arms` (the other masking mode, bf16, the
image-size configurations at N=8771 and the short-call sweep), and with N > 1 `gather_ok` (one
NCCL all-gather of per-rank outputs outside every timed region).

`--impl reference` times that CPU port alone, with all host threads, on a bounded sample of the
same workload (the reference's own kernels are AMD gfx1201 binaries and cannot run here).
`--accuracy` prints the accuracy table instead (CUDA path and oracle against fp32 SDPA, and the
CUDA path against the oracle, for the five configurations) and exits.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "sageattention-rdna4_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

B, H, N, D = 1, 48, 47520, 128
SEED = 0
METRIC = "attention TFLOPS (full call incl. quant) at H=48 N=47520 D=128"
# DRAM bytes of one attention-kernel launch, scaled from the ncu capture of the small case
# (H=16, N=16384: 103.9 MB read + 34.4 MB written against 100.7 + 3 + 67 MB algorithmic, the rest
# of the output still in L2 when the kernel ends): traffic grows with the operand sizes, so a full
# launch moves about its algorithmic bytes.  The figure is derived, not measured in this run.
TRAFFIC_SOURCE = ("derived, not measured in this run: algorithmic bytes x 0.984, the ratio of DRAM bytes to algorithmic "
                  "bytes in the ncu launch list of profiles/attn_fwd_kernel_H16_N16384_fp16_noncausal.md")
TRAFFIC_RATIO = 1464.0 / 1488.0


def attention_algorithmic_bytes(batch: int = B) -> float:
    """Compulsory HBM traffic of one attention launch: codes of Q, K, V^T once, the four scale
    vectors, the output."""
    bh, n_pad = batch * H, (N + 127) // 128 * 128
    return bh * N * D + 2 * bh * n_pad * D + 4 * (bh * N + 2 * bh * n_pad) + bh * N * D * 2


def flops(causal: bool, batch: int = B) -> float:
    return 4.0 * batch * H * N * N * D * (0.5 if causal else 1.0)


def prologue_bytes() -> float:
    """Minimum traffic of the prologue: read Q, K, V once; write the three code tensors and the
    scales (K read once; the second read for the mean is not counted)."""
    bh, n_pad = B * H, (N + 127) // 128 * 128
    return 3 * bh * N * D * 2 + bh * N * D + 2 * bh * n_pad * D + 4 * (bh * N + 3 * bh * n_pad)


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        return dict(source="measured", hbm_gbs=float(m["hbm_gbs"]), bf16_tflops=float(m["bf16_tflops"]),
                    bf16_tflops_sustained=float(m.get("bf16_tflops_sustained", m["bf16_tflops"])))
    return dict(source="fallback", hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) during the timed region."""

    def __init__(self, index: int, period: float = 0.05):
        self.period = period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        med = statistics.median(self.samples) if self.samples else None
        return dict(sm_mhz=med, sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons), samples=len(self.samples))


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


def bind_near_gpu(phys_index: int) -> str:
    """Run this process (and so first-touch its pinned host buffers) on the CPU cores next to its
    GPU, as NVML reports them: with several ranks per host the end-to-end copies otherwise cross
    the socket interconnect.  Only this process's CPU affinity changes; no GPU setting is touched."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(phys_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        near = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        near &= os.sched_getaffinity(0)
        if near:
            os.sched_setaffinity(0, near)
            return "%d cores next to GPU %d" % (len(near), phys_index)
        return "unchanged (no allowed core next to the GPU)"
    except Exception as exc:          # NVML missing or affinity not permitted: measure as is
        return "unchanged (%s)" % type(exc).__name__


OUTLIER_FRAC = 0.001


def make_workload(dtype=torch.float16):
    from oracle import ref_numerics as R   # input generator only; nothing of the oracle is timed here
    return R.make_inputs(B, H, N, D, dtype, seed=SEED, outlier_frac=OUTLIER_FRAC)


def cpu_baseline(causal: bool, rows: int = 0) -> dict:
    """The oracle (PyTorch port of the reference numerics) on the host cores, on a bounded sample:
    the full prologue of ONE of the 48 heads plus the attention of `rows` query rows of that head
    (the first rows against all keys; when causal, the block in the middle of the sequence, which
    sees the average number of keys).  Same flop formula as the GPU number."""
    from oracle import ref_numerics as R
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rows = rows or N
    q, k, v = R.make_inputs(1, 1, N, D, torch.float16, seed=SEED, outlier_frac=0.001)
    row0 = max(0, N // 2 - rows // 2) if causal else 0
    t0 = time.perf_counter()
    pq = R.prologue(q, k, v, smooth_k=True)
    R.attend(pq["q8"][:, :, row0:row0 + rows], pq["sq"][:, :, row0:row0 + rows], pq["k8"], pq["sk"], pq["v8"],
             pq["svp"], pq["S"], N, causal, D ** -0.5, torch.float16, row_chunk=2048, row0=row0)
    dt = time.perf_counter() - t0
    keys = (row0 + rows / 2.0) if causal else N
    fl = 4.0 * rows * keys * D
    return dict(value=fl / dt / 1e12, unit="TFLOP/s", cores=cores, kind="port",
                sample="1 of %d heads: prologue of that head + attention of %d query rows (from row %d) over "
                       "%d keys = %.2e of the call's flops, %.1f s" % (H, rows, row0, int(keys), fl / flops(causal), dt))


def measure_8bit_peaks(dev, phys_index: int, sustain_s: float = 4.0) -> dict:
    """Dense 8-bit matrix-product rate of this GPU, the yardstick for the attention kernel: int8
    (torch._int_mm) and e4m3 (torch._scaled_mm) at 8192^3 through the vendor library, as a burst
    (best of 10 single launches) and sustained (back to back for about `sustain_s` seconds, where
    the power cap settles the clock), each with the median SM clock seen while it ran.  Library
    calls are used here as a measuring stick only; nothing of the product path runs through them."""
    n = 8192
    fl = 2.0 * n ** 3
    res = {"shape": "8192^3", "how": "burst = best of 10 launches (CUDA events); sustained = back to back for ~%.0f s" % sustain_s}

    def burst(name, fn):
        try:
            for _ in range(3):
                fn()
            torch.cuda.synchronize(dev)
            time.sleep(1.0)                            # from an idle, cool GPU
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            best = float("inf")
            with ClockSampler(phys_index, period=0.002) as c0:
                for _ in range(10):
                    a.record()
                    fn()
                    b.record()
                    torch.cuda.synchronize(dev)
                    best = min(best, a.elapsed_time(b))
            res[name] = dict(burst_tflops=fl / (best * 1e-3) / 1e12, burst_ms=best, burst_sm_mhz=c0.summary()["sm_mhz"])
        except Exception as exc:                       # the library refused the call: say so, measure the rest
            res[name] = dict(error="%s: %s" % (type(exc).__name__, str(exc)[:200]))

    def sustained(name, fn):
        if "error" in res.get(name, {}):
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = max(10, int(sustain_s * 1e3 / res[name]["burst_ms"]))
        with ClockSampler(phys_index) as c1:
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            torch.cuda.synchronize(dev)
        sus = a.elapsed_time(b) / iters
        res[name].update(sustained_tflops=fl / (sus * 1e-3) / 1e12, sustained_sm_mhz=c1.summary()["sm_mhz"],
                         sustained_reasons=c1.summary()["reasons"], sustained_iters=iters)

    a8 = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev)
    b8 = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev).t()      # column-major operand
    af = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    bf = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
    one = torch.ones((), dtype=torch.float32, device=dev)
    f_i8 = lambda: torch._int_mm(a8, b8)
    f_f8 = lambda: torch._scaled_mm(af, bf, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    burst("int8", f_i8)                                # both bursts before either long loop heats the part
    burst("e4m3", f_f8)
    sustained("int8", f_i8)
    time.sleep(1.0)
    sustained("e4m3", f_f8)
    del a8, b8, af, bf
    return res


def mixed_peak(p8: dict, key: str, int8_qk: bool):
    """Peak of the attention kernel's mix of products: Q.K^T in int8 (fp16 inputs) or e4m3 (bf16
    inputs) and P.V in e4m3, half of the flops each, so the harmonic mean of the two rates."""
    try:
        qk = p8["int8" if int8_qk else "e4m3"][key]
        pv = p8["e4m3"][key]
        return 2.0 / (1.0 / qk + 1.0 / pv)
    except (KeyError, TypeError, ZeroDivisionError):
        return None


def config5_block(dev, world: int, rank: int, steps: int, sync_all, max_over_ranks) -> dict:
    """The scaling configuration as written: B=4, H=48, N=47520, D=128, bf16, non-causal,
    smooth_k on, Q, K, V ~ N(0,1).  Its 192 (batch, head) units are partitioned over the ranks
    (192 / 96 / 48 / 24 units per GPU at 1 / 2 / 4 / 8 GPUs: total work fixed, strong scaling); no
    collective on the data path.  Timed with CUDA events between barriers, max over ranks."""
    import sageattention
    from sageattention.sharding import partition_units, sageattn_sharded
    units_total = 4 * H
    lo, hi = partition_units(units_total, world, rank)
    u = hi - lo
    g = torch.Generator(device=dev).manual_seed(5000 + lo)
    q, k, v = (torch.randn(1, u, N, D, generator=g, device=dev, dtype=torch.bfloat16) for _ in range(3))
    for _ in range(2):
        out = sageattn_sharded(q, k, v, is_causal=False)
    sync_all()
    n_steps = max(3, min(steps, 5))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_steps):
        out = sageattn_sharded(q, k, v, is_causal=False)
    e1.record()
    sync_all()
    ms = max_over_ranks(e0.elapsed_time(e1)) / n_steps
    finite = bool(torch.isfinite(out[0, 0].float()).all().item())
    del q, k, v, out
    total = 4.0 * units_total * N * N * D / (ms * 1e-3) / 1e12
    return dict(workload="B=4 H=%d N=%d D=%d bf16 non-causal smooth_k: %d (batch, head) units, %d on this rank"
                         % (H, N, D, units_total, u),
                scaling="strong", units_total=units_total, units_rank0=u, steps=n_steps, ms_per_step=ms,
                tflops_total=total, tflops_per_gpu=total / world, output_finite=finite)


def gather_check(dev, world: int, rank: int) -> bool:
    """One all-gather of per-rank outputs over NCCL, outside every timed region: every rank
    computes its partition of a small replicated call, the outputs are gathered, and the result
    must equal the same call computed whole on this rank, bit for bit (units are independent)."""
    import torch.distributed as dist
    import sageattention
    from sageattention.sharding import partition_units, sageattn_sharded
    units = 2 * world + 1                                # ragged: the first rank takes one more
    g = torch.Generator().manual_seed(77)
    q, k, v = (torch.randn(1, units, 300, D, generator=g).half().to(dev) for _ in range(3))
    lo, hi = partition_units(units, world, rank)
    got = sageattn_sharded(q[:, lo:hi], k[:, lo:hi], v[:, lo:hi], is_causal=True, gather=True)
    whole = sageattention.sageattn(q, k, v, is_causal=True)
    ok = torch.tensor([1 if (got.shape == whole.shape and torch.equal(got, whole)) else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return bool(ok.item())


def other_arms(q, k, v, dev, causal_main: bool) -> dict:
    """Full-call numbers for the arms the headline does not cover: the other masking mode, bf16
    inputs (e4m3 Q.K), and the short-call sweep of the configurations (fp16, H=48, non-causal,
    N in 288..4096, every call timed alone between two synchronisations, median of 20)."""
    import sageattention

    def timed(fn, iters):
        fn(); fn()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b) / iters

    out = {}
    # The headline inputs have 0.1 % dominant keys, on which the attention kernel's negligible-tile
    # fast path skips the exponentials of most key tiles.  Two lines put that in the open: the
    # same call with the path switched off (every tile exponentiated, as the reference does), and
    # the same shape on inputs without dominant keys (nothing to skip).
    from sageattention import _native
    lib = _native.load()
    lib.sage_debug_skip_threshold(0.0)
    try:
        ms = timed(lambda: sageattention.sageattn(q, k, v, is_causal=causal_main), 3)
    finally:
        lib.sage_debug_skip_threshold(-1.0)
    out["headline_fast_path_off"] = dict(ms=ms, tflops=flops(causal_main) / (ms * 1e-3) / 1e12)
    gen = torch.Generator(device=dev).manual_seed(SEED)
    kd = torch.randn(k.shape, generator=gen, device=dev, dtype=torch.float32).to(k.dtype)
    from sageattention import b200_backend as be
    be.reset_adaptive()          # same shape, other data: what the headline calls taught does not apply
    ms = timed(lambda: sageattention.sageattn(q, kd, v, is_causal=causal_main), 3)
    out["headline_shape_without_dominant_keys"] = dict(ms=ms, tflops=flops(causal_main) / (ms * 1e-3) / 1e12)
    del kd
    be.reset_adaptive()
    ms = timed(lambda: sageattention.sageattn(q, k, v, is_causal=not causal_main), 3)
    out["fp16_%s" % ("causal" if not causal_main else "non_causal")] = dict(
        ms=ms, tflops=flops(not causal_main) / (ms * 1e-3) / 1e12)
    qb, kb, vb = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    for c in (False, True):
        ms = timed(lambda: sageattention.sageattn(qb, kb, vb, is_causal=c), 3)
        out["bf16_%s" % ("causal" if c else "non_causal")] = dict(ms=ms, tflops=flops(c) / (ms * 1e-3) / 1e12)
    del qb, kb, vb
    # the image-size configurations (N = 8771): fp16 non-causal with a per-channel K bias and
    # per-head Q/K multipliers; bf16 causal with the K bias.  20 calls back to back.
    from oracle import ref_numerics as R               # input generator only
    n_img = 8771
    fl_img = 4.0 * H * n_img * n_img * D
    q2, k2, v2 = (t.to(dev) for t in R.make_inputs(1, H, n_img, D, torch.float16, seed=SEED, k_bias_std=1.0, head_scale=True))
    ms = timed(lambda: sageattention.sageattn(q2, k2, v2, is_causal=False), 20)
    out["config2_image_size_fp16_non_causal_n8771"] = dict(ms=ms, tflops=fl_img / (ms * 1e-3) / 1e12)
    q3, k3, v3 = (t.to(dev) for t in R.make_inputs(1, H, n_img, D, torch.bfloat16, seed=SEED, k_bias_std=1.0))
    ms = timed(lambda: sageattention.sageattn(q3, k3, v3, is_causal=True), 20)
    out["config3_image_size_bf16_causal_n8771"] = dict(ms=ms, tflops=0.5 * fl_img / (ms * 1e-3) / 1e12)
    del q2, k2, v2, q3, k3, v3
    short = {}
    for n in (288, 512, 1024, 4096):
        qs, ks, vs = (t[:, :, :n].contiguous() for t in (q, k, v))
        sageattention.sageattn(qs, ks, vs)
        samples = []
        for _ in range(20):
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
            sageattention.sageattn(qs, ks, vs)
            torch.cuda.synchronize(dev)
            samples.append((time.perf_counter() - t0) * 1e3)
        med = statistics.median(samples)
        short[str(n)] = dict(ms=med, tflops=4.0 * H * n * n * D / (med * 1e-3) / 1e12)
    out["short_calls_fp16_non_causal_wall_clock"] = short
    # call shapes beyond the reference's hand-written envelope, same H and N as the headline
    n = q.shape[2]
    wide = {}
    ms = timed(lambda: sageattention.sageattn(q, k, v, is_causal=causal_main, return_lse=True), 3)
    wide["return_lse"] = dict(ms=ms, tflops=flops(causal_main) / (ms * 1e-3) / 1e12)
    ms = timed(lambda: sageattention.sageattn(q, k, v, is_causal=causal_main, smooth_v=True), 3)
    wide["smooth_v"] = dict(ms=ms, tflops=flops(causal_main) / (ms * 1e-3) / 1e12)
    kg, vg = k[:, :8].contiguous(), v[:, :8].contiguous()
    ms = timed(lambda: sageattention.sageattn(q, kg, vg, is_causal=causal_main), 3)
    wide["grouped_query_48q_8kv"] = dict(ms=ms, tflops=flops(causal_main) / (ms * 1e-3) / 1e12)
    q64, k64, v64 = (t[..., :64].contiguous() for t in (q, k, v))
    ms = timed(lambda: sageattention.sageattn(q64, k64, v64, is_causal=causal_main), 3)
    wide["head_dim_64"] = dict(ms=ms, tflops=0.5 * flops(causal_main) / (ms * 1e-3) / 1e12,
                               note="flops counted at head_dim 64; the codes are zero-filled to 128 columns")
    del q64, k64, v64, kg, vg
    seqs, ln = 11, 4096                                  # packed batch of 11 sequences of 4096 tokens
    qv, kv, vv = (t[0, :, :seqs * ln].transpose(0, 1).contiguous() for t in (q, k, v))
    cu = torch.arange(0, (seqs + 1) * ln, ln, dtype=torch.int32)
    ms = timed(lambda: sageattention.sageattn_varlen(qv, kv, vv, cu, cu, ln, ln, is_causal=causal_main), 3)
    wide["varlen_11x4096"] = dict(ms=ms, tflops=seqs * 4.0 * H * ln * ln * D * (0.5 if causal_main else 1.0)
                                  / (ms * 1e-3) / 1e12)
    # a ragged packed batch, lengths on the device: one call of the kernels, nothing read back;
    # beside it the same batch split into per-length calls (the form that needs the lengths on the host)
    lens = [8192, 1024, 4096, 2048, 6144, 512, 3072, 7168, 1536, 5120, 6144]
    tot = sum(lens)
    qv, kv, vv = (t[0, :, :tot].transpose(0, 1).contiguous() for t in (q, k, v))
    cu_host = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    cu_dev = cu_host.to(dev)
    rag_flops = sum(4.0 * H * n * n * D for n in lens) * (0.5 if causal_main else 1.0)
    ms = timed(lambda: sageattention.sageattn_varlen(qv, kv, vv, cu_dev, cu_dev, max(lens), max(lens),
                                                     is_causal=causal_main), 3)
    wide["varlen_ragged_11_sequences_one_call"] = dict(ms=ms, tflops=rag_flops / (ms * 1e-3) / 1e12, tokens=tot)
    import sageattention.core as _core
    saved = (_core._VARLEN_SLOT_FACTOR, _core._VARLEN_SLOT_FREE_BYTES)
    _core._VARLEN_SLOT_FACTOR, _core._VARLEN_SLOT_FREE_BYTES = 0, 0
    try:
        ms = timed(lambda: sageattention.sageattn_varlen(qv, kv, vv, cu_host, cu_host, max(lens), max(lens),
                                                         is_causal=causal_main), 3)
    finally:
        _core._VARLEN_SLOT_FACTOR, _core._VARLEN_SLOT_FREE_BYTES = saved
    wide["varlen_ragged_11_sequences_call_per_length"] = dict(ms=ms, tflops=rag_flops / (ms * 1e-3) / 1e12)
    out["wider_call_shapes"] = wide
    return out


def run_accuracy() -> int:
    """Accuracy table of the CUDA path on the benchmark configurations: cosine / relative L1 /
    relative RMS against fp32 SDPA, the oracle's own error against SDPA beside it, and the CUDA
    path against the oracle evaluated with the kernel's 128-key tile and with the reference's
    64-key tile.  The oracle and SDPA are evaluated by torch on the device; for the large
    configurations on a subset of heads (the call itself runs with all heads).  One JSON line."""
    import sageattention
    from oracle import ref_numerics as R
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rows = []

    def add(name, q, k, v, causal, heads):
        out = sageattention.sageattn(q, k, v, is_causal=causal)
        torch.cuda.synchronize(dev)
        sl = torch.tensor(heads, device=dev)
        qs, ks, vs, os_ = q[:, sl], k[:, sl], v[:, sl], out[:, sl]
        ref = R.sdpa_fp32(qs, ks, vs, is_causal=causal)
        o128 = R.sageattn_oracle(qs, ks, vs, is_causal=causal, tile=128)
        o64 = R.sageattn_oracle(qs, ks, vs, is_causal=causal, tile=64)
        m = lambda a, b: dict(cos=R.cosine(a, b), rel_l1=R.rel_l1(a, b), rel_rms=R.rel_rms(a, b))
        rows.append(dict(config=name, heads_compared=len(heads), cuda_vs_sdpa=m(os_, ref), oracle64_vs_sdpa=m(o64, ref),
                         cuda_vs_oracle128=m(os_, o128), cuda_vs_oracle64=m(os_, o64)))

    to = lambda ts: tuple(t.to(dev) for t in ts)
    add("1: B=1 H=4 N=512 fp16 non-causal, K bias 0.5", *to(R.make_inputs(1, 4, 512, D, torch.float16, seed=0, k_bias_std=0.5)),
        False, [0, 1, 2, 3])
    add("2: B=1 H=48 N=8771 fp16 non-causal, K bias 1, head multipliers",
        *to(R.make_inputs(1, 48, 8771, D, torch.float16, seed=0, k_bias_std=1.0, head_scale=True)), False, [0, 15, 31, 47])
    add("3: B=1 H=48 N=8771 bf16 causal, K bias 1",
        *to(R.make_inputs(1, 48, 8771, D, torch.bfloat16, seed=0, k_bias_std=1.0)), True, [0, 15, 31, 47])
    q, k, v = to(R.make_inputs(1, 48, 47520, D, torch.float16, seed=0, outlier_frac=0.001))
    for dt in (torch.float16, torch.bfloat16):
        for causal in (False, True):
            add("4: B=1 H=48 N=47520 %s %s, 0.1%% K tokens x50" % ("fp16" if dt == torch.float16 else "bf16",
                                                                    "causal" if causal else "non-causal"),
                q.to(dt), k.to(dt), v.to(dt), causal, [0, 47])
    del q, k, v
    g = torch.Generator(device=dev).manual_seed(5)
    q, k, v = (torch.randn(4, 48, 47520, D, generator=g, device=dev, dtype=torch.bfloat16) for _ in range(3))
    out = sageattention.sageattn(q, k, v)
    torch.cuda.synchronize(dev)
    qs, ks, vs, os_ = q[3:4, 46:48], k[3:4, 46:48], v[3:4, 46:48], out[3:4, 46:48]
    ref = R.sdpa_fp32(qs, ks, vs)
    o128 = R.sageattn_oracle(qs, ks, vs, tile=128)
    o64 = R.sageattn_oracle(qs, ks, vs, tile=64)
    m = lambda a, b: dict(cos=R.cosine(a, b), rel_l1=R.rel_l1(a, b), rel_rms=R.rel_rms(a, b))
    rows.append(dict(config="5: B=4 H=48 N=47520 bf16 non-causal (units 190, 191 of 192)", heads_compared=2,
                     cuda_vs_sdpa=m(os_, ref), oracle64_vs_sdpa=m(o64, ref), cuda_vs_oracle128=m(os_, o128),
                     cuda_vs_oracle64=m(os_, o64)))
    print(json.dumps(dict(accuracy=rows, note="oracle = PyTorch restatement of the reference numerics; "
                                              "tolerance bars: vs oracle128 cos>=0.9999 rel_l1<=5e-3, vs oracle64 "
                                              "cos>=0.9995 rel_l1<=2e-2, vs SDPA rel_rms<0.08")))
    return 0


def run_reference(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(args.causal)
        if i >= args.warmup:
            times.append(base["value"])
    val = statistics.median(times)
    base["value"] = val
    line = dict(metric=METRIC, value=val, unit="TFLOP/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=None, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="int8+fp8",
                data="synthetic", impl="reference",
                config=workload_config(args.causal, args.gpus), cpu_baseline=base,
                e2e=dict(value=val, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))
    return 0


def workload_config(causal: bool, gpus: int) -> dict:
    return dict(workload="video-length attention B=%d(per GPU) H=%d N=%d D=%d fp16 %s smooth_k, %s"
                % (B, H, N, D, "causal" if causal else "non-causal",
                   ("%.2g%% K tokens x50" % (100 * OUTLIER_FRAC)) if OUTLIER_FRAC else "no dominant keys (profiling aid)"),
                global_batch=B * gpus, heads=H, seq_len=N, head_dim=D, causal=causal, seed=SEED,
                sharding="batch x head units across GPUs, no collective" if gpus > 1 else "single GPU",
                l2="inputs (3 x 584 MB) exceed the 126 MB L2; no explicit flush")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the causal / bf16 / short-call arms")
    ap.add_argument("--no-peak", action="store_true", help="skip the dense 8-bit peak measurement")
    ap.add_argument("--no-config5", action="store_true", help="skip the strong-scaling configuration")
    ap.add_argument("--accuracy", action="store_true", help="print the accuracy table and exit")
    ap.add_argument("--no-outliers", action="store_true",
                    help="profiling aid: inputs without the x50 key tokens (no key tile is negligible then)")
    ap.add_argument("--outlier-frac", type=float, default=None,
                    help="profiling aid: another share of x50 key tokens (a small --shape with as many such "
                         "tokens as the full-size workload skips a comparable share of its key tiles)")
    ap.add_argument("--e2e-groups", type=int, default=0,
                    help="head groups a step of the end-to-end pipeline is issued as (0: the default)")
    ap.add_argument("--shape", default=None, metavar="H,N",
                    help="override heads and sequence length (profiling captures on a smaller case)")
    args = ap.parse_args()
    if args.shape:
        global H, N
        H, N = (int(x) for x in args.shape.split(","))
    global OUTLIER_FRAC
    if args.no_outliers:
        OUTLIER_FRAC = 0.0
    elif args.outlier_frac is not None:
        OUTLIER_FRAC = float(args.outlier_frac)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    if args.accuracy:
        return run_accuracy()

    import torch.distributed as dist
    import sageattention
    from sageattention import b200_backend as be

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    causal = args.causal
    workload = make_workload()
    all_cores = os.sched_getaffinity(0)
    affinity = bind_near_gpu(physical_gpu_index(local))      # the pinned buffers are first touched here
    q_h, k_h, v_h = (t.pin_memory() for t in workload)
    out_h = torch.empty_like(q_h).pin_memory()
    out_h_alt = torch.empty_like(q_h).pin_memory()
    os.sched_setaffinity(0, all_cores)                       # everything else (CPU baseline included) as before
    del workload
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    stream = torch.cuda.current_stream(dev)

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- the prologue alone, before the GPU has been under the attention kernel for seconds ----
    # (after that its SM clock sags under the power cap for a while and the quantiser, which keeps the
    # SMs busy while it streams, reads 1 to 5 % slower; the HBM yardstick was taken on a GPU at rest).
    # The prologue lasts about half a millisecond: timed call by call from an idle GPU, the host's
    # launch latency before the first kernel would be counted as kernel time.  So it is timed as a
    # back-to-back batch (the GPU is still busy with call i when call i+1 is enqueued).
    pq = be.quant_qkv(q, k, v)
    for _ in range(3):
        pq = be.quant_qkv(q, k, v, reuse=pq)
    torch.cuda.synchronize(dev)
    pro_iters = max(args.steps, 20)
    pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pe0.record(stream)
    for _ in range(pro_iters):
        pq = be.quant_qkv(q, k, v, reuse=pq)
    pe1.record(stream)
    torch.cuda.synchronize(dev)
    pro = pe0.elapsed_time(pe1) / pro_iters
    sync_all()

    # ---- device-resident throughput through the public API ----
    for _ in range(args.warmup):
        out = sageattention.sageattn(q, k, v, is_causal=causal)
    sync_all()

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local)) as clk:
        e0.record(stream)
        for _ in range(args.steps):
            out = sageattention.sageattn(q, k, v, is_causal=causal)
        e1.record(stream)
        sync_all()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    value = flops(causal, B * world) / (ms_step * 1e-3) / 1e12
    status = be.last_status(q, B, H, N)

    # ---- per-kernel durations (same launches through the two reference-shaped entry points) ----
    o2 = torch.empty_like(q)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    att_ms = []
    for i in range(args.warmup + args.steps):
        ev[0].record(stream)
        pq = be.quant_qkv(q, k, v, reuse=pq)
        ev[1].record(stream)
        be.attn_launch(pq, o2, causal, D ** -0.5, status=st)
        ev[2].record(stream)
        torch.cuda.synchronize(dev)
        if i >= args.warmup:
            att_ms.append(ev[1].elapsed_time(ev[2]))
    att = statistics.mean(att_ms)
    pk = peaks()
    achieved = flops(causal) / (att * 1e-3) / 1e12
    # The yardstick: this GPU's own dense 8-bit rate, measured in this run on rank 0 (the other
    # ranks wait).  The kernel's products are half int8 (Q.K^T) and half e4m3 (P.V).
    p8 = measure_8bit_peaks(dev, physical_gpu_index(local)) if (rank == 0 and not args.no_peak) else None
    if world > 1:
        dist.barrier()
    burst = mixed_peak(p8, "burst_tflops", True) if p8 else None
    sustained = mixed_peak(p8, "sustained_tflops", True) if p8 else None
    if burst:
        peak8, basis = burst, ("measured in this run: harmonic mean of the int8 and e4m3 8192^3 burst rates "
                               "(torch._int_mm / torch._scaled_mm); a launch is timed alone, so the burst figure")
    else:
        peak8, basis = 2.0 * pk["bf16_tflops"], "2 x bf16_tflops burst (%s) of MEASURED_PEAKS.json: no 8-bit figure measured in this run" % pk["source"]
    roofline = dict(bound="tensor", kernel="attn_fwd_kernel", achieved=achieved, peak=peak8, unit="TFLOP/s",
                    frac=achieved / peak8, ms_per_launch=att, peak_basis=basis,
                    peak_8bit_measured=p8,
                    frac_vs_measured_sustained=(achieved / sustained) if sustained else None,
                    frac_vs_2x_bf16_burst=achieved / (2 * pk["bf16_tflops"]),
                    frac_vs_2x_bf16_sustained=achieved / (2 * pk["bf16_tflops_sustained"]),
                    frac_vs_nominal_4500=achieved / 4500.0,
                    bf16_peaks_file=dict(source=pk["source"], burst=pk["bf16_tflops"], sustained=pk["bf16_tflops_sustained"]),
                    traffic=(attention_algorithmic_bytes() * TRAFFIC_RATIO) if not causal else None,
                    traffic_source=TRAFFIC_SOURCE,
                    algorithmic_bytes=attention_algorithmic_bytes())
    pro_gbs = prologue_bytes() / (pro * 1e-3) / 1e9
    prologue = dict(bound="hbm", kernel="clear_ctrl_kernel + kmean_kernel + quant_qkv_kernel", achieved=pro_gbs, peak=pk["hbm_gbs"],
                    unit="GB/s", frac=pro_gbs / pk["hbm_gbs"], ms=pro, algorithmic_bytes=prologue_bytes())

    # ---- end to end from pinned host buffers through the public API ----
    # Every step copies its three inputs from pinned host memory and reads its result back.
    # (a) serial: copies and the call on one stream; (b) pipelined, what a serving loop does: a
    # copy-in stream, the compute stream and a copy-out stream with two sets of device buffers,
    # so that step i+1's H2D and step i-1's D2H overlap step i's call.  (b) is the reported E.
    def e2e_step():
        qd = q_h.to(dev, non_blocking=True)
        kd = k_h.to(dev, non_blocking=True)
        vd = v_h.to(dev, non_blocking=True)
        o = sageattention.sageattn(qd, kd, vd, is_causal=causal)
        out_h.copy_(o, non_blocking=True)

    for _ in range(2):
        e2e_step()
    sync_all()
    e0.record(stream)
    for _ in range(args.steps):
        e2e_step()
    e1.record(stream)
    sync_all()
    e2e_serial_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps

    # The call shards over heads, so a step is issued as GROUPS head groups: group g's call starts as
    # soon as its slice has arrived and its result leaves as soon as it is done, which shortens the
    # fill and drain of the pipeline.  Consecutive groups alternate between two compute streams so
    # that the last CTAs of one group share the GPU with the first CTAs of the next.
    # (measured at the headline shape, ms per step: 4 groups 46.9, 6: 47.0, 8: 45.9, 12: 47.8, 16: 45.7
    # against 45.6 with the inputs resident: a group whose CTAs end in a nearly empty last wave costs more
    # than the shorter fill of a finer split returns)
    GROUPS = next((g for g in (16, 8, 4) if H % g == 0), 1)
    if args.e2e_groups > 0 and H % args.e2e_groups == 0:
        GROUPS = args.e2e_groups
    hg = H // GROUPS
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_cmp = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
    bufs = [tuple(torch.empty_like(q) for _ in range(3)) for _ in range(2)]
    ev_in = [[torch.cuda.Event() for _ in range(GROUPS)] for _ in range(2)]
    ev_cmp = [[torch.cuda.Event() for _ in range(GROUPS)] for _ in range(2)]
    out_h2 = [out_h, out_h_alt]

    def pipelined(n_steps, first):
        for i in range(first, first + n_steps):
            b = i & 1
            for g in range(GROUPS):
                hs = slice(g * hg, (g + 1) * hg)
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_cmp[b][g])              # the call that read this slice two steps ago is done
                    for dst, src in zip(bufs[b], (q_h, k_h, v_h)):
                        dst[:, hs].copy_(src[:, hs], non_blocking=True)
                    ev_in[b][g].record(s_in)
                sc = s_cmp[g & 1]
                with torch.cuda.stream(sc):
                    sc.wait_event(ev_in[b][g])
                    o = sageattention.sageattn(bufs[b][0][:, hs], bufs[b][1][:, hs], bufs[b][2][:, hs],
                                               is_causal=causal)
                    ev_cmp[b][g].record(sc)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[b][g])
                    out_h2[b][:, hs].copy_(o, non_blocking=True)
                    o.record_stream(s_out)

    pipelined(2, 0)
    sync_all()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(s_in)
    pipelined(args.steps, 2)
    s_out.wait_stream(s_in)
    s_out.wait_stream(s_cmp[0])
    s_out.wait_stream(s_cmp[1])
    t1.record(s_out)
    sync_all()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1)) / args.steps
    del bufs
    nbytes = q_h.numel() * q_h.element_size()
    e2e = dict(value=flops(causal, B * world) / (e2e_ms * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=e2e_ms,
               h2d_bytes_per_step=3 * nbytes, d2h_bytes_per_step=nbytes,
               how="copy-in, copy-out and two compute streams, two sets of device buffers; a step is issued as %d "
                   "head groups through the public API so that copies of one group overlap the calls of the others" % GROUPS,
               host_copy_gbs_per_rank=4 * nbytes / (e2e_ms * 1e-3) / 1e9,
               host_copy_gbs_aggregate=world * 4 * nbytes / (e2e_ms * 1e-3) / 1e9,
               host_affinity=affinity, serial_ms_per_step=e2e_serial_ms,
               serial_value=flops(causal, B * world) / (e2e_serial_ms * 1e-3) / 1e12)

    # ---- the scaling configuration (strong scaling over the 192 units) and the NCCL gather ----
    c5 = None if (args.shape or args.no_config5) else config5_block(dev, world, rank, args.steps, sync_all, max_over_ranks)
    gather_ok = gather_check(dev, world, rank) if world > 1 else None

    # ---- the other arms of the configurations (informative; N = 1 only) ----
    others = None
    if world == 1 and not args.no_extras and not args.shape:
        others = other_arms(q, k, v, dev, causal)

    if world > 1:
        dist.barrier()
    if rank == 0:
        line = dict(metric=METRIC, value=value, unit="TFLOP/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=ms_step, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="int8+fp8", data="synthetic", config=workload_config(causal, world),
                    roofline=roofline, prologue=prologue, e2e=e2e, gpu_launches=4 * args.steps,
                    clocks=clk.summary(), kernel_status=status)
        if c5 is not None:
            line["config5"] = c5
        if gather_ok is not None:
            line["gather_ok"] = gather_ok
        if others is not None:
            line["other_arms"] = others
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(causal)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
