// Quantisation prologue for B200: sequence mean of K (smooth_k; of V too with smooth_v), then one
// persistent, TMA-fed pass over the 128-token tiles of K, V and Q that writes the int8 / e4m3
// codes, the per-token scales and V transposed, and closes with the fold of the per-head S and its
// staged factor.
//
// Arithmetic contract (reference: kernels/hip/h34_prologue.hip:116-211,259-282;
// kernels/hip/sk1_t6i.hip:104-117; kernels/hip/sk1_t4a1sb.hip:89-100;
// sageattention/sk1_backend/__init__.py:577-579).  Every operation below is a separate correctly
// rounded fp32 operation, written with the __f*_rn intrinsics so that no contraction or fast-math
// flag can change it:
//   mean  = f32( sum_n f64(K[n,d]) / f64(N) )
//   K     : x = f32(k) - mean; sk = max(amax/127, 1e-12); code = clamp(rne(x / sk), -128, 127)
//           e4m3 arm: sk = max(amax/448, 1e-12); code = e4m3(min(x / sk, 448))
//   V     : sv = max(amax/448, 1e-12); code = e4m3(min(v / sv, 448)); stored transposed
//   Q     : amax = max(amax, 1e-12); code = clamp(rint(q * (127/amax))); scale = amax/127
//           e4m3 arm: code = e4m3(clamp(q * (448/amax), +-448)); scale = amax/448
//   pad   : K8 = 0, SK = 1, V8T = 0, SV = 0
//   S     = max(max_n sv, 1); SVP = fl(fl(sv / S) * 448)
// The clamps to +-448 are done by the saturating e4m3 conversion (same codes).
// The fp64 mean is summed in a different (wider) order than the reference's eight strided
// partials; both are exact, hence identical, whenever the fp64 partial sums are exact, which holds
// for fp16 data when sum|K| < 2^29 per channel and for bf16 data of ordinary dynamic range.
#include <cuda.h>

#include <algorithm>
#include <type_traits>

#include "sage_common.cuh"
#include "sage_internal.h"

namespace sage {

// ------------------------------------------------------------------------------------------------
// Kernel 0: clears the control words (arrival counters, running maxima, status words, work and
// skip counters) of a call.  A kernel rather than a memset so that it and the mean kernel behind it
// can be launched as programmatic dependents: their CTAs are placed while the kernel before them
// on the stream drains, and the stream has no memset node to serialise on.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) clear_ctrl_kernel(unsigned* __restrict__ words, int n) {
  wait_for_predecessor();            // an earlier call may still be using these words
  allow_successor();
  for (int i = threadIdx.x; i < n; i += 256) words[i] = 0u;
}

// ------------------------------------------------------------------------------------------------
// Kernel 1: partial fp64 column sums of K; the last CTA of a head combines them in split order.
// grid (nsplit, B*H), block 256 = 16 row lanes x 16 column chunks of 8 elements.
// ------------------------------------------------------------------------------------------------
template <typename T, bool VARLEN>
__global__ void __launch_bounds__(256)
kmean_kernel(const T* __restrict__ K, float* __restrict__ mean, double* __restrict__ partial,
             unsigned* __restrict__ arrivals, long long N, long long H,
             long long sb, long long sh, long long sr, int nsplit, long long chunk, int D,
             const int* __restrict__ cu, long long tokens) {
  __shared__ double red[16][HD];
  __shared__ int s_last;
  wait_for_predecessor();            // the cleared arrival counters
  allow_successor();                 // one wave: every CTA of this grid is resident
  const int tid = threadIdx.x, c = tid & 15, r = tid >> 4;
  const int split = blockIdx.x, bh = blockIdx.y;
  const long long b = bh / H, h = bh - b * H;
  const T* base = K + b * sb + h * sh + 8 * c;
  if (VARLEN) {                      // packed batch: this sequence's own length and first token
    // whatever the arrays hold, nothing outside the packed tokens is read
    const long long s0 = min(max((long long)cu[b], 0LL), tokens), s1 = min((long long)cu[b + 1], tokens);
    N = min(max(s1 - s0, 0LL), N);
    base = K + s0 * sr + h * sh + 8 * c;
  }
  const long long n0 = (long long)split * chunk;
  const long long n1 = min(N, n0 + chunk);

  double acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.0;
  const long long n_end = (8 * c < D) ? n1 : n0;   // columns past head_dim: nothing to read, mean 0
#pragma unroll 8
  for (long long n = n0 + r; n < n_end; n += 16) {
    const uint4 u = __ldcs(reinterpret_cast<const uint4*>(base + n * sr));   // streaming: read once here
    float x[8];
    unpack8<T>(u, x);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += (double)x[e];
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[r][8 * c + e] = acc[e];
  __syncthreads();
  if (tid < HD) {
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < 16; ++i) s += red[i][tid];
    partial[((size_t)bh * nsplit + split) * HD + tid] = s;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(&arrivals[bh], 1u) == (unsigned)(nsplit - 1));
  __syncthreads();
  if (s_last && tid < HD) {
    __threadfence();
    double tot = 0.0;
    for (int sp = 0; sp < nsplit; ++sp) tot += __ldcg(&partial[((size_t)bh * nsplit + sp) * HD + tid]);
    mean[(size_t)bh * HD + tid] = (!VARLEN || N > 0) ? (float)(tot / (double)N) : 0.f;
  }
}

// ------------------------------------------------------------------------------------------------
// Division.  K and V are divided by their scale with an IEEE-correct quotient obtained as
//   rc = rn(1/s) (correctly rounded);  q0 = rn(x*rc);  r = x - q0*s (one fma, exact);  q = fma(r, rc, q0)
// which equals rn(x/s) whenever rc is the correctly rounded reciprocal and nothing over/underflows
// (Markstein's theorem; |x/s| <= 448 and 1e-12 <= s here).  Three operations per element instead
// of a full division routine; checked against true division on 8e7 random samples on the host.
// Rounding to int8 uses the add-magic-constant trick (1.5*2^23): the addition rounds to nearest
// even, the low byte of the sum is the two's-complement code; |x/s| <= 127 needs no clamp.
// ------------------------------------------------------------------------------------------------
struct QuantArgs {
  uint8_t *q8, *k8, *v8t;
  float *sq, *sk, *sv, *svp, *s_fold;
  const float* mean;
  const float* vmean;             // optional: sequence mean of V, subtracted before quantising (smooth_v)
  unsigned* svmax_bits;           // per K/V head: running maximum of the V scales, as float bits
  unsigned* arrivals;             // per K/V head: V tiles whose scales are published
  long long N, N_pad, H;          // keys: length, padded length, K/V heads per batch element
  long long Nq, Hq, group;        // queries: length, heads per batch element, Hq / H (1 without GQA)
  long long BHq, BHkv;            // B*Hq, B*H
  float* qm;                      // optional (B*Hq, Nq): dot(q row, K mean of its K/V head), for the LSE
  int sub_mean;
  int32_t* status;                // set non-zero when a wait on a tile load ran out
  int32_t* status2;               // optional second word that receives the same report
  unsigned long long* next_item;  // global work counter (zeroed with the control block)
  const int *cu_q, *cu_k;         // VARLEN kernels: cumulative token counts of the packed batch (B + 1 entries each)
  long long Tq, Tk;               // VARLEN kernels: tokens in the packed q and k/v tensors
};

// rn(x / s) given rc = rn(1/s)
__device__ __forceinline__ float div_by_scale(float x, float s, float rc) {
  const float q0 = __fmul_rn(x, rc);
  const float r = -__fmaf_rn(q0, s, -x);      // x - q0*s, written so that a zero keeps x's sign
  return __fmaf_rn(r, rc, q0);
}

// ------------------------------------------------------------------------------------------------
// Kernel 2: persistent CTAs (three per SM) draw 128-token tiles of K, V and Q from one global work
// counter; thread 0 keeps the next tile's 32 KB tensor-map load in flight into a shared-memory
// ring while the 256 threads quantise the tile that has landed.  Out-of-range rows and, for
// head_dim < 128, out-of-range columns arrive as zeros from the tensor map.
// Thread (c = tid & 7, r0 = tid >> 3) owns columns 8c..8c+7 and 64+8c..64+8c+7 of rows r0, r0+32,
// r0+64, r0+96: a quarter-warp reads one 256-byte row with two conflict-free 16-byte loads and the
// row maximum is three shuffles.
// ------------------------------------------------------------------------------------------------
constexpr int QT_STAGES = 2;        // shared-memory ring: one tile being quantised, one in flight
constexpr int QT_MINBLOCKS = 3;     // CTAs per SM (3 x 64 KB of shared memory, 80 registers per thread)
constexpr int FOLD_KEYS = 4096;     // keys per fold item
constexpr uint32_t QT_STAGE_BYTES = TILE * HD * 2;
constexpr uint32_t QT_SMEM_BYTES = QT_STAGES * QT_STAGE_BYTES + 128 /* alignment slack */ + 64 /* barriers */;
constexpr long long QT_WAIT_CYCLES = 4000000000LL;

__device__ __forceinline__ uint32_t qt_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t qt_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ float quarter_warp_max(float x) {
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 4));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
  return x;
}
// rn(a / d) for a compile-time divisor: rc = rn(1/d) is a constant, the rest is Markstein's sequence
// (checked against true division over every mantissa of several binades for d = 127 and 448).
template <int DIV>
__device__ __forceinline__ float div_const(float a) {
  constexpr float d = (float)DIV, rc = 1.0f / (float)DIV;
  const float q0 = __fmul_rn(a, rc);
  const float r = __fmaf_rn(-q0, d, a);
  return __fmaf_rn(r, rc, q0);
}
__device__ __forceinline__ uint32_t i8x4_magic2(float2 ab, float2 cd) {
  const float2 m = make_float2(12582912.0f, 12582912.0f);
  const float2 u = __fadd2_rn(ab, m), v = __fadd2_rn(cd, m);
  return __byte_perm(__byte_perm(__float_as_uint(u.x), __float_as_uint(u.y), 0x0040),
                     __byte_perm(__float_as_uint(v.x), __float_as_uint(v.y), 0x0040), 0x5410);
}

// VARLEN: a packed batch.  N, N_pad and Nq are then the capacity of a sequence's slot in the outputs
// (sized for the longest sequence allowed); every sequence has its own length and its own first
// token in the inputs, read from cu_q / cu_k.  Tiles past a sequence's end are neither loaded nor
// written (the attention kernel never visits them).
template <typename T, bool INT8, bool VARLEN>
__global__ void __launch_bounds__(256, QT_MINBLOCKS)
quant_qkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const QuantArgs a) {
  extern __shared__ uint8_t qt_smem[];
  __shared__ long long s_item[QT_STAGES];
  wait_for_predecessor();            // the means and the cleared control block
  allow_successor();                 // persistent grid: every CTA is resident
  constexpr float QMAX = INT8 ? I8_MAX : F8_MAX;
  constexpr int QDIV = INT8 ? 127 : 448;

  const uint32_t raw_addr = qt_smem_u32(qt_smem);
  const uint32_t base = (raw_addr + 127u) & ~127u;
  uint8_t* gbase = qt_smem + (base - raw_addr);
  const uint32_t bar0 = base + QT_STAGES * QT_STAGE_BYTES;
  const int tid = threadIdx.x, c = tid & 7, r0 = tid >> 3, lane = tid & 31, warp = tid >> 5;

  const long long tiles_q = (a.Nq + TILE - 1) / TILE, tiles_k = a.N_pad / TILE;
  const long long items_k = a.BHkv * tiles_k, items_q = a.BHq * tiles_q;
  const long long fold_per_head = (a.N_pad + FOLD_KEYS - 1) / FOLD_KEYS;
  const long long items_f = a.BHkv * fold_per_head;
  const long long total = 2 * items_k + items_q + items_f;

  // item -> (tensor, head, tile): K first with the last heads first (their rows are still in L2
  // after the mean pass), then V (so that the per-head folds overlap the Q items), then Q
  auto decode = [&](long long it, int& which, long long& bh, long long& tile) {
    if (it < items_k) { which = 1; bh = a.BHkv - 1 - it / tiles_k; tile = it % tiles_k; }
    else if (it < 2 * items_k) { const long long j = it - items_k; which = 2; bh = a.BHkv - 1 - j / tiles_k; tile = j % tiles_k; }
    else if (it < 2 * items_k + items_q) { const long long j = it - 2 * items_k; which = 0; bh = a.BHq - 1 - j / tiles_q; tile = j % tiles_q; }
    else { const long long j = it - 2 * items_k - items_q; which = 3; bh = a.BHkv - 1 - j / fold_per_head; tile = j % fold_per_head; }
  };
  // length and first input token of the sequence an item belongs to
  auto seq_of = [&](int which, long long bh, long long& start) -> long long {
    if (!VARLEN) { start = 0; return (which == 0) ? a.Nq : a.N; }
    const long long b = bh / ((which == 0) ? a.Hq : a.H);
    const int* cu = (which == 0) ? a.cu_q : a.cu_k;
    // clamped to the packed tensor: whatever the arrays hold, a sequence lies inside it
    const long long T = (which == 0) ? a.Tq : a.Tk;
    const long long s0 = min(max((long long)__ldg(cu + b), 0LL), T), s1 = min((long long)__ldg(cu + b + 1), T);
    start = s0;
    return min(max(s1 - s0, 0LL), (which == 0) ? a.Nq : a.N);
  };
  // Items are handed out through one global counter: a CTA that is held up (by a head's fold, say)
  // simply takes fewer of them.  Thread 0 publishes the item of a stage in s_item and starts its
  // load; past the end it publishes -1 and completes the stage's barrier by hand.  The counter is
  // drawn one item ahead, so the atomic's round trip is off the critical path.
  auto draw = [&]() { return (long long)atomicAdd(a.next_item, 1ULL); };
  auto issue = [&](int stage, long long it) {
    const uint32_t bar_ = bar0 + 8u * (uint32_t)stage;
    if (it >= total) {
      s_item[stage] = -1;
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_) : "memory");
      return;
    }
    s_item[stage] = it;
    int which; long long bh, tile;
    decode(it, which, bh, tile);
    if (which == 3) {                  // fold items read no tile
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_) : "memory");
      return;
    }
    const long long heads = (which == 0) ? a.Hq : a.H;
    int b = (int)(bh / heads);
    const int h = (int)(bh - (long long)b * heads);
    long long row = tile * TILE;
    if (VARLEN) {                      // a tile past the sequence's end is not loaded; the map has one batch entry
      long long start;
      if (row >= seq_of(which, bh, start)) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_) : "memory");
        return;
      }
      row += start;
      b = 0;
    }
    const CUtensorMap* map = (which == 0) ? &tm_q : (which == 1 ? &tm_k : &tm_v);
    const uint32_t bar = bar0 + 8u * (uint32_t)stage, dst = base + (uint32_t)stage * QT_STAGE_BYTES;
    // the stage was last touched by ordinary loads and stores (V tiles are staged back into it);
    // order them before the copy engine's writes
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(QT_STAGE_BYTES) : "memory");
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"((int)row), "r"(h), "r"(b) : "memory");
  };

  if (tid == 0) {
    for (int s = 0; s < QT_STAGES; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 8u * (uint32_t)s), "r"(1u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  long long drawn = 0;
  if (tid == 0) {
    for (int p = 0; p < QT_STAGES - 1; ++p) issue(p, draw());
    drawn = draw();
  }

  for (uint32_t n = 0;; ++n) {
    const int stage = (int)(n % QT_STAGES);
    const uint32_t parity = (n / QT_STAGES) & 1u;
    if (tid == 0) {                    // into the stage released by the previous item
      issue((int)((n + QT_STAGES - 1) % QT_STAGES), drawn);
      drawn = draw();                  // consumed one iteration later
    }
    // bounded wait for this item's tile
    int ok = 1;
    {
      const uint32_t bar = bar0 + 8u * (uint32_t)stage;
      if (!qt_try_wait(bar, parity)) {
        const long long t0 = clock64();
        uint32_t spins = 0;
        while (!qt_try_wait(bar, parity)) {
          if ((++spins & 1023u) == 0u && clock64() - t0 > QT_WAIT_CYCLES) { ok = 0; break; }
        }
      }
    }
    if (!__syncthreads_and(ok)) {
      if (tid == 0) { atomicOr(a.status, 1); if (a.status2) atomicOr(a.status2, 8); }
      const long long t0 = clock64();
      while (clock64() - t0 < 400000) { }     // give copies still in flight a moment to land
      break;
    }

    const long long it = s_item[stage];
    if (it < 0) break;                 // the list is exhausted (every thread reads the same value)
    int which; long long bh, tile;
    decode(it, which, bh, tile);
    const long long n_base = tile * TILE;
    const uint8_t* st = gbase + (size_t)stage * QT_STAGE_BYTES;
    long long seq_start;
    const long long seq_len = seq_of(which == 3 ? 1 : which, bh, seq_start);
    const bool beyond = VARLEN && which != 3 && n_base >= seq_len;   // nothing was loaded, nothing is written

    if (beyond) {
    } else if (which == 0) {
      // ---------------------------------- Q ----------------------------------
      const long long N = VARLEN ? seq_len : a.Nq;
      float mu[16];
      if (a.qm != nullptr) {
        const long long b = bh / a.Hq, h = bh - b * a.Hq, bh_kv = b * a.H + h / a.group;
#pragma unroll
        for (int e = 0; e < 8; ++e) { mu[e] = a.mean[(size_t)bh_kv * HD + 8 * c + e]; mu[8 + e] = a.mean[(size_t)bh_kv * HD + 64 + 8 * c + e]; }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = r0 + 32 * i;
        const long long nrow = n_base + t;
        float x[16];
        unpack8<T>(*reinterpret_cast<const uint4*>(st + t * 256 + 16 * c), x);
        unpack8<T>(*reinterpret_cast<const uint4*>(st + t * 256 + 128 + 16 * c), x + 8);
        float amax = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(x[e]));
        amax = fmaxf(quarter_warp_max(amax), SCALE_FLOOR);
        const float qinv = __fdiv_rn(QMAX, amax);
        float2 y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = make_float2(__fmul_rn(x[2 * e], qinv), __fmul_rn(x[2 * e + 1], qinv));
        uint2 w0, w1;
        if (INT8) {
          w0.x = i8x4_magic2(y[0], y[1]); w0.y = i8x4_magic2(y[2], y[3]);
          w1.x = i8x4_magic2(y[4], y[5]); w1.y = i8x4_magic2(y[6], y[7]);
        } else {
          w0.x = e4m3x4(y[0].x, y[0].y, y[1].x, y[1].y); w0.y = e4m3x4(y[2].x, y[2].y, y[3].x, y[3].y);
          w1.x = e4m3x4(y[4].x, y[4].y, y[5].x, y[5].y); w1.y = e4m3x4(y[6].x, y[6].y, y[7].x, y[7].y);
        }
        if (nrow < N) {
          uint8_t* dst = a.q8 + ((size_t)bh * a.Nq + nrow) * HD + 8 * c;
          *reinterpret_cast<uint2*>(dst) = w0;
          *reinterpret_cast<uint2*>(dst + 64) = w1;
          if (c == 0) a.sq[(size_t)bh * a.Nq + nrow] = div_const<QDIV>(amax);
        }
        if (a.qm != nullptr) {                          // fixed-order fp32 dot product of the raw row
          float d = 0.f;
#pragma unroll
          for (int e = 0; e < 16; ++e) d = __fmaf_rn(x[e], mu[e], d);
          d += __shfl_xor_sync(0xffffffffu, d, 4);
          d += __shfl_xor_sync(0xffffffffu, d, 2);
          d += __shfl_xor_sync(0xffffffffu, d, 1);
          if (c == 0 && nrow < N) a.qm[(size_t)bh * a.Nq + nrow] = d;
        }
      }
    } else if (which == 1) {
      // ---------------------------------- K ----------------------------------
      const long long N = VARLEN ? seq_len : a.N, N_pad = a.N_pad;
      float2 nmu[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float* m0 = a.mean + (size_t)bh * HD + 8 * c + 2 * e;
        nmu[e] = a.sub_mean ? make_float2(-m0[0], -m0[1]) : make_float2(0.f, 0.f);
        nmu[4 + e] = a.sub_mean ? make_float2(-m0[64], -m0[65]) : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = r0 + 32 * i;
        const long long nrow = n_base + t;
        const bool live = nrow < N;
        float x[16];
        unpack8<T>(*reinterpret_cast<const uint4*>(st + t * 256 + 16 * c), x);
        unpack8<T>(*reinterpret_cast<const uint4*>(st + t * 256 + 128 + 16 * c), x + 8);
        float2 xs[8];
        float amax = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xs[e] = __fadd2_rn(make_float2(x[2 * e], x[2 * e + 1]), nmu[e]);
          amax = fmaxf(amax, fmaxf(fabsf(xs[e].x), fabsf(xs[e].y)));
        }
        amax = quarter_warp_max(live ? amax : 0.f);
        const float sk = fmaxf(div_const<QDIV>(amax), SCALE_FLOOR);
        const float rc = __frcp_rn(sk);
        uint2 w0, w1;
        if (INT8) {
          // the sign of a zero quotient does not reach an int8 code, so the packed form is enough
          const float2 rc2 = make_float2(rc, rc), ns2 = make_float2(-sk, -sk);
          float2 y[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float2 q0 = __fmul2_rn(xs[e], rc2);
            const float2 r = __ffma2_rn(q0, ns2, xs[e]);
            y[e] = __ffma2_rn(r, rc2, q0);
          }
          w0.x = i8x4_magic2(y[0], y[1]); w0.y = i8x4_magic2(y[2], y[3]);
          w1.x = i8x4_magic2(y[4], y[5]); w1.y = i8x4_magic2(y[6], y[7]);
        } else {
          float y[16];
#pragma unroll
          for (int e = 0; e < 8; ++e) { y[2 * e] = div_by_scale(xs[e].x, sk, rc); y[2 * e + 1] = div_by_scale(xs[e].y, sk, rc); }
          w0.x = e4m3x4(y[0], y[1], y[2], y[3]); w0.y = e4m3x4(y[4], y[5], y[6], y[7]);
          w1.x = e4m3x4(y[8], y[9], y[10], y[11]); w1.y = e4m3x4(y[12], y[13], y[14], y[15]);
        }
        if (!live) { w0 = make_uint2(0u, 0u); w1 = w0; }
        // rows are stored permuted inside 16-row blocks: key 4cc + jj of a block goes to row
        // 2cc + jj (jj < 2) or 8 + 2cc + jj - 2, the order in which the attention kernel's
        // 16-lane TMEM loads hand a thread four consecutive keys
        const long long o16 = nrow & 15, srow = (nrow & ~15LL) | ((o16 & 2) ? 8 + 2 * (o16 >> 2) + (o16 & 1) : 2 * (o16 >> 2) + (o16 & 1));
        uint8_t* dst = a.k8 + ((size_t)bh * N_pad + srow) * HD + 8 * c;
        *reinterpret_cast<uint2*>(dst) = w0;
        *reinterpret_cast<uint2*>(dst + 64) = w1;
        if (c == 0) a.sk[(size_t)bh * N_pad + nrow] = live ? sk : 1.0f;
      }
    } else if (which == 2) {
      // ---------------------------------- V ----------------------------------
      const long long N = VARLEN ? seq_len : a.N, N_pad = a.N_pad;
      float vmu[16];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        vmu[e] = a.vmean ? a.vmean[(size_t)bh * HD + 8 * c + e] : 0.f;
        vmu[8 + e] = a.vmean ? a.vmean[(size_t)bh * HD + 64 + 8 * c + e] : 0.f;
      }
      float svmax = 0.f;
      uint2 w0[4], w1[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = r0 + 32 * i;
        const long long nrow = n_base + t;
        const bool live = nrow < N;
        float x[16];
        unpack8<T>(*reinterpret_cast<const uint4*>(st + t * 256 + 16 * c), x);
        unpack8<T>(*reinterpret_cast<const uint4*>(st + t * 256 + 128 + 16 * c), x + 8);
        float amax = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          if (a.vmean) x[e] = live ? __fsub_rn(x[e], vmu[e]) : 0.f;
          if (VARLEN && !live) x[e] = 0.f;               // the rows behind a packed sequence are its neighbour's
          amax = fmaxf(amax, fabsf(x[e]));
        }
        amax = quarter_warp_max(amax);
        const float sv = fmaxf(div_const<448>(amax), SCALE_FLOOR);
        const float rc = __frcp_rn(sv);
        float y[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) y[e] = div_by_scale(x[e], sv, rc);
        w0[i].x = e4m3x4(y[0], y[1], y[2], y[3]); w0[i].y = e4m3x4(y[4], y[5], y[6], y[7]);
        w1[i].x = e4m3x4(y[8], y[9], y[10], y[11]); w1[i].y = e4m3x4(y[12], y[13], y[14], y[15]);
        if (c == 0) {
          a.sv[(size_t)bh * N_pad + nrow] = live ? sv : 0.0f;
          if (live) svmax = fmaxf(svmax, sv);
        }
      }
      __syncthreads();                 // every thread has read its rows: the stage becomes the code tile
      uint32_t* vt = reinterpret_cast<uint32_t*>(gbase + (size_t)stage * QT_STAGE_BYTES);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = r0 + 32 * i;
        const int key = (((t >> 4) & 7) << 2) ^ ((t & 1) << 4);
        *reinterpret_cast<uint2*>(&vt[t * 32 + ((2 * c) ^ key)]) = w0[i];
        *reinterpret_cast<uint2*>(&vt[t * 32 + ((16 + 2 * c) ^ key)]) = w1[i];
      }
      __syncthreads();
      {
        const int tg = lane & 7, dq = 4 * warp + (lane >> 3);
        uint32_t o[4][4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int tk = 16 * tg + 4 * g;
          const uint32_t w0_ = vt[(tk + 0) * 32 + (dq ^ (tg << 2))];
          const uint32_t w1_ = vt[(tk + 1) * 32 + (dq ^ (tg << 2) ^ 16)];
          const uint32_t w2_ = vt[(tk + 2) * 32 + (dq ^ (tg << 2))];
          const uint32_t w3_ = vt[(tk + 3) * 32 + (dq ^ (tg << 2) ^ 16)];
          const uint32_t t0 = __byte_perm(w0_, w1_, 0x5140), t1 = __byte_perm(w2_, w3_, 0x5140);
          const uint32_t t2 = __byte_perm(w0_, w1_, 0x7362), t3 = __byte_perm(w2_, w3_, 0x7362);
          o[0][g] = __byte_perm(t0, t1, 0x5410);
          o[1][g] = __byte_perm(t0, t1, 0x7632);
          o[2][g] = __byte_perm(t2, t3, 0x5410);
          o[3][g] = __byte_perm(t2, t3, 0x7632);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          uint8_t* dst = a.v8t + ((size_t)bh * HD + 4 * dq + e) * N_pad + n_base + 16 * tg;
          *reinterpret_cast<uint4*>(dst) = make_uint4(o[e][0], o[e][1], o[e][2], o[e][3]);
        }
      }
      // per-head max of the V scale (all scales are >= 0, so the unsigned order of the bit patterns
      // is the float order); S and SVP are folded by the closing items of the list
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) svmax = fmaxf(svmax, __shfl_xor_sync(0xffffffffu, svmax, off));
      if (lane == 0 && svmax > 0.f) atomicMax(&a.svmax_bits[bh], __float_as_uint(svmax));
    } else if (which == 3) {
      // ------------------------- fold of one head's V scales -------------------------
      // S = max(max sv, 1), SVP = fl(fl(sv / S) * 448) for FOLD_KEYS keys (the reference's
      // fold_v_scale and the attention kernel's staging).  These items close the list, long after
      // the head's V tiles were drawn; thread 0 still waits, bounded, for their arrivals.
      int done = 1;
      if (tid == 0) {
        const unsigned want = VARLEN ? (unsigned)((seq_len + TILE - 1) / TILE) : (unsigned)tiles_k;
        const volatile unsigned* arr = a.arrivals + bh;
        if (*arr != want) {
          const long long t0 = clock64();
          while (*arr != want) {
            if (clock64() - t0 > QT_WAIT_CYCLES) { done = 0; break; }
          }
        }
        __threadfence();               // acquire: the V scales of every arrived tile are visible
      }
      if (!__syncthreads_and(done)) {
        if (tid == 0) { atomicOr(a.status, 2); if (a.status2) atomicOr(a.status2, 8); }
        break;
      }
      const long long N_pad = a.N_pad;
      const long long n_fold = VARLEN ? (seq_len + TILE - 1) / TILE * TILE : N_pad;   // rows that were written
      const float S = fmaxf(__uint_as_float(__ldcg(&a.svmax_bits[bh])), 1.0f);
      if (tile == 0 && tid == 0) a.s_fold[bh] = S;
#pragma unroll
      for (int i = 0; i < FOLD_KEYS / 1024; ++i) {
        const long long nn = tile * FOLD_KEYS + (long long)i * 1024 + 4 * tid;
        if (nn < n_fold) {             // a multiple of 128: whole float4s
          const float4 v = __ldcg(reinterpret_cast<const float4*>(a.sv + (size_t)bh * N_pad + nn));
          float4 o;
          o.x = __fmul_rn(__fdiv_rn(v.x, S), F8_MAX); o.y = __fmul_rn(__fdiv_rn(v.y, S), F8_MAX);
          o.z = __fmul_rn(__fdiv_rn(v.z, S), F8_MAX); o.w = __fmul_rn(__fdiv_rn(v.w, S), F8_MAX);
          *reinterpret_cast<float4*>(a.svp + (size_t)bh * N_pad + nn) = o;
        }
      }
    }
    __syncthreads();                   // the stage may be refilled
    if (which == 2 && !beyond && tid == 0) {   // this tile's V scales and maximum are published: one release per CTA
      __threadfence();
      atomicAdd(a.arrivals + bh, 1u);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Host launcher.
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}
// 4-D map over a logical (B, H, N, D) view of 2-byte elements with (batch, head, row) element
// strides: box 128 columns x 128 rows, no swizzle, out-of-range elements read as zero.
static bool make_map4(CUtensorMap* m, const void* ptr, CUtensorMapDataType dt, int64_t D, int64_t N, int64_t H,
                      int64_t B, const int64_t strides_bhr[3]) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)strides_bhr[2] * 2, (cuuint64_t)strides_bhr[1] * 2, (cuuint64_t)strides_bhr[0] * 2};
  cuuint32_t box[4] = {128, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(m, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T>
static cudaError_t launch_typed(const PrologueParams& p, cudaStream_t st) {
  const int64_t bh = p.B * p.H;
  unsigned* words = reinterpret_cast<unsigned*>(p.ctrl);
  double* partial = reinterpret_cast<double*>(reinterpret_cast<char*>(p.ctrl) + CtrlHeader::partial_off(bh));
  // SM count and the opt-in to 64 KB of dynamic shared memory: looked up once per device
  static int sm_count[64] = {0};
  static bool opted_in[64][4] = {{false}};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (sm_count[dev] == 0) {
    e = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  e = launch_after_predecessor(clear_ctrl_kernel, dim3(1), dim3(256), 0, st, words, (int)CtrlHeader::words(bh));
  if (e != cudaSuccess) return e;
  const int nsplit = std::min(kmean_splits(bh, p.N, sm_count[dev]), kmean_splits_max(bh, p.N));
  if (p.smooth_k) {
    long long chunk = (p.N + nsplit - 1) / nsplit;
    chunk = (chunk + 15) / 16 * 16;
    dim3 grid(nsplit, (unsigned)bh);
    auto kmean = p.cu_k ? kmean_kernel<T, true> : kmean_kernel<T, false>;
    e = launch_after_predecessor(kmean, grid, dim3(256), 0, st, reinterpret_cast<const T*>(p.k), p.mean, partial, words,
                                 (long long)p.N, (long long)p.H, (long long)p.k_strides[0], (long long)p.k_strides[1],
                                 (long long)p.k_strides[2], nsplit, chunk, (int)p.D, p.cu_k, (long long)p.Tk);
    if (e != cudaSuccess) return e;
  }
  if (p.vmean) {
    long long chunk = (p.N + nsplit - 1) / nsplit;
    chunk = (chunk + 15) / 16 * 16;
    dim3 grid(nsplit, (unsigned)bh);
    auto kmean = p.cu_k ? kmean_kernel<T, true> : kmean_kernel<T, false>;
    e = launch_after_predecessor(kmean, grid, dim3(256), 0, st, reinterpret_cast<const T*>(p.v), p.vmean, partial, words + 3 * bh,
                                 (long long)p.N, (long long)p.H, (long long)p.v_strides[0], (long long)p.v_strides[1],
                                 (long long)p.v_strides[2], nsplit, chunk, (int)p.D, p.cu_k, (long long)p.Tk);
    if (e != cudaSuccess) return e;
  }
  QuantArgs a;
  a.q8 = reinterpret_cast<uint8_t*>(p.q8); a.k8 = reinterpret_cast<uint8_t*>(p.k8);
  a.v8t = reinterpret_cast<uint8_t*>(p.v8t);
  a.sq = p.sq; a.sk = p.sk; a.sv = p.sv; a.svp = p.svp; a.s_fold = p.s_fold; a.mean = p.mean; a.vmean = p.vmean;
  a.svmax_bits = words + 2 * bh; a.arrivals = words + bh;
  a.N = p.N; a.N_pad = p.N_pad; a.H = p.H;
  a.Nq = p.Nq; a.Hq = p.Hq; a.group = p.Hq / p.H; a.BHq = p.B * p.Hq; a.BHkv = bh; a.qm = p.qm;
  a.sub_mean = p.smooth_k ? 1 : 0;
  a.cu_q = p.cu_q; a.cu_k = p.cu_k; a.Tq = p.Tq; a.Tk = p.Tk;
  const bool varlen = p.cu_q != nullptr;
  const int64_t tq = (p.Nq + TILE - 1) / TILE, tk = p.N_pad / TILE;
  a.status = reinterpret_cast<int32_t*>(words + CtrlHeader::status_word(bh));
  a.status2 = p.status;
  a.next_item = reinterpret_cast<unsigned long long*>(words + CtrlHeader::status_word(bh) + 2);
  CUtensorMap mq, mk, mv;
  const CUtensorMapDataType dt = (sizeof(T) == 2 && std::is_same<T, __half>::value) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                                      : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (varlen) {
    // packed (tokens, heads, D) tensors: one batch entry that holds every token
    const int64_t qs[3] = {p.q_strides[1], p.q_strides[1], p.q_strides[2]};
    const int64_t ks[3] = {p.k_strides[1], p.k_strides[1], p.k_strides[2]};
    const int64_t vs[3] = {p.v_strides[1], p.v_strides[1], p.v_strides[2]};
    if (!make_map4(&mq, p.q, dt, p.D, p.Tq, p.Hq, 1, qs) || !make_map4(&mk, p.k, dt, p.D, p.Tk, p.H, 1, ks) ||
        !make_map4(&mv, p.v, dt, p.D, p.Tk, p.H, 1, vs))
      return cudaErrorInvalidValue;
  } else if (!make_map4(&mq, p.q, dt, p.D, p.Nq, p.Hq, p.B, p.q_strides) ||
             !make_map4(&mk, p.k, dt, p.D, p.N, p.H, p.B, p.k_strides) ||
             !make_map4(&mv, p.v, dt, p.D, p.N, p.H, p.B, p.v_strides))
    return cudaErrorInvalidValue;
  const long long total = 2 * (long long)bh * tk + (long long)a.BHq * tq;
  long long ctas = (long long)sm_count[dev] * QT_MINBLOCKS;
  if (ctas > total) ctas = total;
  auto kern = varlen ? ((p.qk_mode == 0) ? quant_qkv_kernel<T, true, true> : quant_qkv_kernel<T, false, true>)
                     : ((p.qk_mode == 0) ? quant_qkv_kernel<T, true, false> : quant_qkv_kernel<T, false, false>);
  const int which_kern = (p.qk_mode == 0 ? 1 : 0) | (varlen ? 2 : 0);
  if (!opted_in[dev][which_kern]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)QT_SMEM_BYTES);
    if (e != cudaSuccess) return e;
    opted_in[dev][which_kern] = true;
  }
  return launch_after_predecessor(kern, dim3((unsigned)ctas), dim3(256), QT_SMEM_BYTES, st, mq, mk, mv, a);
}

cudaError_t launch_prologue(const PrologueParams& p, cudaStream_t st) {
  return p.dtype == 0 ? launch_typed<__half>(p, st) : launch_typed<__nv_bfloat16>(p, st);
}

size_t prologue_ctrl_bytes(int64_t B, int64_t H, int64_t N) {
  const int64_t bh = B * H;
  return CtrlHeader::partial_off(bh) + (size_t)bh * kmean_splits_max(bh, N) * HD * sizeof(double);
}

}  // namespace sage
