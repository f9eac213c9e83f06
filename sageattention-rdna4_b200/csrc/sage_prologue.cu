// Quantisation prologue for B200: sequence mean of K (smooth_k), then one pass over a 128-token
// tile of Q, K and V that writes the int8 / e4m3 codes, the per-token scales, V transposed, and
// the per-head fold S with its staged factor.
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
// The fp64 mean is summed in a different (wider) order than the reference's eight strided
// partials; both are exact, hence identical, whenever the fp64 partial sums are exact, which holds
// for fp16 data when sum|K| < 2^29 per channel and for bf16 data of ordinary dynamic range.
#include "sage_common.cuh"
#include "sage_internal.h"

namespace sage {

// ------------------------------------------------------------------------------------------------
// Kernel 1: partial fp64 column sums of K; the last CTA of a head combines them in split order.
// grid (nsplit, B*H), block 256 = 16 row lanes x 16 column chunks of 8 elements.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
kmean_kernel(const T* __restrict__ K, float* __restrict__ mean, double* __restrict__ partial,
             unsigned* __restrict__ arrivals, long long N, long long H,
             long long sb, long long sh, long long sr, int nsplit, long long chunk, int D) {
  __shared__ double red[16][HD];
  __shared__ int s_last;
  const int tid = threadIdx.x, c = tid & 15, r = tid >> 4;
  const int split = blockIdx.x, bh = blockIdx.y;
  const long long b = bh / H, h = bh - b * H;
  const T* base = K + b * sb + h * sh + 8 * c;
  const long long n0 = (long long)split * chunk;
  const long long n1 = min(N, n0 + chunk);

  double acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.0;
  const long long n_end = (8 * c < D) ? n1 : n0;   // columns past head_dim: nothing to read, mean 0
#pragma unroll 8
  for (long long n = n0 + r; n < n_end; n += 16) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(base + n * sr));
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
    mean[(size_t)bh * HD + tid] = (float)(tot / (double)N);
  }
}

// ------------------------------------------------------------------------------------------------
// Kernel 2: quantise one 128-token tile of ONE of Q, K, V.  grid (N_pad/128, B*H, 3), block 256,
// four CTAs per SM.  blockIdx.z selects the tensor, so CTAs in different phases (load, convert,
// store) share an SM and keep the memory system busy.
// Thread (c = tid & 15, r0 = tid >> 4) owns columns 8c..8c+7 of rows r0, r0+16, ..., r0+112, so a
// half-warp reads one 256-byte row with 16-byte loads and the row absmax is four shuffles.
//
// Division.  K and V are divided by their scale with an IEEE-correct quotient obtained as
//   rc = rn(1/s) (correctly rounded);  q0 = rn(x*rc);  r = x - q0*s (one fma, exact);  q = fma(r, rc, q0)
// which equals rn(x/s) whenever rc is the correctly rounded reciprocal and nothing over/underflows
// (Markstein's theorem; |x/s| <= 448 and 1e-12 <= s here).  Three operations per element instead
// of a full division routine; checked against true division on 8e7 random samples on the host.
// Rounding to int8 uses the add-magic-constant trick (1.5*2^23): the addition rounds to nearest
// even, the low byte of the sum is the two's-complement code; |x/s| <= 127 needs no clamp.
// ------------------------------------------------------------------------------------------------
struct QuantArgs {
  const void *q, *k, *v;
  uint8_t *q8, *k8, *v8t;
  float *sq, *sk, *sv, *svp, *s_fold;
  const float* mean;
  const float* vmean;             // optional: sequence mean of V, subtracted before quantising (smooth_v)
  unsigned *arrivals, *svmax_bits;
  long long N, N_pad, H;          // keys: length, padded length, K/V heads per batch element
  long long Nq, Hq, group;        // queries: length, heads per batch element, Hq / H (1 without GQA)
  long long BHq, BHkv;            // B*Hq, B*H
  float* qm;                      // optional (B*Hq, Nq): dot(q row, K mean of its K/V head), for the LSE
  long long q_sb, q_sh, q_sr, k_sb, k_sh, k_sr, v_sb, v_sh, v_sr;
  int sub_mean;
  int D;                          // head_dim of the q/k/v rows; code columns D..127 are zero
};

__device__ __forceinline__ float half_warp_max(float x) {
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 8));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 4));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
  return x;
}

template <typename T>
__device__ __forceinline__ void load_rows(const T* base, long long sr, long long n_base, int r0,
                                          long long N, bool col_live, uint4* raw) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const long long n = n_base + r0 + 16 * i;
    raw[i] = (n < N && col_live) ? __ldg(reinterpret_cast<const uint4*>(base + n * sr)) : make_uint4(0, 0, 0, 0);
  }
}

// rn(x / s) given rc = rn(1/s)
__device__ __forceinline__ float div_by_scale(float x, float s, float rc) {
  const float q0 = __fmul_rn(x, rc);
  const float r = -__fmaf_rn(q0, s, -x);      // x - q0*s, written so that a zero keeps x's sign
  return __fmaf_rn(r, rc, q0);
}
// round-half-even of |y| < 2^22 to an int8 code, four per word (a in the low byte)
__device__ __forceinline__ uint32_t i8x4_magic(float a, float b, float c, float d) {
  const uint32_t ua = __float_as_uint(__fadd_rn(a, 12582912.0f)), ub = __float_as_uint(__fadd_rn(b, 12582912.0f));
  const uint32_t uc = __float_as_uint(__fadd_rn(c, 12582912.0f)), ud = __float_as_uint(__fadd_rn(d, 12582912.0f));
  return __byte_perm(__byte_perm(ua, ub, 0x0040), __byte_perm(uc, ud, 0x0040), 0x5410);
}

template <typename T, bool INT8>
__global__ void __launch_bounds__(256, 4)
quant_qkv_kernel(const QuantArgs a) {
  __shared__ __align__(16) uint32_t vt[TILE * 32];   // e4m3 V tile, [token][32 words], XOR-swizzled
  __shared__ float s_wmax[8];
  __shared__ int s_last;
  constexpr float QMAX = INT8 ? I8_MAX : F8_MAX;

  const int tid = threadIdx.x, c = tid & 15, r0 = tid >> 4, lane = tid & 31, warp = tid >> 5;
  const int bh = gridDim.y - 1 - blockIdx.y;         // last heads first: their K is still in L2 after the mean pass
  const int which = blockIdx.z == 0 ? 1 : (blockIdx.z == 1 ? 0 : 2);   // 0 Q, 1 K, 2 V; K tiles are issued first
  const long long n_base = (long long)blockIdx.x * TILE;
  uint4 raw[8];
  const bool col_live = 8 * c < a.D;

  if (which == 0) {
    // ---------------------------------- Q ----------------------------------
    const long long N = a.Nq;
    if (bh >= a.BHq || n_base >= N) return;
    const long long b = bh / a.Hq, h = bh - b * a.Hq;
    const T* qb = reinterpret_cast<const T*>(a.q) + b * a.q_sb + h * a.q_sh + 8 * c;
    load_rows<T>(qb, a.q_sr, n_base, r0, N, col_live, raw);
    float mu[8];
    if (a.qm != nullptr) {                            // the K mean of this query head's K/V head
      const long long bh_kv = b * a.H + h / a.group;
#pragma unroll
      for (int e = 0; e < 8; ++e) mu[e] = a.mean[(size_t)bh_kv * HD + 8 * c + e];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const long long n = n_base + r0 + 16 * i;
      float x[8];
      unpack8<T>(raw[i], x);
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(x[e]));
      amax = fmaxf(half_warp_max(amax), SCALE_FLOOR);
      const float qinv = __fdiv_rn(QMAX, amax);
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = __fmul_rn(x[e], qinv);
      uint2 w;
      if (INT8) {
        w.x = i8x4_magic(y[0], y[1], y[2], y[3]);
        w.y = i8x4_magic(y[4], y[5], y[6], y[7]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = fminf(fmaxf(y[e], -F8_MAX), F8_MAX);
        w.x = e4m3x4(y[0], y[1], y[2], y[3]);
        w.y = e4m3x4(y[4], y[5], y[6], y[7]);
      }
      if (n < N) {
        *reinterpret_cast<uint2*>(a.q8 + ((size_t)bh * N + n) * HD + 8 * c) = w;
        if (c == 0) a.sq[(size_t)bh * N + n] = __fdiv_rn(amax, QMAX);
      }
      if (a.qm != nullptr) {                          // fixed-order fp32 dot product of the raw row
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = __fmaf_rn(x[e], mu[e], d);
        d += __shfl_xor_sync(0xffffffffu, d, 8);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        if (c == 0 && n < N) a.qm[(size_t)bh * N + n] = d;
      }
    }
    return;
  }

  const long long N = a.N, N_pad = a.N_pad;
  if (bh >= a.BHkv || n_base >= N_pad) return;
  const long long b = bh / a.H, h = bh - b * a.H;

  if (which == 1) {
    // ---------------------------------- K ----------------------------------
    const T* kb = reinterpret_cast<const T*>(a.k) + b * a.k_sb + h * a.k_sh + 8 * c;
    load_rows<T>(kb, a.k_sr, n_base, r0, N, col_live, raw);
    float mu[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) mu[e] = a.sub_mean ? a.mean[(size_t)bh * HD + 8 * c + e] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const long long n = n_base + r0 + 16 * i;
      const bool live = n < N;
      float x[8];
      unpack8<T>(raw[i], x);
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        x[e] = (live && col_live) ? __fsub_rn(x[e], mu[e]) : 0.f;
        amax = fmaxf(amax, fabsf(x[e]));
      }
      amax = half_warp_max(amax);
      const float sk = fmaxf(__fdiv_rn(amax, QMAX), SCALE_FLOOR);
      const float rc = __frcp_rn(sk);
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = div_by_scale(x[e], sk, rc);
      uint2 w;
      if (INT8) {
        w.x = i8x4_magic(y[0], y[1], y[2], y[3]);
        w.y = i8x4_magic(y[4], y[5], y[6], y[7]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = fminf(y[e], F8_MAX);
        w.x = e4m3x4(y[0], y[1], y[2], y[3]);
        w.y = e4m3x4(y[4], y[5], y[6], y[7]);
      }
      *reinterpret_cast<uint2*>(a.k8 + ((size_t)bh * N_pad + n) * HD + 8 * c) = w;
      if (c == 0) a.sk[(size_t)bh * N_pad + n] = live ? sk : 1.0f;
    }
    return;
  }

  // ---------------------------------- V ----------------------------------
  float svmax = 0.f;
  {
    const T* vb = reinterpret_cast<const T*>(a.v) + b * a.v_sb + h * a.v_sh + 8 * c;
    load_rows<T>(vb, a.v_sr, n_base, r0, N, col_live, raw);
    float vmu[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) vmu[e] = a.vmean ? a.vmean[(size_t)bh * HD + 8 * c + e] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = r0 + 16 * i;                    // token within the tile; its 16-group is i
      const long long n = n_base + t;
      const bool live = n < N;
      float x[8];
      unpack8<T>(raw[i], x);
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (a.vmean) x[e] = (live && col_live) ? __fsub_rn(x[e], vmu[e]) : 0.f;
        amax = fmaxf(amax, fabsf(x[e]));
      }
      amax = half_warp_max(amax);
      const float sv = fmaxf(__fdiv_rn(amax, F8_MAX), SCALE_FLOOR);
      const float rc = __frcp_rn(sv);
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = fminf(div_by_scale(x[e], sv, rc), F8_MAX);
      uint2 w;
      w.x = e4m3x4(y[0], y[1], y[2], y[3]);
      w.y = e4m3x4(y[4], y[5], y[6], y[7]);
      // word column 2c (and 2c+1) of row t, XOR-swizzled by the row's 16-group so that the
      // transposed read below is bank-conflict free
      *reinterpret_cast<uint2*>(&vt[t * 32 + ((2 * c) ^ (i << 2))]) = w;
      if (c == 0) {
        a.sv[(size_t)bh * N_pad + n] = live ? sv : 0.0f;
        if (live) svmax = fmaxf(svmax, sv);
      }
    }
  }
  __syncthreads();

  // Transposed store: lane (tg = lane & 7, dqo = lane >> 3) of warp w takes the 4 channels
  // 4*(4w + dqo) .. +3 for tokens 16*tg .. 16*tg + 15, i.e. four 16-byte stores; the eight tg
  // lanes cover one 128-byte row of V8T.
  {
    const int tg = lane & 7, dq = 4 * warp + (lane >> 3);
    uint32_t o[4][4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t w0 = vt[(16 * tg + 4 * g + 0) * 32 + (dq ^ (tg << 2))];
      uint32_t w1 = vt[(16 * tg + 4 * g + 1) * 32 + (dq ^ (tg << 2))];
      uint32_t w2 = vt[(16 * tg + 4 * g + 2) * 32 + (dq ^ (tg << 2))];
      uint32_t w3 = vt[(16 * tg + 4 * g + 3) * 32 + (dq ^ (tg << 2))];
      const uint32_t t0 = __byte_perm(w0, w1, 0x5140), t1 = __byte_perm(w2, w3, 0x5140);
      const uint32_t t2 = __byte_perm(w0, w1, 0x7362), t3 = __byte_perm(w2, w3, 0x7362);
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

  // Per-head max of the V scale (all scales are >= 0, so the unsigned order of the bit patterns
  // is the float order) and the last-CTA fold: S = max(max sv, 1), SVP = fl(fl(sv/S)*448).
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) svmax = fmaxf(svmax, __shfl_xor_sync(0xffffffffu, svmax, off));
  if (lane == 0) s_wmax[warp] = svmax;
  __threadfence();                 // this thread's SV stores are visible before the arrival below
  __syncthreads();
  if (tid == 0) {
    float m = s_wmax[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, s_wmax[w]);
    atomicMax(&a.svmax_bits[bh], __float_as_uint(m));
    __threadfence();
    s_last = (atomicAdd(&a.arrivals[bh], 1u) == (unsigned)(N_pad / TILE) - 1u);
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    const float S = fmaxf(__uint_as_float(__ldcg(&a.svmax_bits[bh])), 1.0f);
    if (tid == 0) a.s_fold[bh] = S;
    for (long long n = tid; n < N_pad; n += 256) {
      const float sv = __ldcg(&a.sv[(size_t)bh * N_pad + n]);
      a.svp[(size_t)bh * N_pad + n] = __fmul_rn(__fdiv_rn(sv, S), F8_MAX);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Host launcher.
// ------------------------------------------------------------------------------------------------
template <typename T>
static cudaError_t launch_typed(const PrologueParams& p, cudaStream_t st) {
  const int64_t bh = p.B * p.H;
  unsigned* words = reinterpret_cast<unsigned*>(p.ctrl);
  double* partial = reinterpret_cast<double*>(reinterpret_cast<char*>(p.ctrl) + CtrlHeader::partial_off(bh));
  cudaError_t e = cudaMemsetAsync(p.ctrl, 0, CtrlHeader::words(bh) * 4, st);
  if (e != cudaSuccess) return e;
  if (p.smooth_k) {
    const int nsplit = kmean_splits(bh, p.N);
    long long chunk = (p.N + nsplit - 1) / nsplit;
    chunk = (chunk + 15) / 16 * 16;
    dim3 grid(nsplit, (unsigned)bh);
    kmean_kernel<T><<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(p.k), p.mean, partial, words,
                                          p.N, p.H, p.k_strides[0], p.k_strides[1], p.k_strides[2],
                                          nsplit, chunk, (int)p.D);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  if (p.vmean) {
    const int nsplit = kmean_splits(bh, p.N);
    long long chunk = (p.N + nsplit - 1) / nsplit;
    chunk = (chunk + 15) / 16 * 16;
    dim3 grid(nsplit, (unsigned)bh);
    kmean_kernel<T><<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(p.v), p.vmean, partial, words + 3 * bh,
                                          p.N, p.H, p.v_strides[0], p.v_strides[1], p.v_strides[2],
                                          nsplit, chunk, (int)p.D);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  QuantArgs a;
  a.q = p.q; a.k = p.k; a.v = p.v;
  a.q8 = reinterpret_cast<uint8_t*>(p.q8); a.k8 = reinterpret_cast<uint8_t*>(p.k8);
  a.v8t = reinterpret_cast<uint8_t*>(p.v8t);
  a.sq = p.sq; a.sk = p.sk; a.sv = p.sv; a.svp = p.svp; a.s_fold = p.s_fold; a.mean = p.mean; a.vmean = p.vmean;
  a.arrivals = words + bh; a.svmax_bits = words + 2 * bh;
  a.N = p.N; a.N_pad = p.N_pad; a.H = p.H;
  a.Nq = p.Nq; a.Hq = p.Hq; a.group = p.Hq / p.H; a.BHq = p.B * p.Hq; a.BHkv = bh; a.qm = p.qm;
  a.q_sb = p.q_strides[0]; a.q_sh = p.q_strides[1]; a.q_sr = p.q_strides[2];
  a.k_sb = p.k_strides[0]; a.k_sh = p.k_strides[1]; a.k_sr = p.k_strides[2];
  a.v_sb = p.v_strides[0]; a.v_sh = p.v_strides[1]; a.v_sr = p.v_strides[2];
  a.sub_mean = p.smooth_k ? 1 : 0;
  a.D = (int)p.D;
  const int64_t tq = (p.Nq + TILE - 1) / TILE, tk = p.N_pad / TILE;
  dim3 grid((unsigned)(tq > tk ? tq : tk), (unsigned)(a.BHq > bh ? a.BHq : bh), 3);
  if (p.qk_mode == 0) quant_qkv_kernel<T, true><<<grid, 256, 0, st>>>(a);
  else quant_qkv_kernel<T, false><<<grid, 256, 0, st>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_prologue(const PrologueParams& p, cudaStream_t st) {
  return p.dtype == 0 ? launch_typed<__half>(p, st) : launch_typed<__nv_bfloat16>(p, st);
}

size_t prologue_ctrl_bytes(int64_t B, int64_t H, int64_t N) {
  const int64_t bh = B * H;
  return CtrlHeader::partial_off(bh) + (size_t)bh * kmean_splits(bh, N) * HD * sizeof(double);
}

}  // namespace sage
