// Shared device/host helpers of the B200 quantize-then-attend library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sage {

constexpr int HD = 128;        // head dim
constexpr int TILE = 128;      // query tile == key tile == prologue token tile
constexpr float I8_MAX = 127.0f;
constexpr float F8_MAX = 448.0f;
constexpr float SCALE_FLOOR = 1e-12f;
constexpr float LOG2E_F = 1.4426950408889634f;

// Control block of the prologue (device memory, zeroed by a small kernel at the start of every call).
struct CtrlHeader {
  // per head: [0] arrivals of the K mean kernel, [1] V tiles quantised so far, [2] max V scale bits, [3] arrivals
  // of the V mean kernel (smooth_v), laid out as four arrays of BH words; then one status word
  // (non-zero when a wait inside the quantiser ran out), one pad word and the quantiser's 64-bit
  // work counter; the fp64 partial sums (shared by the two mean launches, which run one after the
  // other) follow at `partial_off`.
  // (four more words follow the work counter: the attention kernel's count of skipped
  // (warp, key tile) pairs, then three spare words; all of them are cleared by the same kernel)
  static __host__ __device__ inline size_t words(int64_t bh) { return (size_t)4 * (size_t)bh + 8; }
  static __host__ __device__ inline size_t status_word(int64_t bh) { return (size_t)4 * (size_t)bh; }
  static __host__ __device__ inline size_t partial_off(int64_t bh) {
    return (words(bh) * 4 + 255) / 256 * 256;
  }
};

// Programmatic dependent launch.  A kernel launched with launch_after_predecessor() may be placed
// on the GPU while the kernel before it on the stream is still draining; it must call
// wait_for_predecessor() before it touches anything that kernel (or anything earlier on the
// stream) wrote.  allow_successor() in the earlier kernel says "my CTAs are all resident, the
// next kernel's may be scheduled as mine retire".  Without the launch attribute both calls are
// no-ops, so the kernels behave the same under a plain launch.
#ifdef __CUDACC__
__device__ __forceinline__ void wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_successor() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_after_predecessor(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

// How many CTAs share one head's sequence in the mean kernel on a device with `sms` SMs: one full
// wave of four resident CTAs per SM, at least 256 tokens per CTA, at most 64 splits.
inline int kmean_splits(int64_t bh, int64_t n, int sms) {
  int64_t want = (4 * (int64_t)sms) / bh;
  int64_t cap = (n + 255) / 256;
  if (want > cap) want = cap;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  return (int)want;
}
// The scratch for the partial sums is sized without a device at hand, for the largest SM count
// an sm_100 part has; a launch never uses more splits than that.
constexpr int KMEAN_SIZING_SMS = 160;
inline int kmean_splits_max(int64_t bh, int64_t n) { return kmean_splits(bh, n, KMEAN_SIZING_SMS); }

template <typename T> struct Elem;
template <> struct Elem<__half> {
  static __device__ __forceinline__ float2 cvt2(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float2 cvt2(uint32_t w) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  }
};

// 16 bytes = 8 elements -> 8 floats (exact widening).
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float* x) {
  float2 a = Elem<T>::cvt2(u.x), b = Elem<T>::cvt2(u.y), c = Elem<T>::cvt2(u.z), d = Elem<T>::cvt2(u.w);
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}

// Two floats -> two e4m3 bytes (a in the low byte), round to nearest even, saturating.
__device__ __forceinline__ uint32_t e4m3x2(float a, float b) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  return e4m3x2(a, b) | (e4m3x2(c, d) << 16);
}

// Round-half-even to int8 with the [-128, 127] clamp, four codes per word (a in the low byte).
__device__ __forceinline__ uint32_t i8_rne(float y) {
  int q = __float2int_rn(y);
  q = max(-128, min(127, q));
  return (uint32_t)q & 0xFFu;
}
__device__ __forceinline__ uint32_t i8x4(float a, float b, float c, float d) {
  return i8_rne(a) | (i8_rne(b) << 8) | (i8_rne(c) << 16) | (i8_rne(d) << 24);
}

}  // namespace sage
