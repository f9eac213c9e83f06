// extern "C" boundary of libsage_b200.so (declared in include/sage_b200.h): argument checks,
// workspace carving and the two launches.  Nothing here allocates or synchronises.
#include <stdarg.h>

#include <mutex>
#include <stdio.h>
#include <string.h>

#include "../../include/sage_b200.h"
#include "sage_common.cuh"
#include "sage_internal.h"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// ---- built-in control scratch for sage_prologue_static_ctrl ------------------------------------
// Some hosts may not call an allocator at all at the point where they run the prologue: a plugin
// whose enqueue step is handed a fixed set of buffers, a serving process pinned under a memory
// cap, code on a path where cudaMalloc's implicit device synchronisation is unacceptable.  For
// them the prologue's scratch (per-head arrival counters, the running maximum of the V scale and
// the fp64 partial sums of the mean) lives in this file-scope device array instead of in
// caller-owned memory.  Every GPU that loads the library carries the array until the process
// exits.  In host code the array's name is only a handle: the device address is obtained once per
// device with cudaGetSymbolAddress and that pointer is what the kernels receive.
constexpr size_t kStaticCtrlBytes = (size_t)1 << 20;                  // 1 MiB
static __device__ __align__(256) unsigned char g_static_ctrl[kStaticCtrlBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_ctrl_mutex;
void* g_static_ctrl_ptr[kMaxDevices] = {nullptr};

// Device address of the built-in block on the CURRENT device (looked up on first use there).
int static_ctrl_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(SAGE_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(SAGE_E_UNSUPPORTED, "device ordinal %d is out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_ctrl_mutex);
  if (g_static_ctrl_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_ctrl);
    if (e != cudaSuccess || p == nullptr)
      return fail(SAGE_E_CUDA, "cudaGetSymbolAddress(built-in control scratch): %s", cudaGetErrorString(e));
    g_static_ctrl_ptr[dev] = p;
  }
  *out = g_static_ctrl_ptr[dev];
  return SAGE_OK;
}

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_strides(const char* name, const int64_t s[3]) {
  if (!s) return fail(SAGE_E_ARG, "%s strides are null", name);
  for (int i = 0; i < 3; ++i) {
    if (s[i] <= 0) return fail(SAGE_E_ARG, "%s stride %d is not positive", name, i);
    if (s[i] % 8) return fail(SAGE_E_ARG, "%s stride %d is not a multiple of 8 elements", name, i);
  }
  return SAGE_OK;
}

int check_dims(int64_t B, int64_t H, int64_t N) {
  if (B < 1 || H < 1 || N < 1) return fail(SAGE_E_ARG, "B, H and N must be >= 1 (got %lld, %lld, %lld)",
                                            (long long)B, (long long)H, (long long)N);
  if (B * H > 65535) return fail(SAGE_E_UNSUPPORTED, "B*H = %lld exceeds the grid limit 65535", (long long)(B * H));
  if (N > (int64_t)1 << 30) return fail(SAGE_E_UNSUPPORTED, "N = %lld exceeds 2^30", (long long)N);
  return SAGE_OK;
}

struct Layout {
  size_t q8, sq, k8, sk, v8t, sv, svp, s_fold, mean, ctrl, status, total;
};

Layout carve(int64_t B, int64_t H, int64_t N) {
  const size_t bh = (size_t)(B * H), n = (size_t)N, np = (size_t)sage_pad_len(N);
  Layout L;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align256(off + bytes); return o; };
  L.q8 = take(bh * n * sage::HD);
  L.sq = take(bh * n * 4);
  L.k8 = take(bh * np * sage::HD);
  L.sk = take(bh * np * 4);
  L.v8t = take(bh * np * sage::HD);
  L.sv = take(bh * np * 4);
  L.svp = take(bh * np * 4);
  L.s_fold = take(bh * 4);
  L.mean = take(bh * sage::HD * 4);
  L.ctrl = take(sage::prologue_ctrl_bytes(B, H, N));
  L.status = take(256);
  L.total = off;
  return L;
}

}  // namespace

extern "C" {

int sage_version(void) { return 100; }

const char* sage_last_error(void) { return g_err; }

int64_t sage_pad_len(int64_t n) { return (n + SAGE_TILE - 1) / SAGE_TILE * SAGE_TILE; }

size_t sage_prologue_ctrl_bytes(int64_t B, int64_t H, int64_t N) {
  if (B < 1 || H < 1 || N < 1) return 0;
  return sage::prologue_ctrl_bytes(B, H, N);
}

int sage_prologue(const void* q, const void* k, const void* v,
                  void* q8, float* sq, void* k8, float* sk, void* v8t, float* sv, float* svp,
                  float* s_fold, float* mean, void* ctrl,
                  int64_t B, int64_t H, int64_t N, int64_t N_pad,
                  const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                  int dtype, int qk_mode, int smooth_k, void* stream) {
  g_err[0] = 0;
  int rc = check_dims(B, H, N);
  if (rc) return rc;
  if (!q || !k || !v || !q8 || !sq || !k8 || !sk || !v8t || !sv || !svp || !s_fold || !ctrl)
    return fail(SAGE_E_ARG, "sage_prologue: null pointer argument");
  if (smooth_k && !mean) return fail(SAGE_E_ARG, "sage_prologue: smooth_k needs a mean buffer");
  if (N_pad != sage_pad_len(N)) return fail(SAGE_E_ARG, "sage_prologue: N_pad must be %lld", (long long)sage_pad_len(N));
  if (dtype != SAGE_F16 && dtype != SAGE_BF16) return fail(SAGE_E_ARG, "sage_prologue: dtype must be SAGE_F16 or SAGE_BF16");
  if (qk_mode != SAGE_QK_INT8 && qk_mode != SAGE_QK_E4M3) return fail(SAGE_E_ARG, "sage_prologue: bad qk_mode");
  if ((rc = check_strides("q", q_strides)) || (rc = check_strides("k", k_strides)) || (rc = check_strides("v", v_strides)))
    return rc;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(q8) || !aligned16(k8) || !aligned16(v8t) ||
      !aligned16(sk) || !aligned16(svp) || !aligned16(ctrl))
    return fail(SAGE_E_ARG, "sage_prologue: pointers must be 16-byte aligned");
  sage::PrologueParams p;
  p.q = q; p.k = k; p.v = v; p.q8 = q8; p.k8 = k8; p.v8t = v8t;
  p.sq = sq; p.sk = sk; p.sv = sv; p.svp = svp; p.s_fold = s_fold; p.mean = mean; p.ctrl = ctrl;
  p.B = B; p.H = H; p.N = N; p.N_pad = N_pad;
  for (int i = 0; i < 3; ++i) { p.q_strides[i] = q_strides[i]; p.k_strides[i] = k_strides[i]; p.v_strides[i] = v_strides[i]; }
  p.dtype = dtype; p.qk_mode = qk_mode; p.smooth_k = smooth_k;
  cudaError_t e = sage::launch_prologue(p, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(SAGE_E_CUDA, "sage_prologue: %s", cudaGetErrorString(e));
  return SAGE_OK;
}

size_t sage_prologue_static_ctrl_capacity(void) { return kStaticCtrlBytes; }

int sage_prologue_static_ctrl(const void* q, const void* k, const void* v,
                              void* q8, float* sq, void* k8, float* sk, void* v8t, float* sv,
                              float* svp, float* s_fold, float* mean,
                              int64_t B, int64_t H, int64_t N, int64_t N_pad,
                              const int64_t q_strides[3], const int64_t k_strides[3],
                              const int64_t v_strides[3],
                              int dtype, int qk_mode, int smooth_k, void* stream) {
  g_err[0] = 0;
  int rc = check_dims(B, H, N);
  if (rc) return rc;
  const size_t need = sage::prologue_ctrl_bytes(B, H, N);
  if (need > kStaticCtrlBytes)
    return fail(SAGE_E_UNSUPPORTED,
                "sage_prologue_static_ctrl: this shape needs %zu bytes of control scratch, the built-in block "
                "holds %zu; use sage_prologue with caller-owned scratch", need, (size_t)kStaticCtrlBytes);
  void* ctrl = nullptr;
  rc = static_ctrl_address(&ctrl);
  if (rc) return rc;
  return sage_prologue(q, k, v, q8, sq, k8, sk, v8t, sv, svp, s_fold, mean, ctrl, B, H, N, N_pad,
                       q_strides, k_strides, v_strides, dtype, qk_mode, smooth_k, stream);
}

int sage_attn_fwd(const void* q8, const float* sq, const void* k8, const float* sk,
                  const void* v8t, const float* svp, const float* s_fold, void* out,
                  int64_t B, int64_t H, int64_t N, int64_t N_pad, const int64_t o_strides[3],
                  int causal, float sm_scale, int out_dtype, int qk_mode,
                  int32_t* status, void* stream) {
  g_err[0] = 0;
  int rc = check_dims(B, H, N);
  if (rc) return rc;
  if (!q8 || !sq || !k8 || !sk || !v8t || !svp || !s_fold || !out || !status)
    return fail(SAGE_E_ARG, "sage_attn_fwd: null pointer argument");
  if (N_pad != sage_pad_len(N)) return fail(SAGE_E_ARG, "sage_attn_fwd: N_pad must be %lld", (long long)sage_pad_len(N));
  if (out_dtype != SAGE_F16 && out_dtype != SAGE_BF16) return fail(SAGE_E_ARG, "sage_attn_fwd: bad out_dtype");
  if (qk_mode != SAGE_QK_INT8 && qk_mode != SAGE_QK_E4M3) return fail(SAGE_E_ARG, "sage_attn_fwd: bad qk_mode");
  if ((rc = check_strides("out", o_strides))) return rc;
  if (!aligned16(q8) || !aligned16(k8) || !aligned16(v8t) || !aligned16(sk) || !aligned16(svp) || !aligned16(out))
    return fail(SAGE_E_ARG, "sage_attn_fwd: pointers must be 16-byte aligned");
  if (!(sm_scale == sm_scale)) return fail(SAGE_E_ARG, "sage_attn_fwd: sm_scale is NaN");
  sage::AttnParams p;
  p.q8 = q8; p.k8 = k8; p.v8t = v8t; p.sq = sq; p.sk = sk; p.svp = svp; p.s_fold = s_fold; p.out = out;
  p.B = B; p.H = H; p.N = N; p.N_pad = N_pad;
  for (int i = 0; i < 3; ++i) p.o_strides[i] = o_strides[i];
  p.causal = causal ? 1 : 0; p.sm_scale = sm_scale; p.out_dtype = out_dtype; p.qk_mode = qk_mode;
  p.status = status;
  const char* why = nullptr;
  cudaError_t e = sage::launch_attention(p, reinterpret_cast<cudaStream_t>(stream), &why);
  if (e != cudaSuccess) return fail(SAGE_E_CUDA, "sage_attn_fwd: %s (%s)", why ? why : "", cudaGetErrorString(e));
  return SAGE_OK;
}

void sage_debug_score_dump(void* ptr, int key_tile) { sage::set_score_dump(ptr, key_tile); }

size_t sage_workspace_bytes(int64_t B, int64_t H, int64_t N) {
  if (B < 1 || H < 1 || N < 1) return 0;
  return carve(B, H, N).total;
}

int sage_workspace_layout(int64_t B, int64_t H, int64_t N, size_t offsets[11]) {
  if (B < 1 || H < 1 || N < 1 || !offsets) return fail(SAGE_E_ARG, "sage_workspace_layout: bad argument");
  const Layout L = carve(B, H, N);
  const size_t o[11] = {L.q8, L.sq, L.k8, L.sk, L.v8t, L.sv, L.svp, L.s_fold, L.mean, L.ctrl, L.status};
  memcpy(offsets, o, sizeof(o));
  return 11;
}

int sage_attention(const void* q, const void* k, const void* v, void* out,
                   void* workspace, size_t workspace_bytes,
                   int64_t B, int64_t H, int64_t N,
                   const int64_t q_strides[3], const int64_t k_strides[3],
                   const int64_t v_strides[3], const int64_t o_strides[3],
                   int dtype, int qk_mode, int causal, int smooth_k, float sm_scale, void* stream) {
  g_err[0] = 0;
  int rc = check_dims(B, H, N);
  if (rc) return rc;
  if (!workspace) return fail(SAGE_E_ARG, "sage_attention: workspace is null");
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(SAGE_E_ARG, "sage_attention: workspace must be 256-byte aligned");
  const Layout L = carve(B, H, N);
  if (workspace_bytes < L.total)
    return fail(SAGE_E_WORKSPACE, "sage_attention: workspace has %zu bytes, needs %zu", workspace_bytes, L.total);
  if (qk_mode < 0) qk_mode = (dtype == SAGE_BF16) ? SAGE_QK_E4M3 : SAGE_QK_INT8;
  char* w = reinterpret_cast<char*>(workspace);
  const int64_t N_pad = sage_pad_len(N);
  int32_t* status = reinterpret_cast<int32_t*>(w + L.status);
  cudaError_t e = cudaMemsetAsync(status, 0, 4, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(SAGE_E_CUDA, "sage_attention: %s", cudaGetErrorString(e));
  rc = sage_prologue(q, k, v, w + L.q8, reinterpret_cast<float*>(w + L.sq), w + L.k8,
                     reinterpret_cast<float*>(w + L.sk), w + L.v8t, reinterpret_cast<float*>(w + L.sv),
                     reinterpret_cast<float*>(w + L.svp), reinterpret_cast<float*>(w + L.s_fold),
                     reinterpret_cast<float*>(w + L.mean), w + L.ctrl, B, H, N, N_pad,
                     q_strides, k_strides, v_strides, dtype, qk_mode, smooth_k, stream);
  if (rc) return rc;
  return sage_attn_fwd(w + L.q8, reinterpret_cast<float*>(w + L.sq), w + L.k8,
                       reinterpret_cast<float*>(w + L.sk), w + L.v8t, reinterpret_cast<float*>(w + L.svp),
                       reinterpret_cast<float*>(w + L.s_fold), out, B, H, N, N_pad, o_strides,
                       causal, sm_scale, dtype, qk_mode, status, stream);
}

}  // extern "C"
