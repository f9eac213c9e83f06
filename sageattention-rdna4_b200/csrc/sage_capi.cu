// extern "C" boundary of libsage_b200.so (declared in include/sage_b200.h): argument checks,
// workspace carving and the launches.  Nothing here allocates or synchronises.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

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
    if (s[i] >= ((int64_t)1 << 39)) return fail(SAGE_E_UNSUPPORTED, "%s stride %d exceeds 2^39 elements", name, i);
  }
  return SAGE_OK;
}

// Shape of one call: B batches; Hq query heads sharing Hkv key/value heads (Hq a multiple of Hkv);
// Nq query rows; Nk keys; D elements per q/k/v/out row (the quantised codes are always 128 wide).
struct Dims {
  int64_t B, Hq, Hkv, Nq, Nk, D;
};

int check_dims(const Dims& d) {
  if (d.B < 1 || d.Hq < 1 || d.Hkv < 1 || d.Nq < 1 || d.Nk < 1)
    return fail(SAGE_E_ARG, "B, heads and lengths must be >= 1 (got B=%lld Hq=%lld Hkv=%lld Nq=%lld Nk=%lld)",
                (long long)d.B, (long long)d.Hq, (long long)d.Hkv, (long long)d.Nq, (long long)d.Nk);
  if (d.D < 8 || d.D > sage::HD || d.D % 8)
    return fail(SAGE_E_UNSUPPORTED, "head_dim must be a multiple of 8 in 8..128 (got %lld)", (long long)d.D);
  if (d.Hq % d.Hkv) return fail(SAGE_E_ARG, "query heads (%lld) must be a multiple of key/value heads (%lld)",
                                (long long)d.Hq, (long long)d.Hkv);
  if (d.B * d.Hq > 65535) return fail(SAGE_E_UNSUPPORTED, "B*H = %lld exceeds the grid limit 65535", (long long)(d.B * d.Hq));
  if (d.Nq > (int64_t)1 << 30 || d.Nk > (int64_t)1 << 30) return fail(SAGE_E_UNSUPPORTED, "sequence length exceeds 2^30");
  return SAGE_OK;
}

// A packed variable-length batch: device arrays of B + 1 cumulative token counts and the token
// counts of the packed tensors (null / 0 for a fixed-length call).
struct Packed {
  const int32_t *cu_q, *cu_k;
  int64_t Tq, Tk;
};
constexpr Packed kNotPacked = {nullptr, nullptr, 0, 0};

struct Layout {
  size_t q8, sq, k8, sk, v8t, sv, svp, s_fold, mean, ctrl, status, qm, vmean, total;
};

Layout carve(const Dims& d) {
  const size_t bhq = (size_t)(d.B * d.Hq), bhk = (size_t)(d.B * d.Hkv);
  const size_t nq = (size_t)d.Nq, np = (size_t)sage_pad_len(d.Nk);
  Layout L;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align256(off + bytes); return o; };
  L.q8 = take(bhq * nq * sage::HD);
  L.sq = take(bhq * nq * 4);
  L.k8 = take(bhk * np * sage::HD);
  L.sk = take(bhk * np * 4);
  L.v8t = take(bhk * np * sage::HD);
  L.sv = take(bhk * np * 4);
  L.svp = take(bhk * np * 4);
  L.s_fold = take(bhk * 4);
  L.mean = take(bhk * sage::HD * 4);
  L.ctrl = take(sage::prologue_ctrl_bytes(d.B, d.Hkv, d.Nk));
  // the attention kernel's status word is the spare word of the control header, so that the
  // prologue's clearing kernel clears it too
  L.status = L.ctrl + 4 * (sage::CtrlHeader::status_word((int64_t)bhk) + 1);
  L.qm = take(bhq * nq * 4);
  L.vmean = take(bhk * sage::HD * 4);
  L.total = off;
  return L;
}

int prologue_impl(const void* q, const void* k, const void* v,
                  void* q8, float* sq, void* k8, float* sk, void* v8t, float* sv, float* svp,
                  float* s_fold, float* mean, float* qm, float* vmean, void* ctrl, const Dims& d, int64_t Nk_pad,
                  const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                  int dtype, int qk_mode, int smooth_k, void* stream, const char* who,
                  int32_t* status = nullptr, const Packed& pk = kNotPacked) {
  g_err[0] = 0;
  int rc = check_dims(d);
  if (rc) return rc;
  if (!q || !k || !v || !q8 || !sq || !k8 || !sk || !v8t || !sv || !svp || !s_fold || !ctrl)
    return fail(SAGE_E_ARG, "%s: null pointer argument", who);
  if (smooth_k && !mean) return fail(SAGE_E_ARG, "%s: smooth_k needs a mean buffer", who);
  if (qm && !smooth_k) return fail(SAGE_E_ARG, "%s: the q.mean output only exists with smooth_k", who);
  if (Nk_pad != sage_pad_len(d.Nk)) return fail(SAGE_E_ARG, "%s: padded key length must be %lld", who, (long long)sage_pad_len(d.Nk));
  if (dtype != SAGE_F16 && dtype != SAGE_BF16) return fail(SAGE_E_ARG, "%s: dtype must be SAGE_F16 or SAGE_BF16", who);
  if (qk_mode != SAGE_QK_INT8 && qk_mode != SAGE_QK_E4M3) return fail(SAGE_E_ARG, "%s: bad qk_mode", who);
  if ((rc = check_strides("q", q_strides)) || (rc = check_strides("k", k_strides)) || (rc = check_strides("v", v_strides)))
    return rc;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(q8) || !aligned16(k8) || !aligned16(v8t) ||
      !aligned16(sk) || !aligned16(sv) || !aligned16(svp) || !aligned16(ctrl) || !aligned16(vmean))
    return fail(SAGE_E_ARG, "%s: pointers must be 16-byte aligned", who);
  if (status && (reinterpret_cast<uintptr_t>(status) & 3u)) return fail(SAGE_E_ARG, "%s: status must be 4-byte aligned", who);
  sage::PrologueParams p;
  p.q = q; p.k = k; p.v = v; p.q8 = q8; p.k8 = k8; p.v8t = v8t;
  p.sq = sq; p.sk = sk; p.sv = sv; p.svp = svp; p.s_fold = s_fold; p.mean = mean; p.ctrl = ctrl; p.qm = qm; p.vmean = vmean; p.status = status;
  p.B = d.B; p.H = d.Hkv; p.N = d.Nk; p.N_pad = Nk_pad; p.Hq = d.Hq; p.Nq = d.Nq; p.D = d.D;
  for (int i = 0; i < 3; ++i) { p.q_strides[i] = q_strides[i]; p.k_strides[i] = k_strides[i]; p.v_strides[i] = v_strides[i]; }
  p.dtype = dtype; p.qk_mode = qk_mode; p.smooth_k = smooth_k;
  p.cu_q = pk.cu_q; p.cu_k = pk.cu_k; p.Tq = pk.Tq; p.Tk = pk.Tk;
  cudaError_t e = sage::launch_prologue(p, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(SAGE_E_CUDA, "%s: %s", who, cudaGetErrorString(e));
  return SAGE_OK;
}

int attn_impl(const void* q8, const float* sq, const void* k8, const float* sk,
              const void* v8t, const float* svp, const float* s_fold, void* out, float* lse, const float* qm,
              const float* vmean, const Dims& d, int64_t Nk_pad, const int64_t o_strides[3],
              int causal, float sm_scale, int out_dtype, int qk_mode, int32_t* status, void* stream,
              const char* who, unsigned* skipped = nullptr, const Packed& pk = kNotPacked) {
  g_err[0] = 0;
  int rc = check_dims(d);
  if (rc) return rc;
  const int no_fast_path = (qk_mode & SAGE_QK_NO_FAST_PATH) ? 1 : 0;
  qk_mode &= ~SAGE_QK_NO_FAST_PATH;
  if (!q8 || !sq || !k8 || !sk || !v8t || !svp || !s_fold || !out || !status)
    return fail(SAGE_E_ARG, "%s: null pointer argument", who);
  if (Nk_pad != sage_pad_len(d.Nk)) return fail(SAGE_E_ARG, "%s: padded key length must be %lld", who, (long long)sage_pad_len(d.Nk));
  if (causal && d.Nq != d.Nk) return fail(SAGE_E_ARG, "%s: a causal call needs as many queries as keys", who);
  if (out_dtype != SAGE_F16 && out_dtype != SAGE_BF16) return fail(SAGE_E_ARG, "%s: bad out_dtype", who);
  if (qk_mode != SAGE_QK_INT8 && qk_mode != SAGE_QK_E4M3) return fail(SAGE_E_ARG, "%s: bad qk_mode", who);
  if ((rc = check_strides("out", o_strides))) return rc;
  if (!aligned16(q8) || !aligned16(k8) || !aligned16(v8t) || !aligned16(sk) || !aligned16(svp) || !aligned16(out) ||
      !aligned16(vmean))
    return fail(SAGE_E_ARG, "%s: pointers must be 16-byte aligned", who);
  // The kernel takes the row maximum before it multiplies by sm_scale * log2(e) * sq, which keeps
  // the order only for a positive factor.
  if (!(sm_scale > 0.f) || !(sm_scale <= 3.0e38f))
    return fail(SAGE_E_ARG, "%s: sm_scale must be finite and positive (got %g)", who, (double)sm_scale);
  sage::AttnParams p;
  p.q8 = q8; p.k8 = k8; p.v8t = v8t; p.sq = sq; p.sk = sk; p.svp = svp; p.s_fold = s_fold; p.out = out;
  p.lse = lse; p.qm = qm; p.vmean = vmean;
  p.B = d.B; p.H = d.Hkv; p.N = d.Nk; p.N_pad = Nk_pad; p.Hq = d.Hq; p.Nq = d.Nq; p.D = d.D;
  for (int i = 0; i < 3; ++i) p.o_strides[i] = o_strides[i];
  p.causal = causal ? 1 : 0; p.sm_scale = sm_scale; p.out_dtype = out_dtype; p.qk_mode = qk_mode;
  p.status = status;
  p.no_fast_path = no_fast_path; p.skipped = skipped;
  p.cu_q = pk.cu_q; p.cu_k = pk.cu_k; p.Tq = pk.Tq; p.Tk = pk.Tk;
  const char* why = nullptr;
  cudaError_t e = sage::launch_attention(p, reinterpret_cast<cudaStream_t>(stream), &why);
  if (e != cudaSuccess) return fail(SAGE_E_CUDA, "%s: %s (%s)", who, why ? why : "", cudaGetErrorString(e));
  return SAGE_OK;
}

int attention_impl(const void* q, const void* k, const void* v, void* out, float* lse,
                   void* workspace, size_t workspace_bytes, const Dims& d,
                   const int64_t q_strides[3], const int64_t k_strides[3],
                   const int64_t v_strides[3], const int64_t o_strides[3],
                   int dtype, int qk_mode, int causal, int smooth_k, int smooth_v, float sm_scale, void* stream,
                   const char* who, const Packed& pk = kNotPacked) {
  g_err[0] = 0;
  int rc = check_dims(d);
  if (rc) return rc;
  if (!workspace) return fail(SAGE_E_ARG, "%s: workspace is null", who);
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(SAGE_E_ARG, "%s: workspace must be 256-byte aligned", who);
  const Layout L = carve(d);
  if (workspace_bytes < L.total)
    return fail(SAGE_E_WORKSPACE, "%s: workspace has %zu bytes, needs %zu", who, workspace_bytes, L.total);
  // what the attention step would refuse is refused before the prologue is launched
  if (!out) return fail(SAGE_E_ARG, "%s: null pointer argument", who);
  if (causal && d.Nq != d.Nk) return fail(SAGE_E_ARG, "%s: a causal call needs as many queries as keys", who);
  if ((rc = check_strides("out", o_strides))) return rc;
  if (!aligned16(out)) return fail(SAGE_E_ARG, "%s: pointers must be 16-byte aligned", who);
  if (!(sm_scale > 0.f) || !(sm_scale <= 3.0e38f))
    return fail(SAGE_E_ARG, "%s: sm_scale must be finite and positive (got %g)", who, (double)sm_scale);
  const int flags = (qk_mode >= 0) ? (qk_mode & SAGE_QK_NO_FAST_PATH) : (((-qk_mode) & SAGE_QK_NO_FAST_PATH));
  if (qk_mode < 0) qk_mode = (dtype == SAGE_BF16) ? SAGE_QK_E4M3 : SAGE_QK_INT8;
  else qk_mode &= ~SAGE_QK_NO_FAST_PATH;
  char* w = reinterpret_cast<char*>(workspace);
  const int64_t Nk_pad = sage_pad_len(d.Nk);
  int32_t* status = reinterpret_cast<int32_t*>(w + L.status);     // zeroed by the prologue's clearing kernel
  float* qm = (lse && smooth_k) ? reinterpret_cast<float*>(w + L.qm) : nullptr;
  float* vmean = smooth_v ? reinterpret_cast<float*>(w + L.vmean) : nullptr;
  rc = prologue_impl(q, k, v, w + L.q8, reinterpret_cast<float*>(w + L.sq), w + L.k8,
                     reinterpret_cast<float*>(w + L.sk), w + L.v8t, reinterpret_cast<float*>(w + L.sv),
                     reinterpret_cast<float*>(w + L.svp), reinterpret_cast<float*>(w + L.s_fold),
                     reinterpret_cast<float*>(w + L.mean), qm, vmean, w + L.ctrl, d, Nk_pad,
                     q_strides, k_strides, v_strides, dtype, qk_mode, smooth_k, stream, who, status, pk);
  if (rc) return rc;
  return attn_impl(w + L.q8, reinterpret_cast<float*>(w + L.sq), w + L.k8,
                   reinterpret_cast<float*>(w + L.sk), w + L.v8t, reinterpret_cast<float*>(w + L.svp),
                   reinterpret_cast<float*>(w + L.s_fold), out, lse, qm, vmean, d, Nk_pad, o_strides,
                   causal, sm_scale, dtype, qk_mode | flags, status, stream, who,
                   reinterpret_cast<unsigned*>(status) + 3, pk);
}

}  // namespace

extern "C" {

int sage_version(void) { return 200; }

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
  const Dims d = {B, H, H, N, N, sage::HD};
  return prologue_impl(q, k, v, q8, sq, k8, sk, v8t, sv, svp, s_fold, mean, nullptr, nullptr, ctrl, d, N_pad,
                       q_strides, k_strides, v_strides, dtype, qk_mode, smooth_k, stream, "sage_prologue");
}

int sage_prologue_ex(const void* q, const void* k, const void* v,
                     void* q8, float* sq, void* k8, float* sk, void* v8t, float* sv, float* svp,
                     float* s_fold, float* mean, float* qm, float* vmean, void* ctrl,
                     int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk, int64_t Nk_pad, int64_t head_dim,
                     const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                     int dtype, int qk_mode, int smooth_k, void* stream) {
  const Dims d = {B, Hq, Hkv, Nq, Nk, head_dim};
  return prologue_impl(q, k, v, q8, sq, k8, sk, v8t, sv, svp, s_fold, mean, qm, vmean, ctrl, d, Nk_pad,
                       q_strides, k_strides, v_strides, dtype, qk_mode, smooth_k, stream, "sage_prologue_ex");
}

size_t sage_prologue_static_ctrl_capacity(void) { return kStaticCtrlBytes; }

int sage_prologue_static_ctrl(const void* q, const void* k, const void* v,
                              void* q8, float* sq, void* k8, float* sk, void* v8t, float* sv,
                              float* svp, float* s_fold, float* mean,
                              int64_t B, int64_t H, int64_t N, int64_t N_pad,
                              const int64_t q_strides[3], const int64_t k_strides[3],
                              const int64_t v_strides[3],
                              int dtype, int qk_mode, int smooth_k, int32_t* status, void* stream) {
  g_err[0] = 0;
  const Dims d = {B, H, H, N, N, sage::HD};
  int rc = check_dims(d);
  if (rc) return rc;
  const size_t need = sage::prologue_ctrl_bytes(B, H, N);
  if (need > kStaticCtrlBytes)
    return fail(SAGE_E_UNSUPPORTED,
                "sage_prologue_static_ctrl: this shape needs %zu bytes of control scratch, the built-in block "
                "holds %zu; use sage_prologue with caller-owned scratch", need, (size_t)kStaticCtrlBytes);
  void* ctrl = nullptr;
  rc = static_ctrl_address(&ctrl);
  if (rc) return rc;
  return prologue_impl(q, k, v, q8, sq, k8, sk, v8t, sv, svp, s_fold, mean, nullptr, nullptr, ctrl, d, N_pad,
                       q_strides, k_strides, v_strides, dtype, qk_mode, smooth_k, stream,
                       "sage_prologue_static_ctrl", status);
}

int sage_attn_fwd(const void* q8, const float* sq, const void* k8, const float* sk,
                  const void* v8t, const float* svp, const float* s_fold, void* out,
                  int64_t B, int64_t H, int64_t N, int64_t N_pad, const int64_t o_strides[3],
                  int causal, float sm_scale, int out_dtype, int qk_mode,
                  int32_t* status, void* stream) {
  const Dims d = {B, H, H, N, N, sage::HD};
  return attn_impl(q8, sq, k8, sk, v8t, svp, s_fold, out, nullptr, nullptr, nullptr, d, N_pad, o_strides,
                   causal, sm_scale, out_dtype, qk_mode, status, stream, "sage_attn_fwd");
}

int sage_attn_fwd_ex(const void* q8, const float* sq, const void* k8, const float* sk,
                     const void* v8t, const float* svp, const float* s_fold, void* out,
                     float* lse, const float* qm, const float* vmean,
                     int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk, int64_t Nk_pad, int64_t head_dim,
                     const int64_t o_strides[3], int causal, float sm_scale, int out_dtype, int qk_mode,
                     int32_t* status, void* stream) {
  const Dims d = {B, Hq, Hkv, Nq, Nk, head_dim};
  return attn_impl(q8, sq, k8, sk, v8t, svp, s_fold, out, lse, qm, vmean, d, Nk_pad, o_strides,
                   causal, sm_scale, out_dtype, qk_mode, status, stream, "sage_attn_fwd_ex");
}

int sage_status_mirror(const int32_t* status_dev, int32_t* status_host, int words, void* stream) {
  g_err[0] = 0;
  if (!status_dev || !status_host) return fail(SAGE_E_ARG, "sage_status_mirror: null pointer argument");
  if (words < 1 || words > 4) return fail(SAGE_E_ARG, "sage_status_mirror: words must be 1..4");
  if ((reinterpret_cast<uintptr_t>(status_dev) | reinterpret_cast<uintptr_t>(status_host)) & 3u)
    return fail(SAGE_E_ARG, "sage_status_mirror: pointers must be 4-byte aligned");
  cudaError_t e = cudaMemcpyAsync(status_host, status_dev, sizeof(int32_t) * (size_t)words, cudaMemcpyDeviceToHost,
                                  reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(SAGE_E_CUDA, "sage_status_mirror: %s", cudaGetErrorString(e));
  return SAGE_OK;
}

void sage_debug_tiles_per_cta(int n) { sage::set_tiles_per_cta(n); }

void sage_debug_skip_threshold(float log2_units) { sage::set_skip_log2(log2_units); }

int sage_attention_tiles_per_cta(int64_t B, int64_t Hq, int64_t Nq, int causal, int sm_count) {
  if (B < 1 || Hq < 1 || Nq < 1 || sm_count < 1) return 0;
  return sage::choose_tiles_per_cta((Nq + sage::TILE - 1) / sage::TILE, B * Hq, causal != 0, sm_count);
}

size_t sage_workspace_bytes(int64_t B, int64_t H, int64_t N) {
  if (B < 1 || H < 1 || N < 1) return 0;
  const Dims d = {B, H, H, N, N, sage::HD};
  return carve(d).total;
}

size_t sage_workspace_bytes_ex(int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk) {
  const Dims d = {B, Hq, Hkv, Nq, Nk, sage::HD};
  if (B < 1 || Hq < 1 || Hkv < 1 || Nq < 1 || Nk < 1 || Hq % Hkv) return 0;
  return carve(d).total;
}

static int layout_out(const Dims& d, size_t* offsets, int n) {
  const Layout L = carve(d);
  const size_t o[13] = {L.q8, L.sq, L.k8, L.sk, L.v8t, L.sv, L.svp, L.s_fold, L.mean, L.ctrl, L.status, L.qm, L.vmean};
  memcpy(offsets, o, sizeof(size_t) * (size_t)n);
  return n;
}

int sage_workspace_layout(int64_t B, int64_t H, int64_t N, size_t offsets[11]) {
  if (B < 1 || H < 1 || N < 1 || !offsets) return fail(SAGE_E_ARG, "sage_workspace_layout: bad argument");
  const Dims d = {B, H, H, N, N, sage::HD};
  return layout_out(d, offsets, 11);
}

int sage_workspace_layout_ex(int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk, size_t offsets[13]) {
  if (B < 1 || Hq < 1 || Hkv < 1 || Nq < 1 || Nk < 1 || Hq % Hkv || !offsets)
    return fail(SAGE_E_ARG, "sage_workspace_layout_ex: bad argument");
  const Dims d = {B, Hq, Hkv, Nq, Nk, sage::HD};
  return layout_out(d, offsets, 13);
}

int sage_attention(const void* q, const void* k, const void* v, void* out,
                   void* workspace, size_t workspace_bytes,
                   int64_t B, int64_t H, int64_t N,
                   const int64_t q_strides[3], const int64_t k_strides[3],
                   const int64_t v_strides[3], const int64_t o_strides[3],
                   int dtype, int qk_mode, int causal, int smooth_k, float sm_scale, void* stream) {
  const Dims d = {B, H, H, N, N, sage::HD};
  return attention_impl(q, k, v, out, nullptr, workspace, workspace_bytes, d, q_strides, k_strides, v_strides,
                        o_strides, dtype, qk_mode, causal, smooth_k, 0, sm_scale, stream, "sage_attention");
}

int sage_attention_ex(const void* q, const void* k, const void* v, void* out, float* lse,
                      void* workspace, size_t workspace_bytes,
                      int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk, int64_t head_dim,
                      const int64_t q_strides[3], const int64_t k_strides[3],
                      const int64_t v_strides[3], const int64_t o_strides[3],
                      int dtype, int qk_mode, int causal, int smooth_k, int smooth_v, float sm_scale, void* stream) {
  const Dims d = {B, Hq, Hkv, Nq, Nk, head_dim};
  return attention_impl(q, k, v, out, lse, workspace, workspace_bytes, d, q_strides, k_strides, v_strides,
                        o_strides, dtype, qk_mode, causal, smooth_k, smooth_v, sm_scale, stream, "sage_attention_ex");
}

int sage_attention_varlen(const void* q, const void* k, const void* v, void* out,
                          const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                          void* workspace, size_t workspace_bytes,
                          int64_t n_seq, int64_t Hq, int64_t Hkv,
                          int64_t total_q, int64_t total_k, int64_t max_q, int64_t max_k, int64_t head_dim,
                          const int64_t q_strides[2], const int64_t k_strides[2],
                          const int64_t v_strides[2], const int64_t o_strides[2],
                          int dtype, int qk_mode, int causal, int smooth_k, float sm_scale, void* stream) {
  g_err[0] = 0;
  if (!cu_seqlens_q || !cu_seqlens_k) return fail(SAGE_E_ARG, "sage_attention_varlen: cu_seqlens pointer is null");
  if ((reinterpret_cast<uintptr_t>(cu_seqlens_q) | reinterpret_cast<uintptr_t>(cu_seqlens_k)) & 3u)
    return fail(SAGE_E_ARG, "sage_attention_varlen: cu_seqlens must be 4-byte aligned");
  if (total_q < 1 || total_k < 1) return fail(SAGE_E_ARG, "sage_attention_varlen: the packed tensors hold no tokens");
  if (max_q > total_q || max_k > total_k)
    return fail(SAGE_E_ARG, "sage_attention_varlen: a longest length exceeds the packed token count");
  if (total_q >= ((int64_t)1 << 31) || total_k >= ((int64_t)1 << 31))
    return fail(SAGE_E_UNSUPPORTED, "sage_attention_varlen: more than 2^31 - 1 packed tokens");
  if (!q_strides || !k_strides || !v_strides || !o_strides) return fail(SAGE_E_ARG, "sage_attention_varlen: strides are null");
  // (batch, head, row) triples for the shared checks; the batch entry is not used by the kernels
  const int64_t qs[3] = {q_strides[0], q_strides[1], q_strides[0]}, ks[3] = {k_strides[0], k_strides[1], k_strides[0]};
  const int64_t vs[3] = {v_strides[0], v_strides[1], v_strides[0]}, os[3] = {o_strides[0], o_strides[1], o_strides[0]};
  const Dims d = {n_seq, Hq, Hkv, max_q, max_k, head_dim};
  const Packed pk = {cu_seqlens_q, cu_seqlens_k, total_q, total_k};
  return attention_impl(q, k, v, out, nullptr, workspace, workspace_bytes, d, qs, ks, vs, os, dtype, qk_mode,
                        causal, smooth_k, 0, sm_scale, stream, "sage_attention_varlen", pk);
}

}  // extern "C"
