// Internal C++ interface between the C-ABI translation unit and the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sage {

struct PrologueParams {
  const void *q, *k, *v;
  void *q8, *k8, *v8t;
  float *sq, *sk, *sv, *svp, *s_fold, *mean;
  void* ctrl;
  float* qm;                                           // optional (B*Hq, Nq): q . K-mean, for the LSE
  float* vmean;                                        // optional (B*H, 128): smooth_v subtracts the sequence mean of V
  int32_t* status;                                     // optional: receives bit 8 if a wait on a tile load ran out
  int64_t B, H, N, N_pad;                              // K/V side: heads, keys, padded keys
  int64_t Hq, Nq;                                      // query side (Hq a multiple of H)
  int64_t D;                                           // head_dim of q/k/v rows (multiple of 8, <= 128); codes are 128 wide, zero-filled
  int64_t q_strides[3], k_strides[3], v_strides[3];   // (batch, head, row) in elements
  int dtype;      // 0 fp16, 1 bf16
  int qk_mode;    // 0 int8, 1 e4m3
  int smooth_k;
  // Packed variable-length batch (both null for a fixed-length call): device arrays of B + 1
  // cumulative token counts.  Sequence b then has cu_q[b+1] - cu_q[b] queries and
  // cu_k[b+1] - cu_k[b] keys, its rows start at token cu[b] of the packed (tokens, heads, D)
  // tensors (the batch strides are not used), Nq / N are the largest lengths allowed and size the
  // outputs, Tq / Tk the token counts of the packed tensors.
  const int32_t *cu_q, *cu_k;
  int64_t Tq, Tk;
};

struct AttnParams {
  const void *q8, *k8, *v8t;
  const float *sq, *sk, *svp, *s_fold;
  void* out;
  float* lse;                                          // optional (B*Hq, Nq) natural-log sum of exponentials
  const float* qm;                                     // with lse and smooth_k: q . K-mean per query row
  const float* vmean;                                  // with smooth_v: (B*H, 128) mean of V, added back to every output row
  int64_t B, H, N, N_pad;                              // K/V side: heads, keys, padded keys
  int64_t Hq, Nq;                                      // query side
  int64_t D;                                           // columns of an output row that exist (head_dim)
  int64_t o_strides[3];                                // (batch, head, row) in elements
  int causal;
  float sm_scale;
  int out_dtype;  // 0 fp16, 1 bf16
  int qk_mode;    // 0 int8, 1 e4m3
  int32_t* status;
  int no_fast_path;                                    // 1: the kernels without the negligible-tile tests
  unsigned* skipped;                                   // optional: (warp, key tile) pairs the fast path skipped
  const int32_t *cu_q, *cu_k;                          // packed variable-length batch (see PrologueParams); null otherwise
  int64_t Tq, Tk;                                      // with cu_q / cu_k: tokens in the packed tensors
};

cudaError_t launch_prologue(const PrologueParams& p, cudaStream_t st);
size_t prologue_ctrl_bytes(int64_t B, int64_t H, int64_t N);

// Returns cudaSuccess or an error; `why` (if non-null) receives a static description on failure.
cudaError_t launch_attention(const AttnParams& p, cudaStream_t st, const char** why);

// Test hook: force the attention kernel's shape (1 or 2 query tiles per CTA; 0 = automatic).
void set_tiles_per_cta(int n);
// Test hook: threshold (log2 units) of the attention kernel's negligible-tile fast path; 0 = off, < 0 = default.
void set_skip_log2(float t);
int choose_tiles_per_cta(int64_t q_tiles, int64_t bhq, bool causal, int sms);

}  // namespace sage
