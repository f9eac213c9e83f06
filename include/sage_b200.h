/* C-ABI of libsage_b200.so: the quantize-then-attend hot path for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; no torch types, no C++ exceptions across the boundary.  Every
 * function returns 0 on success or a negative SAGE_E_* code, and `sage_last_error()` then returns a
 * one-line description (thread-local).  All pointers except `strides` arrays are DEVICE pointers.
 * All work is enqueued on `stream` (a cudaStream_t passed as void*, NULL = default stream); nothing
 * synchronises, nothing allocates: the caller owns every buffer, as in the reference, where the
 * Python side allocates with torch.empty and hands raw pointers to extern "C" kernels.
 *
 * Citations below are paths inside the reference project (IxMxAMAR/SageAttention-RDNA4).
 */
#ifndef SAGE_B200_H
#define SAGE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SAGE_HEAD_DIM 128        /* the only head_dim the hand-written path serves            */
#define SAGE_TILE 128            /* query tile and key tile; key length is padded to this     */

enum { SAGE_F16 = 0, SAGE_BF16 = 1 };            /* element type of q, k, v and of the output  */
enum { SAGE_QK_INT8 = 0, SAGE_QK_E4M3 = 1 };     /* code type of the quantised Q and K         */
/* May be ORed into the qk_mode of the attention entry points (sage_attn_fwd*, sage_attention*; for
 * the "default" mode of sage_attention* pass -SAGE_QK_NO_FAST_PATH instead of -1): the attention
 * kernel then runs without its negligible-tile tests.  Those tests skip the exponentials of key
 * tiles that lie at least 40 exponent units below the running row maxima (see
 * sage_debug_skip_threshold); they cost 3 to 6 % on inputs where no tile can be skipped, so a
 * host that knows its inputs have no dominant keys switches them off.  The Python package does so
 * by itself from the skipped-tile counts of earlier calls. */
#define SAGE_QK_NO_FAST_PATH 0x100

enum {
  SAGE_OK = 0,
  SAGE_E_ARG = -1,        /* contract violation: null pointer, bad size, misaligned pointer    */
  SAGE_E_UNSUPPORTED = -2,/* valid request this build does not serve                           */
  SAGE_E_CUDA = -3,       /* a CUDA runtime/driver call failed; see sage_last_error()          */
  SAGE_E_WORKSPACE = -4   /* workspace too small                                               */
};

/* Library version (major*10000 + minor*100 + patch). */
int sage_version(void);

/* Description of the last failure on the calling thread ("" if none). */
const char* sage_last_error(void);

/* Padded key length: N rounded up to SAGE_TILE.  Replaces `n_pad = ceil(N/64)*64`
 * (sageattention/sk1_backend/hip_prologue.py:93-95); the tile here is 128 keys. */
int64_t sage_pad_len(int64_t n);

/* Bytes of the control block `ctrl` the prologue needs for B*H heads (mean partial sums, per-head
 * arrival counters, per-head running max of the V scale).  256-byte aligned device memory. */
size_t sage_prologue_ctrl_bytes(int64_t B, int64_t H, int64_t N);

/* The quantisation prologue: Q, K, V -> Q8, SQ, K8, SK, V8T, SV, SVP, S (and MEAN).
 *
 * Replaces HipPrologue.quant_kv (sageattention/sk1_backend/hip_prologue.py:188-244, kernels
 * h34_kseq_mean_* and h34_quant_kv_* in kernels/hip/h34_prologue.hip:91-294), the in-kernel Q
 * quantisation of the attention kernels (kernels/hip/sk1_t6i.hip:91-117,
 * kernels/hip/sk1_t4a1sb.hip:73-100) and fold_v_scale
 * (sageattention/sk1_backend/__init__.py:561-579).
 *
 *   q, k, v   logical (B,H,N,128) fp16/bf16 views; q_strides/k_strides/v_strides give the
 *             (batch, head, row) strides in ELEMENTS; the last axis is contiguous; every stride is
 *             a multiple of 8 and every base pointer 16-byte aligned.
 *   q8        (B*H, N, 128)      int8 | e4m3 codes of Q, one scale per token
 *   sq        (B*H, N)           fp32 dequant scale of Q: amax/127 (int8) or amax/448 (e4m3)
 *   k8        (B*H, N_pad, 128)  codes of K - mean; pad rows 0.  Row order: inside every block of
 *                                16 keys, key 4c + j is stored in row 2c + j (j < 2) or
 *                                8 + 2c + j - 2 (j = 2, 3), the order the attention kernel's
 *                                TMEM loads want; sk, sv, svp and v8t are in key order
 *   sk        (B*H, N_pad)       fp32 scale of K; pad rows 1.0
 *   v8t       (B*H, 128, N_pad)  e4m3 codes of V, transposed; pad columns 0
 *   sv        (B*H, N_pad)       fp32 scale of V; pad rows 0.0
 *   svp       (B*H, N_pad)       fp32 staged factor  fl(fl(sv / S) * 448)
 *   s_fold    (B*H)              S = max(max_n sv, 1)
 *   mean      (B*H, 128)         fp32 sequence mean of K (written only when smooth_k != 0)
 *   ctrl      sage_prologue_ctrl_bytes() of scratch; contents need not be initialised.  After the
 *             call its 32-bit word number 4*B*H is non-zero if a bounded wait inside the quantiser
 *             ran out (the outputs are then undefined); sage_attention reports the same event as
 *             the value 8 ORed into its status word
 *   N_pad     must equal sage_pad_len(N)
 * Alignment: q, k, v, q8, k8, v8t, sk, sv, svp and ctrl (and vmean of sage_prologue_ex) are read or
 * written with 16-byte vector accesses and must be 16-byte aligned; a misaligned one is refused
 * with SAGE_E_ARG before anything is launched.  sq, s_fold, mean and qm need 4-byte alignment.
 * Three kernel launches (a one-block kernel that clears the control words, mean, quantise). */
int sage_prologue(const void* q, const void* k, const void* v,
                  void* q8, float* sq, void* k8, float* sk, void* v8t, float* sv, float* svp,
                  float* s_fold, float* mean, void* ctrl,
                  int64_t B, int64_t H, int64_t N, int64_t N_pad,
                  const int64_t q_strides[3], const int64_t k_strides[3],
                  const int64_t v_strides[3],
                  int dtype, int qk_mode, int smooth_k, void* stream);

/* The prologue for callers that must not allocate.  It has no counterpart in the reference.
 *
 * Same work and same results as sage_prologue, but the `ctrl` scratch is not passed in: it is a
 * 1 MiB array built into the library's device image (sage_prologue_static_ctrl_capacity() bytes;
 * every GPU that loads the library holds it until the process exits).  Meant for hosts that may
 * not call cudaMalloc where they run the prologue -- a plugin's enqueue step that only gets
 * pre-assigned buffers, a serving process under a hard memory cap, a latency path that cannot
 * take cudaMalloc's implicit synchronisation.  The function calls no cudaMalloc, no cudaFree and
 * no allocating library routine; inputs and outputs are still the caller's.
 *   - Shapes whose scratch need (sage_prologue_ctrl_bytes) exceeds the capacity are refused with
 *     SAGE_E_UNSUPPORTED and a message; nothing is launched.
 *   - The first call on each device looks up the array's device address (the device must be
 *     current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array, and it keeps the previous call's contents; the
 *     words that must start at zero are cleared on the stream at the start of each call.  Two
 *     calls whose GPU work overlaps (different streams, no ordering between them) race on it:
 *     order them, or give one of them its own scratch through sage_prologue.
 *   - `status` (optional, may be NULL): one int32 in the caller's device memory.  The quantiser's
 *     own failure flag lives inside the built-in array, which the caller cannot read, so a
 *     bounded wait that ran out is reported here instead: the value 8 is ORed into the word and
 *     the outputs of that call are undefined.  The call never clears the word; zero it once and
 *     read it whenever the stream is known to have passed the call. */
size_t sage_prologue_static_ctrl_capacity(void);
int sage_prologue_static_ctrl(const void* q, const void* k, const void* v,
                              void* q8, float* sq, void* k8, float* sk, void* v8t, float* sv,
                              float* svp, float* s_fold, float* mean,
                              int64_t B, int64_t H, int64_t N, int64_t N_pad,
                              const int64_t q_strides[3], const int64_t k_strides[3],
                              const int64_t v_strides[3],
                              int dtype, int qk_mode, int smooth_k, int32_t* status, void* stream);

/* The attention kernel on quantised operands.
 *
 * Replaces Sk1Attn.launch / launch_strided (sageattention/sk1_backend/sk1_loader.py:628-688) and
 * the kernels sk1t6i_attn_fwd_c0/_c1 (kernels/hip/sk1_t6i.hip:69-316) and
 * sk1t4a1sb_attn_fwd_c0/_c1 (kernels/hip/sk1_t4a1sb.hip:51-308).
 *
 *   out        logical (B,H,N,128) fp16/bf16 view with (batch, head, row) ELEMENT strides
 *              o_strides, last axis contiguous, strides multiples of 8, 16-byte aligned base.
 *   status     one int32 in device memory, zero before the call; the kernel ORs in a non-zero
 *              code if one of its bounded waits gave up (the output is then undefined).
 *   sm_scale   finite and > 0 (anything else is refused with SAGE_E_ARG: the kernel takes the row
 *              maximum before it applies the scale).
 * The operands are the prologue's outputs for the same B, H, N, N_pad, qk_mode; q8, k8, v8t, sk,
 * svp, out (and vmean of sage_attn_fwd_ex) must be 16-byte aligned. */
int sage_attn_fwd(const void* q8, const float* sq, const void* k8, const float* sk,
                  const void* v8t, const float* svp, const float* s_fold, void* out,
                  int64_t B, int64_t H, int64_t N, int64_t N_pad, const int64_t o_strides[3],
                  int causal, float sm_scale, int out_dtype, int qk_mode,
                  int32_t* status, void* stream);

/* Enqueue, on `stream`, a copy of `words` (1..4) 32-bit words starting at a status word (device
 * memory: the `status` of sage_attn_fwd with words = 1, or the word at offset 10 of
 * sage_workspace_layout, where word 3 after it counts the (warp, key tile) pairs the attention
 * kernel's fast path skipped in that call: 16 warps per pair of query tiles, so the count divided
 * by 8 * query tiles * key tiles * heads is the skipped share) into `status_host`, which should be pinned
 * host memory so that the copy does not block.  Nothing synchronises: once the stream has passed
 * this point the host word holds the call's status, non-zero after a bounded wait ran out.  This
 * is how a host learns of a device-side failure without waiting for every call; the reference
 * raises for such failures only in strict mode and otherwise falls back
 * (sageattention/sk1_backend/__init__.py:1022-1027,1114-1123).  Status bits: 1 TMA producer,
 * 2 MMA issuer, 4 softmax warp of the attention kernel; 8 tile load of the prologue. */
int sage_status_mirror(const int32_t* status_dev, int32_t* status_host, int words, void* stream);

/* Test hook (one process-wide atomic word): the attention kernel has two shapes, one or two
 * 128-query tiles per CTA, and picks the one it expects to finish sooner for the call's size.
 * n = 1 or 2 forces that shape for later launches from any thread, anything else restores the
 * automatic choice.  Both shapes give bit-identical results. */
void sage_debug_tiles_per_cta(int n);

/* Test hook (one process-wide atomic word): threshold of the attention kernel's negligible-tile
 * fast path.  A key tile whose scores, for all 16 query rows a warp owns, lie at least
 * `log2_units` below those rows' running maxima (in the base-2 exponent domain) is not
 * exponentiated: its P entries are exact zeros either way (p * svp < 2^-40 * 448 rounds to the
 * e4m3 zero) and the row sums lose less than 128 * 2^-log2_units of their largest term per tile.
 * Default 40; 0 switches the path off (every tile is exponentiated, as the reference does:
 * kernels/hip/sk1_t6i.hip:162-279); a negative value restores the default. */
void sage_debug_skip_threshold(float log2_units);

/* The shape the attention kernel takes, left to itself, for B x Hq heads of Nq queries on a device
 * with sm_count SMs: 1 or 2 query tiles per CTA (0 for bad arguments).  Host arithmetic only. */
int sage_attention_tiles_per_cta(int64_t B, int64_t Hq, int64_t Nq, int causal, int sm_count);

/* Bytes of workspace `sage_attention` needs for one call (all intermediates + ctrl + status). */
size_t sage_workspace_bytes(int64_t B, int64_t H, int64_t N);

/* The whole call: prologue + attention, the path `sageattn` takes
 * (sageattention/sk1_backend/__init__.py:982-1284, try_sk1_t1).  `workspace` is
 * sage_workspace_bytes() of 256-byte aligned device memory owned by the caller.  qk_mode follows
 * the reference's default when negative: int8 for fp16 inputs, e4m3 for bf16. */
int sage_attention(const void* q, const void* k, const void* v, void* out,
                   void* workspace, size_t workspace_bytes,
                   int64_t B, int64_t H, int64_t N,
                   const int64_t q_strides[3], const int64_t k_strides[3],
                   const int64_t v_strides[3], const int64_t o_strides[3],
                   int dtype, int qk_mode, int causal, int smooth_k, float sm_scale,
                   void* stream);

/* ---- The same three entry points for the upstream call shapes the reference's hand-written path
 * refuses and hands to its other backends: grouped-query attention (Hq query heads sharing Hkv
 * key/value heads, Hq a multiple of Hkv), a key length different from the query length
 * (non-causal only), the log-sum-exp output, and a head_dim below 128 (upstream zero-pads such
 * heads to 64 or 128 columns on the host, sageattention/core.py:1524-1533; here the prologue reads
 * `head_dim` columns per row and zero-fills the 128-wide codes itself, and the attention kernel
 * writes `head_dim` output columns).  They replace, for those shapes, the fallback
 * `sageattn_qk_int8_pv_gfx12_native` (sageattention/core.py:470-1034) and follow the upstream
 * contract of `sageattn_qk_int8_pv_fp8_cuda` (sageattention/core.py:1747-1938: num_qo_heads a
 * multiple of num_kv_heads, return_lse with the smooth_k correction of :1893-1897,1935-1936).
 *
 *   q, out     logical (B,Hq,Nq,head_dim); k, v logical (B,Hkv,Nk,head_dim);
 *              head_dim a multiple of 8 in 8..128
 *   lse        optional (B*Hq, Nq) fp32: ln sum_k exp(sm_scale * q.k) of the UNquantised softmax
 *              the kernel evaluates (its row maximum and row sum), plus sm_scale * q.mean(K) when
 *              smooth_k is on, so that it refers to the caller's K, not the mean-subtracted one
 *   qm         (prologue output / attention input, optional) (B*Hq, Nq) fp32 q.mean(K); needed
 *              only when an LSE is wanted and smooth_k is on
 *   vmean      (prologue output / attention input, optional) (B*Hkv, 128) fp32 mean of V over its
 *              keys: upstream's `smooth_v` (sageattention/core.py:1917-1923, quant.py:297-301).  When
 *              given, V minus this mean is what gets quantised and the attention kernel adds the
 *              mean back to every output row (the softmax weights of a row sum to one)
 * Every size of K/V tensors (k8, sk, v8t, sv, svp, s_fold, mean, ctrl) is as for sage_prologue with
 * H = Hkv and N = Nk; q8 and sq are (B*Hq, Nq, 128) and (B*Hq, Nq). */
int sage_prologue_ex(const void* q, const void* k, const void* v,
                     void* q8, float* sq, void* k8, float* sk, void* v8t, float* sv, float* svp,
                     float* s_fold, float* mean, float* qm, float* vmean, void* ctrl,
                     int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk, int64_t Nk_pad,
                     int64_t head_dim, const int64_t q_strides[3], const int64_t k_strides[3],
                     const int64_t v_strides[3],
                     int dtype, int qk_mode, int smooth_k, void* stream);
int sage_attn_fwd_ex(const void* q8, const float* sq, const void* k8, const float* sk,
                     const void* v8t, const float* svp, const float* s_fold, void* out,
                     float* lse, const float* qm, const float* vmean,
                     int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk, int64_t Nk_pad,
                     int64_t head_dim, const int64_t o_strides[3], int causal, float sm_scale, int out_dtype,
                     int qk_mode, int32_t* status, void* stream);
size_t sage_workspace_bytes_ex(int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk);
int sage_attention_ex(const void* q, const void* k, const void* v, void* out, float* lse,
                      void* workspace, size_t workspace_bytes,
                      int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk, int64_t head_dim,
                      const int64_t q_strides[3], const int64_t k_strides[3],
                      const int64_t v_strides[3], const int64_t o_strides[3],
                      int dtype, int qk_mode, int causal, int smooth_k, int smooth_v, float sm_scale,
                      void* stream);
/* As sage_workspace_layout, with two more entries: qm, vmean. */
int sage_workspace_layout_ex(int64_t B, int64_t Hq, int64_t Hkv, int64_t Nq, int64_t Nk,
                             size_t offsets[13]);

/* ---- A packed variable-length batch in one call: replaces `sageattn_varlen`
 * (sageattention/core.py:1444-1558), whose per-block quantisers take `cu_seqlens` and whose kernel
 * is launched once for the whole batch.  The cumulative lengths stay on the device: nothing is read
 * back, so the call neither synchronises nor depends on host copies of the lengths.
 *
 *   q, out         packed (total_q, Hq, head_dim); k, v packed (total_k, Hkv, head_dim); strides are
 *                  (token, head) pairs in elements, multiples of 8, last axis contiguous
 *   cu_seqlens_q/k DEVICE int32 arrays of n_seq + 1 entries, cu[0] = 0, non-decreasing,
 *                  cu[n_seq] = total_q / total_k; sequence i has cu[i+1] - cu[i] rows
 *   max_q, max_k   upper bounds of the sequence lengths: they size the workspace
 *                  (sage_workspace_bytes_ex(n_seq, Hq, Hkv, max_q, max_k)) and the grids.  A
 *                  sequence longer than the bound is cut off at the bound (its further query rows
 *                  are not written, its further keys not seen)
 *   causal         every sequence must have as many keys as queries (max_q == max_k is checked;
 *                  the per-sequence equality is the caller's promise)
 * Each sequence is quantised on its own (its own K mean with smooth_k, its own S), exactly as if it
 * were passed alone to sage_attention_ex: the results are bit-identical to per-sequence calls.
 * A sequence without queries costs nothing; one with queries and no keys gets rows of zeros.
 * The arrays are not validated (that would need them on the host); the kernels clamp every start
 * and end to the packed token counts, so that no access leaves q, k, v or out whatever they hold.
 * The kernels run the one-tile shape without the negligible-tile tests.  Status word and errors as
 * for sage_attention (the layout is sage_workspace_layout_ex(n_seq, Hq, Hkv, max_q, max_k)). */
int sage_attention_varlen(const void* q, const void* k, const void* v, void* out,
                          const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                          void* workspace, size_t workspace_bytes,
                          int64_t n_seq, int64_t Hq, int64_t Hkv,
                          int64_t total_q, int64_t total_k, int64_t max_q, int64_t max_k,
                          int64_t head_dim,
                          const int64_t q_strides[2], const int64_t k_strides[2],
                          const int64_t v_strides[2], const int64_t o_strides[2],
                          int dtype, int qk_mode, int causal, int smooth_k, float sm_scale,
                          void* stream);

/* Offsets (bytes from `workspace`) of the intermediates sage_attention uses, for callers and
 * tests that want to look at them: order q8, sq, k8, sk, v8t, sv, svp, s_fold, mean, ctrl, status
 * (the status word is a spare word inside the ctrl block, so that one clearing kernel clears both).
 * Returns the number of entries written (11). */
int sage_workspace_layout(int64_t B, int64_t H, int64_t N, size_t offsets[11]);

#ifdef __cplusplus
}
#endif
#endif /* SAGE_B200_H */
