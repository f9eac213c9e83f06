// Quantised flash attention for B200 (sm_100a): tcgen05 tensor cores, TMEM accumulators, TMA tiles.
//
// A query tile is 128 queries of one (batch, head); it streams 128-key tiles.  The kernel comes in
// two shapes (template parameter NQ, query tiles per CTA):
//   NQ = 1   one query tile per CTA, 384 threads, two CTAs per SM, so that one CTA's softmax
//            overlaps the other's matrix products.  Calls whose two-tile grid would end in a
//            nearly empty round (see launch_attention).
//   NQ = 2   two neighbouring query tiles of a head per CTA, 640 threads, one CTA per SM: each K
//            and V^T tile is loaded once for both, each query tile has its own softmax warps,
//            TMEM columns, P tiles and MMA-issuing threads.  (Causal: the second tile
//            visits one key tile more than the first.)
// Both shapes compute every row with the same instructions in the same order.  Roles inside a CTA
// with one query tile:
//   warp 0     TMA producer: the Q tile once, then a 2-deep ring of K tiles (each carrying that
//              tile's 128 K scales and 128 staged V factors into a 4-slot ring) and the V^T tiles
//              (a single stage; the shared memory of a second one holds the second P tile)
//   warp 1     allocates the TMEM columns; one thread issues every tcgen05.mma
//   warps 2, 3 idle: they complete the first warpgroup, whose registers setmaxnreg hands over
// and with two query tiles (256 x 2 TMEM columns, 2-deep rings of K and of V^T tiles), where the
// four product streams of a key tile are spread over the four schedulers of the SM -- issuing a
// tcgen05.mma or a commit holds up the issuing warp's scheduler, and the softmax warps of the most
// loaded scheduler set the CTA's pace:
//   warp 0     loads the Q tiles, then issues Q.K^T of query tile 0
//   warp 1     issues Q.K^T of query tile 1 and, behind each, loads the K tile two ahead (with its
//              scale rows) once both tiles' products on that stage have completed
//   warp 2     issues P.V of query tile 0
//   warp 3     issues P.V of query tile 1 and, behind each, loads the V^T tile two ahead
//              (the loads ride with query tile 1 because it runs behind tile 0: its threads would
//              wait for tile 0's product anyway, tile 0's threads would wait for tile 1's)
//   warps 4-11 (and 12-19 for the second query tile) softmax: a warp owns 16 query rows (TMEM
//              lanes) and all 128 key columns, read with the 16-lane 16x256b shape: four threads
//              share a row, each holds two rows, and a row maximum is two shuffles
// Per key tile j:
//   S  = Q8 . K8^T          kind::i8 (s32) or kind::f8f6f4 (f32), M=N=K=128, into 128 TMEM columns
//   u  = f32(S) * sk[key]; mask; row max m (in the u domain); s = c_q * u is the log2-domain score
//   alpha = exp2(c_q*(m_old - m_new)); O *= alpha in TMEM when some row's max moved
//   p  = exp2(c_q*u - c_q*m); l = l*alpha + sum(p); P8 = e4m3(p * svp[key]) written to shared
//        memory as unswizzled K-major core matrices, four keys (one 32-bit word) at a time; P(j)
//        and P(j+1) go to different tiles, so P(j+1) is written while P.V(j) still reads P(j)
// The rows of a K8 tile arrive permuted inside 16-row blocks (the prologue stores them so) to make
// the four score columns a thread holds of a 16-column block four consecutive keys.
//   O += P8 . V8            kind::f8f6f4 into 128 more TMEM columns
// Epilogue: out = O * (S_fold / (l * 448)) (+ mean of V with smooth_v) -> fp16 / bf16, the first
// head_dim columns of each row; optionally LSE = ln2 * (c_q*m + log2 l) + sm_scale * q.mean(K).
// Grouped-query heads: the CTA of query head h reads the K/V tiles and scales of head h / group.
// (numerics: kernels/hip/sk1_t6i.hip:151-299 and kernels/hip/sk1_t4a1sb.hip:176-189 of the
// reference, with a 128-key instead of a 64-key tile for the running max; the two score factors
// c_q and sk are applied one after the other instead of as one pre-multiplied factor, a
// difference of one rounding in a quantity the reference does not pin bit-wise)
//
// Every kernel is instantiated twice (template parameter FAST).  The FAST kernels test every key
// tile against the running row maxima and do not exponentiate a tile whose scores all lie 40
// exponent units or more below them (its P entries are exact zeros either way); they count what
// they skip.  The others carry none of that code, and the host chooses between the two sets
// (see the comment at the softmax warps' loop and launch_attention).
//
// Every wait on an mbarrier is bounded: after about two seconds, or as soon as another CTA has
// reported a failure, the waiter records a code in the status word, the CTA drains and frees its
// TMEM, and CTAs that start later return at once.
#include <cuda.h>

#include <atomic>

#include "sage_common.cuh"
#include "sage_internal.h"

namespace sage {

constexpr uint32_t TILE_BYTES = TILE * HD;          // 16 KiB: 128 rows x 128 one-byte codes
constexpr uint32_t VEC_BYTES = TILE * 4;            // 128 floats

// Threads, registers, shared memory and TMEM of a CTA that owns NQ query tiles.
template <int NQ> struct Shape {
  static constexpr int THREADS = 128 + 256 * NQ;    // {TMA, MMA, MMA or idle, idle} + 8 softmax warps per tile
  static constexpr int CTAS_PER_SM = (NQ == 1) ? 2 : 1;
  // what __launch_bounds__(THREADS, CTAS_PER_SM) yields: 65536 / (THREADS x CTAS_PER_SM), rounded
  // down to a multiple of 8
  static constexpr int REGS_AT_LAUNCH = (NQ == 1) ? 80 : 96;
  static constexpr int REGS_PRODUCER = 32;                      // after setmaxnreg
  static constexpr int REGS_SOFTMAX = (NQ == 1) ? 104 : 112;
  static constexpr uint32_t OFF_Q = 0;
  static constexpr uint32_t OFF_K = OFF_Q + NQ * TILE_BYTES;    // 2 stages
  // Two P tiles per query tile: the softmax warps write P(j) without waiting for the product that
  // reads P(j-1), and wait for it only where they need the output accumulator.  Two one-tile CTAs
  // share an SM's shared memory, so that shape pays for the second P tile with a single V^T stage:
  // V^T(j) is fetched once P.V(j-1) has completed, a tile ahead of its use, and the K ring runs
  // one tile further ahead so that it is not held up behind that wait.
  static constexpr int V_STAGES = (NQ == 1) ? 1 : 2;
  static constexpr int K_AHEAD = (NQ == 1) ? 1 : 0;
  static constexpr int P_BUFS = 2;
  static constexpr uint32_t OFF_V = OFF_K + 2 * TILE_BYTES;
  static constexpr uint32_t OFF_P = OFF_V + V_STAGES * TILE_BYTES;
  static constexpr uint32_t OFF_SK = OFF_P + NQ * P_BUFS * TILE_BYTES;   // 4-slot ring of K scales (arrive with the K tile)
  static constexpr uint32_t OFF_SV = OFF_SK + 4 * VEC_BYTES;    // 4-slot ring of staged V factors (same barrier)
  static constexpr uint32_t OFF_BAR = OFF_SV + 4 * VEC_BYTES;
  static constexpr uint32_t OFF_MISC = OFF_BAR + 192;
  static constexpr uint32_t SMEM_USED = OFF_MISC + 64;
  static constexpr uint32_t SMEM_BYTES = SMEM_USED + 1024;      // slack for the 1024-byte alignment
  static constexpr uint32_t TMEM_COLS = 256 * NQ;
  // score and output columns of query tile g
  __host__ __device__ static constexpr uint32_t tmem_s(int g) { return 128u * (uint32_t)g; }
  __host__ __device__ static constexpr uint32_t tmem_o(int g) { return 128u * NQ + 128u * (uint32_t)g; }
};

// The K/V stage barriers are shared by the query tiles of a CTA; the last four repeat per query
// tile (+ BAR_PER_TILE x g).
enum Bar { BAR_Q = 0, BAR_KF = 1, BAR_KE = 3, BAR_VF = 5, BAR_VE = 7, BAR_SF = 9, BAR_SFREE = 10,
           BAR_PF = 11, BAR_PV = 12, BAR_PER_TILE = 4, BAR_COUNT = 17 };
static_assert(BAR_COUNT * 8 <= 192, "barrier area");

enum { ST_TIMEOUT_PRODUCER = 1, ST_TIMEOUT_MMA = 2, ST_TIMEOUT_SOFTMAX = 4 };

constexpr long long WAIT_CYCLES = 4000000000LL;      // about two seconds of SM clock

// ------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
// Bounded wait.  Returns false when it gave up (its own time limit, or a failure flagged by
// someone else); the caller then leaves its loop.
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* cta_abort,
                                            int32_t* status, int code) {
  const long long t0 = clock64();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 255u) == 0u) {
      if (*cta_abort) return false;
      if (*reinterpret_cast<volatile int32_t*>(status) != 0) { *cta_abort = 1u; return false; }
      if (clock64() - t0 > WAIT_CYCLES) {
        atomicOr(status, code);
        *cta_abort = 1u;
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* cta_abort,
                                          int32_t* status, int code) {
  // first attempt may suspend the thread in hardware for up to the hinted time (no issue slots)
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
  if (__builtin_expect(ok != 0u, 1)) return true;
  return mbar_wait_slow(bar, parity, cta_abort, status, code);
}
// Arrive from lane 0 only, without a branch.
__device__ __forceinline__ void mbar_arrive_lane0(uint32_t bar, int lane) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.eq.s32 p, %1, 0;\n\t"
      "@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}"
      ::"r"(bar), "r"(lane) : "memory");
}
// Four floats -> four e4m3 bytes in memory order (a lowest), round to nearest even, saturating.
__device__ __forceinline__ uint32_t e4m3x4_pack(float a, float b, float c, float d) {
  uint32_t w;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(w) : "f"(a), "f"(b), "f"(c), "f"(d));
  return w;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <bool INT8>
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  if (INT8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  }
}

// 16 lanes x 256 bits per repetition: thread t holds lanes t/4 (registers 4i, 4i+1) and t/4 + 8
// (registers 4i+2, 4i+3), columns 8i + 2(t%4) and the next one; x8 = 64 columns, 32 registers.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x8.b32 [%32], {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b_x16(uint32_t taddr, uint32_t* r) {
  tmem_ld_16x256b_x8(taddr, r);
  tmem_ld_16x256b_x8(taddr + 64, r + 32);
}
__device__ __forceinline__ void tmem_st_16x256b_x16(uint32_t taddr, const uint32_t* r) {
  tmem_st_16x256b_x8(taddr, r);
  tmem_st_16x256b_x8(taddr + 64, r + 32);
}
__device__ __forceinline__ void sts32u(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory accesses through 32-bit shared-window addresses (half the registers of a pointer).
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

// Shared-memory matrix descriptor of a K-major tile of 128-byte rows written with the 128-byte
// swizzle (what TMA SWIZZLE_128B produces): 8-row groups 1024 bytes apart, descriptor version 1.
__device__ __forceinline__ uint64_t kmajor_sw128_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// K-major operand without swizzle: 8-row x 16-byte core matrices of 128 contiguous bytes; the next
// 16 bytes along K are 128 bytes further (leading offset), the next 8 rows 1024 bytes (stride offset).
__device__ __forceinline__ uint64_t kmajor_nosw_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46);
}
// Instruction descriptor: D format at bit 4, A/B formats at bits 7/10, N>>3 at bit 17, M>>4 at 24.
constexpr uint32_t IDESC_I8 = (2u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t IDESC_F8 = (1u << 4) | (0u << 7) | (0u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

struct AttnKArgs {
  const float *sq, *sk, *svp, *s_fold;
  void* out;
  long long N, N_pad, H;          // keys: length, padded length, K/V heads per batch element
  long long Nq, Hq, group;        // queries: length, heads per batch element, Hq / H
  int D;                          // columns of an output row that exist (head_dim <= 128)
  float* lse;                     // optional (B*Hq, Nq)
  const float* qm;                // optional: dot(q row, K mean), added to the LSE (times sm_scale)
  const float* vmean;             // optional (B*H, 128): added to every output row (smooth_v)
  long long o_sb, o_sh, o_sr;
  float sm_scale;
  float skip_log2;    // FAST kernels: key tiles whose scores all lie this far (exponent domain) below the running maxima are not exponentiated
  unsigned* skipped;  // FAST kernels, optional: receives the number of (warp, key tile) pairs that were skipped
  int32_t* status;
  const int *cu_q, *cu_k;   // VARLEN kernels: cumulative token counts of the packed batch (B + 1 entries each)
  long long Tq, Tk;         // VARLEN kernels: tokens in the packed q / out and k / v tensors
};

template <typename OutT> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// ------------------------------------------------------------------------------------------------
// The kernel.  NQ = 1: grid (ceil(Nq/128), B*Hq), block 384, two CTAs per SM; NQ = 2: grid
// (ceil(Nq/256), B*Hq), block 640, one CTA per SM.
// ------------------------------------------------------------------------------------------------
// VARLEN: a packed batch.  a.Nq, a.N_pad are the capacity of a sequence's slot in the quantised
// operands, the grid is sized for the longest sequence allowed; each sequence's own lengths and the
// first row of its output come from cu_q / cu_k, and a CTA whose query tile lies past its
// sequence's end returns at once.
template <bool INT8, bool CAUSAL, typename OutT, int NQ, bool FAST, bool VARLEN>
__global__ void __launch_bounds__(Shape<NQ>::THREADS, Shape<NQ>::CTAS_PER_SM)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnKArgs a) {
  using L = Shape<NQ>;
  constexpr uint32_t OFF_Q = L::OFF_Q, OFF_K = L::OFF_K, OFF_V = L::OFF_V, OFF_P = L::OFF_P, OFF_SK = L::OFF_SK,
                     OFF_SV = L::OFF_SV, OFF_BAR = L::OFF_BAR, OFF_MISC = L::OFF_MISC;
  extern __shared__ uint8_t smem_raw[];
  wait_for_predecessor();            // the quantised operands and the status word
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw_addr);
  const uint32_t bar0 = base + OFF_BAR;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(gbase + OFF_MISC);  // [0] tmem, [1] abort
  volatile uint32_t* cta_abort = misc + 1;
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // first query tile of this CTA (causal: longest first); softmax group g owns tile q_tile0 + g
  const int q_tile0 = NQ * (CAUSAL ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x);
  const int bh = blockIdx.y;                          // (batch, query head)
  const int bh_kv = (int)((bh / a.Hq) * a.H + (bh % a.Hq) / a.group);   // its (batch, K/V head)
  // Key tiles query tile g visits: all of them, or when causal those up to its diagonal (a causal
  // call has as many key tiles as query tiles; the second tile of the last CTA may not exist, it
  // then repeats the first one's range and stores nothing).  The producer loads the longer range.
  long long Nq_live = a.Nq, Nk_live = a.N, o_first = (bh / a.Hq) * a.o_sb;   // live lengths; first element of this batch entry's output
  if (VARLEN) {
    const long long b = bh / a.Hq;
    // clamped to the packed tensors: whatever the arrays hold, no row outside `out` is written
    const long long q0 = min(max((long long)__ldg(a.cu_q + b), 0LL), a.Tq), k0 = min(max((long long)__ldg(a.cu_k + b), 0LL), a.Tk);
    Nq_live = min(max(min((long long)__ldg(a.cu_q + b + 1), a.Tq) - q0, 0LL), a.Nq);
    Nk_live = min(max(min((long long)__ldg(a.cu_k + b + 1), a.Tk) - k0, 0LL), a.N);
    o_first = q0 * a.o_sr;
    if ((long long)q_tile0 * TILE >= Nq_live) return;       // before any barrier or TMEM column exists
    if (Nk_live == 0) {                                     // queries without keys: rows of zeros
      const long long h = bh % a.Hq;
      for (int i = tid; i < NQ * TILE * (a.D / 2); i += (int)blockDim.x) {
        const long long row = (long long)q_tile0 * TILE + i / (a.D / 2);
        if (row < Nq_live)
          *reinterpret_cast<uint32_t*>(reinterpret_cast<OutT*>(a.out) + o_first + h * a.o_sh + row * a.o_sr + 2 * (i % (a.D / 2))) = 0u;
      }
      return;
    }
  }
  const int key_tiles = VARLEN ? (int)((Nk_live + TILE - 1) / TILE) : (int)(a.N_pad / TILE);
  auto tiles_of = [&](int g) { return CAUSAL ? min(q_tile0 + g + 1, key_tiles) : key_tiles; };
  const int n_load = tiles_of(NQ - 1);

  if (tid == 0) {
    mbar_init(bar(BAR_Q), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(BAR_KF + s), 1);
      mbar_init(bar(BAR_KE + s), NQ);                       // every query tile's Q.K^T of the stage is complete
      mbar_init(bar(BAR_VF + s), 1);
      mbar_init(bar(BAR_VE + s), NQ);
    }
    for (int g = 0; g < NQ; ++g) {
      mbar_init(bar(BAR_SF + BAR_PER_TILE * g), 1);
      mbar_init(bar(BAR_SFREE + BAR_PER_TILE * g), 8);
      mbar_init(bar(BAR_PF + BAR_PER_TILE * g), 8);
      mbar_init(bar(BAR_PV + BAR_PER_TILE * g), 1);
    }
    misc[1] = (*reinterpret_cast<volatile int32_t*>(a.status) != 0) ? 1u : 0u;
    if (FAST) { misc[4] = 0u; misc[5] = 0u; misc[6] = 0u; misc[7] = 0u; }   // skipped-warp counts, see the MMA issuer
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(base + OFF_MISC), "r"(L::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  const bool skip_all = misc[1] != 0u;

  // Registers move from the producer/MMA warpgroup to the softmax warpgroups:
  // 384 x 80 at launch = 128 x 32 + 256 x 104 afterwards (NQ = 2: 640 x 96 = 128 x 32 + 512 x 112).
  // setmaxnreg.inc blocks until the pool holds the registers it asks for, so the two sides must
  // never add up to more than the launch allocation.
  static_assert(128 * L::REGS_PRODUCER + 256 * NQ * L::REGS_SOFTMAX <= L::THREADS * L::REGS_AT_LAUNCH,
                "setmaxnreg.inc would wait for registers that never become free");
  if (!skip_all) {
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(L::REGS_PRODUCER));
    }
    if (NQ == 2 && warp < 4) {
      // Two query tiles: the four product streams of a key tile go to the four warps of this
      // warpgroup, one per scheduler (issuing tcgen05.mma and commits holds up the issuing warp's
      // scheduler, and the softmax warps on the most loaded scheduler set the pace).  There is no
      // separate producer: the threads of query tile 1, which runs behind tile 0, also load the
      // next K tile (after their Q.K^T) and the next V tile (after their P.V), when both tiles'
      // products on the stage have completed.
      if (lane == 0) {
        const int g = warp & 1, gb = BAR_PER_TILE * g;
        const int n_tiles = tiles_of(g);
        bool ok = true;
        if (warp < 2) {
          // ------------------------------- Q.K^T issuers ---------------------------
          constexpr uint32_t IDESC_QK = INT8 ? IDESC_I8 : IDESC_F8;
          const float* sk_row = a.sk + (size_t)bh_kv * a.N_pad;
          const float* sv_row = a.svp + (size_t)bh_kv * a.N_pad;
          auto load_k = [&](int j) -> bool {
            const int s = j & 1;
            const uint32_t par = ((uint32_t)(j >> 1) & 1u) ^ 1u;
            if (!mbar_wait(bar(BAR_KE + s), par, cta_abort, a.status, ST_TIMEOUT_PRODUCER)) return false;
            mbar_expect_tx(bar(BAR_KF + s), TILE_BYTES + 2 * VEC_BYTES);
            tma_load_3d(base + OFF_K + s * TILE_BYTES, &tm_k, bar(BAR_KF + s), 0, j * TILE, bh_kv);
            bulk_load(base + OFF_SK + (j & 3) * VEC_BYTES, sk_row + (size_t)j * TILE, VEC_BYTES, bar(BAR_KF + s));
            bulk_load(base + OFF_SV + (j & 3) * VEC_BYTES, sv_row + (size_t)j * TILE, VEC_BYTES, bar(BAR_KF + s));
            return true;
          };
          if (warp == 0) {
            prefetch_map(&tm_q); prefetch_map(&tm_k); prefetch_map(&tm_v);
            mbar_expect_tx(bar(BAR_Q), NQ * TILE_BYTES);
            for (int t = 0; t < NQ; ++t)                        // rows past the last query arrive as zeros
              tma_load_3d(base + OFF_Q + t * TILE_BYTES, &tm_q, bar(BAR_Q), 0, (q_tile0 + t) * TILE, bh);
          } else {
            ok = load_k(0);
            if (ok && n_load > 1) ok = load_k(1);
          }
          if (ok) ok = mbar_wait(bar(BAR_Q), 0, cta_abort, a.status, ST_TIMEOUT_MMA);
          for (int j = 0; ok && j < n_tiles; ++j) {
            const int s = j & 1;
            ok = mbar_wait(bar(BAR_KF + s), (uint32_t)(j >> 1) & 1u, cta_abort, a.status, ST_TIMEOUT_MMA);
            if (ok && j > 0) ok = mbar_wait(bar(BAR_SFREE + gb), (uint32_t)(j - 1) & 1u, cta_abort, a.status, ST_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_ss<INT8>(tmem + L::tmem_s(g), kmajor_sw128_desc(base + OFF_Q + g * TILE_BYTES + 32 * k),
                           kmajor_sw128_desc(base + OFF_K + s * TILE_BYTES + 32 * k), IDESC_QK, k > 0);
            tc_commit(bar(BAR_KE + s));
            tc_commit(bar(BAR_SF + gb));
            if (warp == 1 && j + 2 < n_load) ok = load_k(j + 2);
          }
        } else {
          // ------------------------------- P.V issuers -----------------------------
          auto load_v = [&](int j) -> bool {
            const int sv = j % L::V_STAGES;
            const uint32_t parv = ((uint32_t)(j / L::V_STAGES) & 1u) ^ 1u;
            if (!mbar_wait(bar(BAR_VE + sv), parv, cta_abort, a.status, ST_TIMEOUT_PRODUCER)) return false;
            mbar_expect_tx(bar(BAR_VF + sv), TILE_BYTES);
            tma_load_3d(base + OFF_V + sv * TILE_BYTES, &tm_v, bar(BAR_VF + sv), j * TILE, 0, bh_kv);
            return true;
          };
          if (warp == 3) {
            for (int j = 0; ok && j < L::V_STAGES && j < n_load; ++j) ok = load_v(j);
          }
          for (int jj = 0; ok && jj < n_tiles; ++jj) {
            const int s = jj % L::V_STAGES;
            ok = mbar_wait(bar(BAR_VF + s), (uint32_t)(jj / L::V_STAGES) & 1u, cta_abort, a.status, ST_TIMEOUT_MMA);
            if (ok) ok = mbar_wait(bar(BAR_PF + gb), (uint32_t)jj & 1u, cta_abort, a.status, ST_TIMEOUT_MMA);
            if (!ok) break;
            bool all_zero = false;
            if (FAST) {
              volatile uint32_t* cnt = misc + 4 + 2 * g + (jj & 1);
              const uint32_t c8 = *cnt;
              if (c8 != 0u) *cnt = 0u;
              all_zero = (c8 == 8u);
            }
            tc_fence_after();
            if (!all_zero)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_ss<false>(tmem + L::tmem_o(g),
                            kmajor_nosw_desc(base + OFF_P + (g * L::P_BUFS + (jj & (L::P_BUFS - 1))) * TILE_BYTES + 256 * k),
                            kmajor_sw128_desc(base + OFF_V + s * TILE_BYTES + 32 * k), IDESC_F8,
                            (jj > 0 || k > 0) ? 1u : 0u);
            tc_commit(bar(BAR_VE + s));
            tc_commit(bar(BAR_PV + gb));
            if (warp == 3 && jj + L::V_STAGES < n_load) ok = load_v(jj + L::V_STAGES);
          }
        }
      }
    } else if (warp == 0) {
      // ------------------------------- TMA producer (one query tile per CTA) ------
      if (lane == 0) {
        prefetch_map(&tm_q); prefetch_map(&tm_k); prefetch_map(&tm_v);
        mbar_expect_tx(bar(BAR_Q), NQ * TILE_BYTES);
        for (int g = 0; g < NQ; ++g)                          // rows past the last query arrive as zeros
          tma_load_3d(base + OFF_Q + g * TILE_BYTES, &tm_q, bar(BAR_Q), 0, (q_tile0 + g) * TILE, bh);
        const float* sk_row = a.sk + (size_t)bh_kv * a.N_pad;
        const float* sv_row = a.svp + (size_t)bh_kv * a.N_pad;
        auto load_k = [&](int j) -> bool {
          const int s = j & 1;
          const uint32_t par = ((uint32_t)(j >> 1) & 1u) ^ 1u;
          if (!mbar_wait(bar(BAR_KE + s), par, cta_abort, a.status, ST_TIMEOUT_PRODUCER)) return false;
          // The tile's scale rows ride on the K barrier into a 4-slot ring: slot j&3 is rewritten
          // only after QK(j+2) has completed, which needs every softmax warp to be past tile j.
          mbar_expect_tx(bar(BAR_KF + s), TILE_BYTES + 2 * VEC_BYTES);
          tma_load_3d(base + OFF_K + s * TILE_BYTES, &tm_k, bar(BAR_KF + s), 0, j * TILE, bh_kv);
          bulk_load(base + OFF_SK + (j & 3) * VEC_BYTES, sk_row + (size_t)j * TILE, VEC_BYTES, bar(BAR_KF + s));
          bulk_load(base + OFF_SV + (j & 3) * VEC_BYTES, sv_row + (size_t)j * TILE, VEC_BYTES, bar(BAR_KF + s));
          return true;
        };
        bool ok = true;
        for (int j = 0; ok && j < L::K_AHEAD && j < n_load; ++j) ok = load_k(j);
        for (int j = 0; ok && j < n_load; ++j) {
          if (j + L::K_AHEAD < n_load && !load_k(j + L::K_AHEAD)) break;
          const int sv = j % L::V_STAGES;
          const uint32_t parv = ((uint32_t)(j / L::V_STAGES) & 1u) ^ 1u;
          if (!mbar_wait(bar(BAR_VE + sv), parv, cta_abort, a.status, ST_TIMEOUT_PRODUCER)) break;
          mbar_expect_tx(bar(BAR_VF + sv), TILE_BYTES);
          tma_load_3d(base + OFF_V + sv * TILE_BYTES, &tm_v, bar(BAR_VF + sv), j * TILE, 0, bh_kv);
        }
      }
    } else if (warp == 1) {
      // ------------------------------- MMA issuer (one query tile per CTA) --------
      const int g = 0;
      const int gb = BAR_PER_TILE * g;
      const int n_tiles = tiles_of(g);
      if (lane == 0) {
        constexpr uint32_t IDESC_QK = INT8 ? IDESC_I8 : IDESC_F8;
        bool ok = mbar_wait(bar(BAR_Q), 0, cta_abort, a.status, ST_TIMEOUT_MMA);
        for (int j = 0; ok && j <= n_tiles; ++j) {
          if (j < n_tiles) {
            const int s = j & 1;
            ok = mbar_wait(bar(BAR_KF + s), (uint32_t)(j >> 1) & 1u, cta_abort, a.status, ST_TIMEOUT_MMA);
            if (ok && j > 0) ok = mbar_wait(bar(BAR_SFREE + gb), (uint32_t)(j - 1) & 1u, cta_abort, a.status, ST_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_ss<INT8>(tmem + L::tmem_s(g), kmajor_sw128_desc(base + OFF_Q + g * TILE_BYTES + 32 * k),
                           kmajor_sw128_desc(base + OFF_K + s * TILE_BYTES + 32 * k), IDESC_QK, k > 0);
            tc_commit(bar(BAR_KE + s));
            tc_commit(bar(BAR_SF + gb));
          }
          if (j > 0) {
            const int jj = j - 1, s = jj % L::V_STAGES;
            ok = mbar_wait(bar(BAR_VF + s), (uint32_t)(jj / L::V_STAGES) & 1u, cta_abort, a.status, ST_TIMEOUT_MMA);
            if (ok) ok = mbar_wait(bar(BAR_PF + gb), (uint32_t)jj & 1u, cta_abort, a.status, ST_TIMEOUT_MMA);
            if (!ok) break;
            // FAST kernels: a warp that skips a tile counts itself before it arrives at the P
            // barrier.  When all eight warps of the query tile did, P(jj) is all zeros and the
            // product is not issued; the two commits still release the V stage and complete the
            // P.V barrier (the first tile is never skipped, so the accumulator is initialised).
            bool all_zero = false;
            if (FAST) {
              volatile uint32_t* cnt = misc + 4 + 2 * g + (jj & 1);
              const uint32_t c8 = *cnt;
              if (c8 != 0u) *cnt = 0u;
              all_zero = (c8 == 8u);
            }
            tc_fence_after();
            if (!all_zero)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_ss<false>(tmem + L::tmem_o(g),
                            kmajor_nosw_desc(base + OFF_P + (g * L::P_BUFS + (jj & (L::P_BUFS - 1))) * TILE_BYTES + 256 * k),
                            kmajor_sw128_desc(base + OFF_V + s * TILE_BYTES + 32 * k), IDESC_F8,
                            (jj > 0 || k > 0) ? 1u : 0u);
            tc_commit(bar(BAR_VE + s));
            tc_commit(bar(BAR_PV + gb));
          }
        }
      }
    } else if (warp >= 4) {
      // ------------------------------- softmax warps ------------------------------
      // A warp owns 16 TMEM lanes (query rows) and all 128 key columns, read with the 16x256b
      // shape: thread t holds rows r0 = t/4 and r0+8, and of every 8-column group the two columns
      // 2c, 2c+1 (c = t%4).  K8 is stored with its rows permuted inside 16-row blocks so that the
      // four columns a thread holds of a 16-column block are four CONSECUTIVE keys 16m+4c..+3:
      // one 16-byte scale load serves both rows, the four e4m3 codes of a row are one 32-bit word of
      // the P tile, and a row's maximum is two shuffles among the four threads that share it.
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(L::REGS_SOFTMAX));
      const int g = (NQ == 1) ? 0 : (warp - 4) >> 3;        // which query tile of the CTA
      const int gb = BAR_PER_TILE * g;
      const int q_tile = q_tile0 + g;
      const int n_tiles = tiles_of(g);
      const int quarter = warp & 3;                         // TMEM lane quarter this warp may touch
      const int sub = ((warp - 4) >> 2) & 1;                // which 16 lanes of the quarter
      const int r0 = lane >> 2, c = lane & 3;
      const int lane_base = 32 * quarter + 16 * sub;
      const int rowA = lane_base + r0, rowB = rowA + 8;     // this thread's two query rows of the tile
      const long long q_rowA = (long long)q_tile * TILE + rowA, q_rowB = q_rowA + 8;
      const uint32_t t_s = tmem + ((uint32_t)lane_base << 16) + L::tmem_s(g);
      const uint32_t t_o = tmem + ((uint32_t)lane_base << 16) + L::tmem_o(g);
      // c_q = f32(f32(sm_scale * log2e) * sq); rows past N get 1 (their scores are all zero)
      const float sl2 = __fmul_rn(a.sm_scale, LOG2E_F);
      const float cqA = (q_rowA < (VARLEN ? Nq_live : a.Nq)) ? __fmul_rn(sl2, __ldg(a.sq + (size_t)bh * a.Nq + q_rowA)) : 1.f;
      const float cqB = (q_rowB < (VARLEN ? Nq_live : a.Nq)) ? __fmul_rn(sl2, __ldg(a.sq + (size_t)bh * a.Nq + q_rowB)) : 1.f;
      const float2 cqA2 = make_float2(cqA, cqA), cqB2 = make_float2(cqB, cqB);
      float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
      bool ok = true;
      // P tile: 16 keys of row r (chunk m) at (r / 8) * 1024 + m * 128 + (r % 8) * 16, so that the
      // eight stores of a row differ by a constant and a warp's store covers 128 contiguous bytes
      const uint32_t p0 = base + OFF_P + (uint32_t)(g * L::P_BUFS) * TILE_BYTES + (uint32_t)lane_base * 128u +
                          16u * (uint32_t)r0 + 4u * (uint32_t)c;
      const uint32_t sk_c = base + OFF_SK + 16u * (uint32_t)c;   // scales of keys 16m+4c..+3 at + 64m

      // Negligible-tile fast path (kernels instantiated with FAST; the others carry none of it:
      // any addition to the code between the row maxima and the exponentials, even two fused
      // multiply-adds and a vote without a branch, costs 3 to 6 % on inputs where no tile can be
      // skipped, so the host picks the instantiation).  A key tile whose every score lies
      // a.skip_log2 (40) or more below the row's running maximum in the exponent domain, for all
      // 16 rows of the warp, adds exact zeros to P (p * svp < 2^-40 * 448 rounds to the e4m3 zero)
      // and less than 128 * 2^-40 of the row's largest term to its sum.  Such a tile is not
      // exponentiated: the warp's P rows are zeros, the row sums and maxima stay as they are.  Two
      // tests, both upper bounds of the tile's largest exponent formed with the same monotone
      // operations as the exponents themselves:
      //   after the conversion   t <= fma(row max of u, c_q, -c_q*m)
      //   before the conversion  u <= fl(f32(max(row max of S, 0)) * max of the tile's sk)
      // The second, cheaper one is tried when the warp's previous tile was skipped.
      // Warp-uniform state: bit b (b < P_BUFS): this warp's rows of P tile b hold zeros; bit 8:
      // the previous tile was skipped; bit 9: armed; bits 12-15: tests failed since the last skip.
      uint32_t fast = 0;
      constexpr uint32_t TRY_BOUND = 256u, ARMED = 512u, FAIL_ONE = 1u << 12, FAIL_MASK = 15u << 12;
      int n_skipped = 0;                                    // tiles this warp skipped (reported once, at the end)
      // What is left of a skipped tile: zeros for the warp's P rows (unless the tile already holds
      // them), the wait for P.V(j-1) (see the comment at the other copy of this wait below) and
      // the arrival at the P barrier.
      auto finish_skipped = [&](int j) -> bool {
        const uint32_t bit = 1u << (j & (L::P_BUFS - 1));
        if (!(fast & bit)) {
          const uint32_t pA = p0 + (uint32_t)(j & (L::P_BUFS - 1)) * TILE_BYTES, pB = pA + 8u * 128u;
#pragma unroll
          for (int m = 0; m < 8; ++m) { sts32u(pA + 128u * (uint32_t)m, 0u); sts32u(pB + 128u * (uint32_t)m, 0u); }
        }
        fast = (fast & ~FAIL_MASK) | bit | TRY_BOUND | ARMED;
        ++n_skipped;
        if (j > 0) {
          const bool w = mbar_wait(bar(BAR_PV + gb), (uint32_t)(j - 1) & 1u, cta_abort, a.status, ST_TIMEOUT_SOFTMAX);
          if (!__all_sync(0xffffffffu, w)) return false;
          tc_fence_after();
        }
        // (after the wait: P.V(j-1) complete means the MMA thread has read and cleared the count of tile j-2)
        if (lane == 0) atomicAdd(const_cast<uint32_t*>(misc) + 4 + 2 * g + (j & 1), 1u);
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        mbar_arrive_lane0(bar(BAR_PF + gb), lane);
        return true;
      };

      for (int j = 0; j < n_tiles; ++j) {
        // S(j) complete implies the K stage, and with it this tile's scale rows, has landed
        ok = mbar_wait(bar(BAR_SF + gb), (uint32_t)j & 1u, cta_abort, a.status, ST_TIMEOUT_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t acc[64];                                   // acc[8m + {0,1,4,5}]: row A keys +0..3; {2,3,6,7}: row B
        tmem_ld_16x256b_x16(t_s, acc);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        mbar_arrive_lane0(bar(BAR_SFREE + gb), lane);

        const uint32_t skv = sk_c + (uint32_t)(j & 3) * VEC_BYTES;        // this tile's K scales
        const uint32_t svv = skv + (OFF_SV - OFF_SK);                      // and its staged V factors
        if (FAST && (fast & TRY_BOUND)) {
          // largest K scale of the tile: lane l looks at keys 4l..4l+3
          const float4 k4 = lds128(skv - 16u * (uint32_t)c + 16u * (uint32_t)lane);
          float km = max3(fmaxf(k4.x, k4.y), k4.z, k4.w);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) km = fmaxf(km, __shfl_xor_sync(0xffffffffu, km, o));
          float sA, sB;
          if (INT8) {
            int a0 = (int)acc[0], a1 = (int)acc[1], b0 = (int)acc[2], b1 = (int)acc[3];
            a0 = __vimax3_s32(a0, (int)acc[4], (int)acc[5]);
            b0 = __vimax3_s32(b0, (int)acc[6], (int)acc[7]);
#pragma unroll
            for (int m = 1; m < 8; ++m) {
              a0 = __vimax3_s32(a0, (int)acc[8 * m + 0], (int)acc[8 * m + 1]);
              a1 = __vimax3_s32(a1, (int)acc[8 * m + 4], (int)acc[8 * m + 5]);
              b0 = __vimax3_s32(b0, (int)acc[8 * m + 2], (int)acc[8 * m + 3]);
              b1 = __vimax3_s32(b1, (int)acc[8 * m + 6], (int)acc[8 * m + 7]);
            }
            int ia = max(max(a0, a1), 0), ib = max(max(b0, b1), 0);
            ia = max(ia, __shfl_xor_sync(0xffffffffu, ia, 1)); ib = max(ib, __shfl_xor_sync(0xffffffffu, ib, 1));
            ia = max(ia, __shfl_xor_sync(0xffffffffu, ia, 2)); ib = max(ib, __shfl_xor_sync(0xffffffffu, ib, 2));
            sA = (float)ia; sB = (float)ib;
          } else {
            float a0 = __uint_as_float(acc[0]), a1 = __uint_as_float(acc[1]);
            float b0 = __uint_as_float(acc[2]), b1 = __uint_as_float(acc[3]);
            a0 = max3(a0, __uint_as_float(acc[4]), __uint_as_float(acc[5]));
            b0 = max3(b0, __uint_as_float(acc[6]), __uint_as_float(acc[7]));
#pragma unroll
            for (int m = 1; m < 8; ++m) {
              a0 = max3(a0, __uint_as_float(acc[8 * m + 0]), __uint_as_float(acc[8 * m + 1]));
              a1 = max3(a1, __uint_as_float(acc[8 * m + 4]), __uint_as_float(acc[8 * m + 5]));
              b0 = max3(b0, __uint_as_float(acc[8 * m + 2]), __uint_as_float(acc[8 * m + 3]));
              b1 = max3(b1, __uint_as_float(acc[8 * m + 6]), __uint_as_float(acc[8 * m + 7]));
            }
            sA = max3(a0, a1, 0.f); sB = max3(b0, b1, 0.f);
            sA = fmaxf(sA, __shfl_xor_sync(0xffffffffu, sA, 1)); sB = fmaxf(sB, __shfl_xor_sync(0xffffffffu, sB, 1));
            sA = fmaxf(sA, __shfl_xor_sync(0xffffffffu, sA, 2)); sB = fmaxf(sB, __shfl_xor_sync(0xffffffffu, sB, 2));
          }
          // (a maximum that is still -inf makes the bound +inf: the comparison fails)
          const float tA = __fmaf_rn(__fmul_rn(sA, km), cqA, -(cqA * mA));
          const float tB = __fmaf_rn(__fmul_rn(sB, km), cqB, -(cqB * mB));
          if (__all_sync(0xffffffffu, fmaxf(tA, tB) <= -a.skip_log2)) {
            ok = finish_skipped(j);
            if (!ok) break;
            continue;
          }
          fast &= ~TRY_BOUND;
        }
        float2 uA[16], uB[16];                              // u[2m], u[2m+1]: keys 16m+4c+{0,1}, +{2,3} (times sk)
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const float4 kk = lds128(skv + 64 * m);
          float a0, a1, a2, a3, b0, b1, b2, b3;
          if (INT8) {
            a0 = (float)(int)acc[8 * m + 0]; a1 = (float)(int)acc[8 * m + 1];
            b0 = (float)(int)acc[8 * m + 2]; b1 = (float)(int)acc[8 * m + 3];
            a2 = (float)(int)acc[8 * m + 4]; a3 = (float)(int)acc[8 * m + 5];
            b2 = (float)(int)acc[8 * m + 6]; b3 = (float)(int)acc[8 * m + 7];
          } else {
            a0 = __uint_as_float(acc[8 * m + 0]); a1 = __uint_as_float(acc[8 * m + 1]);
            b0 = __uint_as_float(acc[8 * m + 2]); b1 = __uint_as_float(acc[8 * m + 3]);
            a2 = __uint_as_float(acc[8 * m + 4]); a3 = __uint_as_float(acc[8 * m + 5]);
            b2 = __uint_as_float(acc[8 * m + 6]); b3 = __uint_as_float(acc[8 * m + 7]);
          }
          const float2 k01 = make_float2(kk.x, kk.y), k23 = make_float2(kk.z, kk.w);
          uA[2 * m + 0] = __fmul2_rn(make_float2(a0, a1), k01);
          uA[2 * m + 1] = __fmul2_rn(make_float2(a2, a3), k23);
          uB[2 * m + 0] = __fmul2_rn(make_float2(b0, b1), k01);
          uB[2 * m + 1] = __fmul2_rn(make_float2(b2, b3), k23);
        }
        // Tile-uniform mask: the diagonal tile when causal, the ragged last tile otherwise.
        if (CAUSAL) {
          if (j == q_tile) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int key = 16 * (i >> 1) + 4 * c + 2 * (i & 1);        // tile-local key of u[i].x
              if (key > rowA) uA[i].x = -INFINITY;
              if (key + 1 > rowA) uA[i].y = -INFINITY;
              if (key > rowB) uB[i].x = -INFINITY;
              if (key + 1 > rowB) uB[i].y = -INFINITY;
            }
          }
        } else {
          if ((long long)(j + 1) * TILE > (VARLEN ? Nk_live : a.N)) {
            const int live = (int)((VARLEN ? Nk_live : a.N) - (long long)j * TILE);   // tile-local key >= live is masked
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int key = 16 * (i >> 1) + 4 * c + 2 * (i & 1);
              if (key >= live) { uA[i].x = -INFINITY; uB[i].x = -INFINITY; }
              if (key + 1 >= live) { uA[i].y = -INFINITY; uB[i].y = -INFINITY; }
            }
          }
        }
        float xa0 = uA[0].x, xa1 = uA[0].y, xb0 = uB[0].x, xb1 = uB[0].y;
#pragma unroll
        for (int i = 1; i < 16; i += 2) {
          xa0 = max3(xa0, uA[i].x, uA[i].y);
          xb0 = max3(xb0, uB[i].x, uB[i].y);
          if (i + 1 < 16) {
            xa1 = max3(xa1, uA[i + 1].x, uA[i + 1].y);
            xb1 = max3(xb1, uB[i + 1].x, uB[i + 1].y);
          }
        }
        float mxA = fmaxf(xa0, xa1), mxB = fmaxf(xb0, xb1);
        // the four threads of a row are the four lanes that differ in their low two bits
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
        const float mA_new = fmaxf(mA, mxA), mB_new = fmaxf(mB, mxB);
        const float mA_use = (mA_new == -INFINITY) ? 0.f : mA_new;
        const float mB_use = (mB_new == -INFINITY) ? 0.f : mB_new;
        float alphaA, alphaB;
        bool rescale;
        if (FAST && ((fast & ARMED) || (j & 3) == 0)) {
          // The first test.  A warp that has not skipped a tile lately makes it on every fourth
          // tile only (the vote holds up the exponentials); one skipped tile arms it for every
          // tile, sixteen tests failed in a row disarm it.
          // One vote for both questions: bit 0 "a maximum moved", bit 1 "a row of mine has an
          // exponent above the threshold".
          const unsigned votes = __reduce_or_sync(0xffffffffu, ((mA_new > mA) || (mB_new > mB) ? 1u : 0u) |
              (fmaxf(__fmaf_rn(mxA, cqA, -(cqA * mA_use)), __fmaf_rn(mxB, cqB, -(cqB * mB_use))) <= -a.skip_log2 ? 0u : 2u));
          if (!(votes & 2u)) {
            ok = finish_skipped(j);
            if (!ok) break;
            continue;
          }
          if (fast & ARMED) { fast += FAIL_ONE; if ((fast & FAIL_MASK) == FAIL_MASK) fast &= ~(ARMED | FAIL_MASK); }
          alphaA = ex2(cqA * (mA - mA_use)); alphaB = ex2(cqB * (mB - mB_use));
          rescale = (j > 0) && (votes & 1u);
        } else {
          alphaA = ex2(cqA * (mA - mA_use)); alphaB = ex2(cqB * (mB - mB_use));
          // The accumulator is rescaled after the exponentials, when the score registers are
          // free; PV(j) is not issued before this warp arrives.
          rescale = (j > 0) && __any_sync(0xffffffffu, (mA_new > mA) || (mB_new > mB));
        }
        mA = mA_new; mB = mB_new;

        const uint32_t pA = p0 + (uint32_t)(j & (L::P_BUFS - 1)) * TILE_BYTES, pB = pA + 8u * 128u;
        const float nmA = -(cqA * mA_use), nmB = -(cqB * mB_use);
        const float2 nmA2 = make_float2(nmA, nmA), nmB2 = make_float2(nmB, nmB);
        float2 psA = make_float2(0.f, 0.f), psB = make_float2(0.f, 0.f);
#pragma unroll
        for (int m = 0; m < 8; ++m) {                       // 16 keys = one 16-byte chunk of a P row; 4 of them here
          const float4 vv = lds128(svv + 64 * m);
          const float2 v01 = make_float2(vv.x, vv.y), v23 = make_float2(vv.z, vv.w);
          {
            const float2 t0 = __ffma2_rn(uA[2 * m + 0], cqA2, nmA2);
            const float2 t1 = __ffma2_rn(uA[2 * m + 1], cqA2, nmA2);
            const float2 p01 = make_float2(ex2(t0.x), ex2(t0.y));
            const float2 p23 = make_float2(ex2(t1.x), ex2(t1.y));
            psA = __fadd2_rn(psA, __fadd2_rn(p01, p23));
            const float2 f01 = __fmul2_rn(p01, v01), f23 = __fmul2_rn(p23, v23);
            sts32u(pA + 128u * (uint32_t)m, e4m3x4_pack(f01.x, f01.y, f23.x, f23.y));
          }
          {
            const float2 t0 = __ffma2_rn(uB[2 * m + 0], cqB2, nmB2);
            const float2 t1 = __ffma2_rn(uB[2 * m + 1], cqB2, nmB2);
            const float2 p01 = make_float2(ex2(t0.x), ex2(t0.y));
            const float2 p23 = make_float2(ex2(t1.x), ex2(t1.y));
            psB = __fadd2_rn(psB, __fadd2_rn(p01, p23));
            const float2 f01 = __fmul2_rn(p01, v01), f23 = __fmul2_rn(p23, v23);
            sts32u(pB + 128u * (uint32_t)m, e4m3x4_pack(f01.x, f01.y, f23.x, f23.y));
          }
        }
        lA = lA * alphaA + (psA.x + psA.y);                 // this thread's quarter of the row sum
        lB = lB * alphaB + (psB.x + psB.y);
        if (FAST) fast &= ~(1u << (j & (L::P_BUFS - 1)));
        // P.V(j-1) must be complete before the accumulator is rescaled.  The wait sits behind the
        // exponentials, where it does not stall: P(j) went to the tile that P.V(j-2) read, and that
        // product was waited for in the previous iteration.  It is made on every tile, rescaling
        // or not: it also keeps this warp from arriving at the P barrier of tile j before the MMA
        // thread has seen the barrier of tile j-1 complete (P.V(j-1) is issued after that), and
        // the MMA thread's parity wait cannot tell a barrier that is two phases ahead.
        if (j > 0) {
          ok = mbar_wait(bar(BAR_PV + gb), (uint32_t)(j - 1) & 1u, cta_abort, a.status, ST_TIMEOUT_SOFTMAX);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
        }
        if (rescale) {
          const float2 aA2 = make_float2(alphaA, alphaA), aB2 = make_float2(alphaB, alphaB);
          uint32_t o[64];
          tmem_ld_16x256b_x16(t_o, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 ra = __fmul2_rn(make_float2(__uint_as_float(o[4 * i + 0]), __uint_as_float(o[4 * i + 1])), aA2);
            const float2 rb = __fmul2_rn(make_float2(__uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3])), aB2);
            o[4 * i + 0] = __float_as_uint(ra.x); o[4 * i + 1] = __float_as_uint(ra.y);
            o[4 * i + 2] = __float_as_uint(rb.x); o[4 * i + 3] = __float_as_uint(rb.y);
          }
          tmem_st_16x256b_x16(t_o, o);
          tmem_st_wait();
        }
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        mbar_arrive_lane0(bar(BAR_PF + gb), lane);
      }

      if (FAST && a.skipped != nullptr && lane == 0 && n_skipped > 0) atomicAdd(a.skipped, (unsigned)n_skipped);

      // ------------------------------- epilogue -----------------------------------
      if (ok) {
        ok = mbar_wait(bar(BAR_PV + gb), (uint32_t)(n_tiles - 1) & 1u, cta_abort, a.status, ST_TIMEOUT_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        // total row sums: the four quarters were scaled with the same running maximum
        lA += __shfl_xor_sync(0xffffffffu, lA, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 1);
        lA += __shfl_xor_sync(0xffffffffu, lA, 2); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
        const float S = __ldg(a.s_fold + bh_kv);
        const float invA = (lA > 0.f) ? __fdiv_rn(S, __fmul_rn(lA, F8_MAX)) : 0.f;
        const float invB = (lB > 0.f) ? __fdiv_rn(S, __fmul_rn(lB, F8_MAX)) : 0.f;
        const long long b = bh / a.Hq, h = bh - b * a.Hq;
        if (a.lse != nullptr && c == 0) {
          // ln sum_k exp(q.k*sm_scale) = ln2 * (c_q*m + log2 l) (+ q.mean*sm_scale with smooth_k)
          if (q_rowA < (VARLEN ? Nq_live : a.Nq)) {
            float v = (lA > 0.f) ? 0.6931471805599453f * (cqA * mA + log2f(lA)) : -INFINITY;
            if (a.qm != nullptr) v += a.sm_scale * __ldg(a.qm + (size_t)bh * a.Nq + q_rowA);
            a.lse[(size_t)bh * a.Nq + q_rowA] = v;
          }
          if (q_rowB < (VARLEN ? Nq_live : a.Nq)) {
            float v = (lB > 0.f) ? 0.6931471805599453f * (cqB * mB + log2f(lB)) : -INFINITY;
            if (a.qm != nullptr) v += a.sm_scale * __ldg(a.qm + (size_t)bh * a.Nq + q_rowB);
            a.lse[(size_t)bh * a.Nq + q_rowB] = v;
          }
        }
        OutT* orowA = reinterpret_cast<OutT*>(a.out) + (VARLEN ? o_first : b * a.o_sb) + h * a.o_sh + q_rowA * a.o_sr + 2 * c;
        OutT* orowB = orowA + 8 * a.o_sr;
        const float* vm = (a.vmean != nullptr) ? a.vmean + (size_t)bh_kv * HD + 2 * c : nullptr;
        uint32_t o[64];
        tmem_ld_16x256b_x16(t_o, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {                      // channels 8i + 2c, 8i + 2c + 1
          if (8 * i + 2 * c < a.D) {
            float fa0 = __uint_as_float(o[4 * i + 0]) * invA, fa1 = __uint_as_float(o[4 * i + 1]) * invA;
            float fb0 = __uint_as_float(o[4 * i + 2]) * invB, fb1 = __uint_as_float(o[4 * i + 3]) * invB;
            if (vm != nullptr) {                            // smooth_v: the rows of P sum to one, so add the mean back
              const float2 mu = __ldg(reinterpret_cast<const float2*>(vm + 8 * i));
              fa0 += mu.x; fa1 += mu.y; fb0 += mu.x; fb1 += mu.y;
            }
            if (q_rowA < (VARLEN ? Nq_live : a.Nq)) *reinterpret_cast<uint32_t*>(orowA + 8 * i) = pack2<OutT>(fa0, fa1);
            if (q_rowB < (VARLEN ? Nq_live : a.Nq)) *reinterpret_cast<uint32_t*>(orowB + 8 * i) = pack2<OutT>(fb0, fb1);
          }
        }
      }
    }
  }

  // Teardown: every role has left its loop (all waits are bounded).  After a failure give copies
  // still in flight a moment to land before the shared memory is released.
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 400000) { }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(L::TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// Host side: tensor maps and launch.
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

// 3-D map over one-byte codes: dims (inner, rows, heads), box 128 x 128 x 1, 128-byte swizzle,
// out-of-range elements read as zero.
static bool make_map(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t rows, uint64_t heads,
                     uint64_t row_stride_bytes, uint64_t head_stride_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {inner, rows, heads};
  cuuint64_t strides[2] = {row_stride_bytes, head_stride_bytes};
  cuuint32_t box[3] = {128, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Test hook: 1 or 2 forces that kernel shape for later launches, 0 leaves the choice to
// choose_tiles_per_cta.  One relaxed atomic word; launches that race with a change take either value.
static std::atomic<int> g_force_tiles_per_cta{0};
void set_tiles_per_cta(int n) { g_force_tiles_per_cta.store((n == 1 || n == 2) ? n : 0, std::memory_order_relaxed); }
// Test hook: the threshold of the negligible-tile fast path in log2 units (0 switches the path
// off, a negative value restores the default).
constexpr float SKIP_LOG2_DEFAULT = 40.f;
static std::atomic<float> g_skip_log2{SKIP_LOG2_DEFAULT};
void set_skip_log2(float t) { g_skip_log2.store(t < 0.f ? SKIP_LOG2_DEFAULT : t, std::memory_order_relaxed); }

template <bool INT8, bool CAUSAL, typename OutT, int NQ, bool FAST, bool VARLEN = false>
static cudaError_t launch_inst(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                               const AttnKArgs& ka, dim3 grid, cudaStream_t st) {
  auto kern = attn_fwd_kernel<INT8, CAUSAL, OutT, NQ, FAST, VARLEN>;
  using L = Shape<NQ>;
  // the opt-in to more than 48 KB of dynamic shared memory is per device and per instantiation;
  // it is made once (short calls are dominated by host-side work)
  static bool opted_in[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !opted_in[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    // The register hand-over inside the kernel assumes the allocation the compiler reported; a
    // build that came out with fewer registers per thread would leave setmaxnreg.inc waiting.
    cudaFuncAttributes attr;
    e = cudaFuncGetAttributes(&attr, kern);
    if (e != cudaSuccess) return e;
    if (attr.numRegs * L::THREADS < 128 * L::REGS_PRODUCER + 256 * NQ * L::REGS_SOFTMAX) return cudaErrorLaunchOutOfResources;
    if (dev >= 0 && dev < 64) opted_in[dev] = true;
  }
  return launch_after_predecessor(kern, grid, dim3(L::THREADS), L::SMEM_BYTES, st, mq, mk, mv, ka);
}

// Which shape: query tiles per CTA for a call of `q_tiles` x `bhq` query tiles on `sms` SMs.
// A two-tile CTA does the work of two one-tile CTAs in about 0.955 of the time the two take side
// by side on an SM (measured 0.91-0.98), but it is handed out in units twice as large.  Non-causal CTAs
// all take the same time, so the count of rounds decides: one-tile CTAs go round in half-SM
// units (ceil(S / SMs) / 2 rounds for S CTAs), two-tile CTAs in whole ones (ceil(P / SMs) rounds
// for P = about S / 2); a call that is resident at once either way is faster with two tiles.
// Causal CTAs differ in length and even out by themselves; they take two tiles once there is
// such a CTA for every SM.
int choose_tiles_per_cta(int64_t q_tiles, int64_t bhq, bool causal, int sms) {
  if (q_tiles < 2 || bhq < 1 || sms < 1) return 1;
  const uint64_t n_one = (uint64_t)q_tiles * (uint64_t)bhq, n_two = (uint64_t)((q_tiles + 1) / 2) * (uint64_t)bhq;
  if (causal) return n_two >= (uint64_t)sms ? 2 : 1;
  if (n_one <= 2 * (uint64_t)sms) return 2;
  const double rounds_one = 0.5 * (double)((n_one + sms - 1) / sms);
  const double rounds_two = 0.955 * (double)((n_two + sms - 1) / sms);
  return rounds_two <= rounds_one ? 2 : 1;
}

cudaError_t launch_attention(const AttnParams& p, cudaStream_t st, const char** why) {
  const uint64_t bh = (uint64_t)(p.B * p.H), N_pad = (uint64_t)p.N_pad;
  const uint64_t bhq = (uint64_t)(p.B * p.Hq), Nq = (uint64_t)p.Nq;
  CUtensorMap mq, mk, mv;
  if (!make_map(&mq, p.q8, HD, Nq, bhq, HD, Nq * HD) ||
      !make_map(&mk, p.k8, HD, N_pad, bh, HD, N_pad * HD) ||
      !make_map(&mv, p.v8t, N_pad, HD, bh, N_pad, N_pad * HD)) {
    if (why) *why = "cuTensorMapEncodeTiled failed (driver entry point missing or bad operand layout)";
    return cudaErrorInvalidValue;
  }
  AttnKArgs ka;
  ka.sq = p.sq; ka.sk = p.sk; ka.svp = p.svp; ka.s_fold = p.s_fold; ka.out = p.out;
  ka.N = p.N; ka.N_pad = p.N_pad; ka.H = p.H;
  ka.Nq = p.Nq; ka.Hq = p.Hq; ka.group = p.Hq / p.H; ka.lse = p.lse; ka.qm = p.qm; ka.D = (int)p.D; ka.vmean = p.vmean;
  ka.o_sb = p.o_strides[0]; ka.o_sh = p.o_strides[1]; ka.o_sr = p.o_strides[2];
  ka.sm_scale = p.sm_scale; ka.status = p.status;
  const unsigned q_tiles = (unsigned)((p.Nq + TILE - 1) / TILE);
  static int sm_count[64] = {0};                          // per device, asked once
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
    if (sm_count[dev] == 0 &&
        cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sm_count[dev] = 148;
    sms = sm_count[dev];
  }
  bool two = choose_tiles_per_cta((int64_t)q_tiles, (int64_t)bhq, p.causal != 0, sms) == 2;
  const int forced = g_force_tiles_per_cta.load(std::memory_order_relaxed);
  if (forced != 0) two = (forced == 2);
  // A packed batch runs on the one-tile kernels without the negligible-tile tests: its sequences
  // differ in length, and the smaller unit of work evens them out.
  const bool varlen = p.cu_q != nullptr;
  ka.cu_q = p.cu_q; ka.cu_k = p.cu_k; ka.Tq = p.Tq; ka.Tk = p.Tk;
  if (varlen) two = false;
  dim3 grid(two ? (q_tiles + 1) / 2 : q_tiles, (unsigned)bhq);
  // Which of the two sets of kernels: with the negligible-tile tests (the default) or without.
  // The threshold hook at 0 and the caller's `no_fast_path` both select the plain set.
  const float skip = g_skip_log2.load(std::memory_order_relaxed);
  const bool fast = !p.no_fast_path && skip > 0.f && !varlen;
  ka.skip_log2 = skip;
  ka.skipped = fast ? p.skipped : nullptr;
  const int key = (p.qk_mode == 0 ? 4 : 0) | (p.causal ? 2 : 0) | (p.out_dtype == 0 ? 1 : 0);
  cudaError_t e;
#define SAGE_LAUNCH(I8, C, T)                                                                          \
  e = varlen ? launch_inst<I8, C, T, 1, false, true>(mq, mk, mv, ka, grid, st) :                       \
      two ? (fast ? launch_inst<I8, C, T, 2, true>(mq, mk, mv, ka, grid, st)                           \
                  : launch_inst<I8, C, T, 2, false>(mq, mk, mv, ka, grid, st))                         \
          : (fast ? launch_inst<I8, C, T, 1, true>(mq, mk, mv, ka, grid, st)                           \
                  : launch_inst<I8, C, T, 1, false>(mq, mk, mv, ka, grid, st))
  switch (key) {
    case 7: SAGE_LAUNCH(true, true, __half); break;
    case 6: SAGE_LAUNCH(true, true, __nv_bfloat16); break;
    case 5: SAGE_LAUNCH(true, false, __half); break;
    case 4: SAGE_LAUNCH(true, false, __nv_bfloat16); break;
    case 3: SAGE_LAUNCH(false, true, __half); break;
    case 2: SAGE_LAUNCH(false, true, __nv_bfloat16); break;
    case 1: SAGE_LAUNCH(false, false, __half); break;
    default: SAGE_LAUNCH(false, false, __nv_bfloat16); break;
  }
#undef SAGE_LAUNCH
  if (e != cudaSuccess && why) *why = "attention kernel launch failed";
  return e;
}

}  // namespace sage
