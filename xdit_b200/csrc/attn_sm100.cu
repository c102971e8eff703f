// Flash-attention forward for sm_100a: tcgen05.mma with TMEM accumulators, operands staged by
// TMA, warp-specialised online softmax.  bf16/fp16, head_dim a multiple of 8 up to 128.
//
// One CTA owns two query tiles of 128 rows and walks all key/value tiles of 128 rows -- or, when the
// launch is too small to fill the GPU, its share of them: the keys are then split over several CTAs per
// pair of query tiles, every CTA writes a normalised fp32 partial result with its log-sum-exp, and
// split_merge_kernel combines the partials into the output.
//   warps 0-3  softmax group for query tile 0   (one thread per query row)
//   warps 4-7  softmax group for query tile 1
//   warp  8    issues every tcgen05.mma (the warp runs converged, one elected lane issues) and owns
//               the TMEM allocation
//   warp  9    issues every TMA load (one lane)
//   warps 10-11 idle: they complete the warpgroup that hands its registers to the softmax warps
//               (setmaxnreg: 40 registers for warps 8-11, 232 for warps 0-7)
// The tensor core alternates between the two query tiles, so that one tile's softmax runs while
// the other tile's S = Q K^T and O += P V are in flight.
//
// TMEM (512 columns x 128 lanes, fp32):  S0 [0,128)  S1 [128,256)  O0 [256,384)  O1 [384,512).
// P (bf16/fp16, two per column) overwrites columns [0,64) of its S tile and is fed to the second
// GEMM as the A operand straight from TMEM.
//
// Shared memory: Q 2 tiles, then a ring of K/V stages (K0,V0,K1,V1,...).  Every tile is stored
// as head_dim slabs of 64 elements: slab s holds [rows][64] with 128-byte rows in the 128-byte
// swizzle, which is both what a TMA box {64 elements, 64 rows} writes and what the UMMA
// descriptors read (K-major for Q and K, MN-major for V).
//
// Sequences are lists of 64-row chunks: a tensor after a Ulysses all-to-all is `nseg` segments
// (one per source rank) and each segment is cut into chunks of its own, the joint (text) K/V
// follow as a second tensor map.  Rows past a segment's end are zero-filled by TMA and masked
// to -inf before the softmax.  Because keys may be visited in any order, no re-layout copy is
// needed between the all-to-all and this kernel.
//
// Every wait on an mbarrier is bounded in time; when one gives up the CTA raises a flag in
// shared memory, all roles leave their loops, outstanding copies and MMAs are drained with
// bounded waits, TMEM is freed and *status is set.
#include <cuda.h>

#include <cmath>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace xdit {
namespace {

constexpr int kChunk = 64;
constexpr int kTile = 128;
constexpr int kThreads = 384;  // 8 softmax warps, MMA warp, TMA warp, 2 idle warps (full register-trading warpgroup)
constexpr int kSlabBytes = kTile * 128;       // one 64-element slab of a 128-row tile
constexpr int kBoxBytes = kChunk * 128;       // one TMA box: 64 rows x 64 elements
constexpr uint32_t kWaitLimitNs = 200000000u;  // default 0.2 s: no legitimate wait comes near this

struct alignas(64) Sm100Args {
  CUtensorMap tm_q, tm_k, tm_v, tm_k2, tm_v2;
  int32_t q_seg_len, q_cps, q_chunks;
  int32_t k_seg_len, k_cps, k_chunks_main, k2_len, kv_chunks, n_kv_tiles, k_tail, k2_tail;
  int32_t H, D, dk16, dv_n;
  int32_t sq_total;
  float scale_log2;
  void* out;
  int64_t out_stride_b, out_stride_h, out_stride_seg, out_stride_row;
  void* out_seg[XDIT_MAX_OUT_SEGMENTS];  // per-segment output bases (possibly peer GPUs' memory); out == nullptr then
  float* lse;
  float* o_acc;
  float* lse_acc;
  int32_t acc_in, acc_out;
  int32_t* status;
  int32_t* status_host;     // optional pinned host word (mapped): written on a timeout only, never read
  uint32_t wait_limit_ns;   // time limit of every mbarrier wait
  int32_t selftest_stall;   // test aid: the loader leaves K/V stage 0 un-armed, so a consumer's wait runs out
  // keys split over kv_splits CTAs per pair of query tiles (blockIdx.x = split * pairs + pair); every split
  // writes a normalised fp32 partial result [kv_splits][part_rows][D] and its log-sum-exp [kv_splits][part_rows]
  int32_t kv_splits, pairs;
  int64_t part_rows;
  float* part_o;
  float* part_lse;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// low word of the nanosecond timer: differences are exact up to 4.29 s, far above the wait limit
__device__ __forceinline__ uint32_t global_timer_ns() {
  uint32_t t;
  asm volatile("mov.u32 %0, %%globaltimer_lo;" : "=r"(t));
  return t;
}
// Bounded wait.  Returns false when the CTA is aborting or the time limit passed (and then
// raises the abort flag itself, recording `code`).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t limit_ns,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint32_t t0 = global_timer_ns();
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((it & 63) == 63 && global_timer_ns() - t0 > limit_ns) {
      *abort_flag = code;
      return false;
    }
  }
}
// A launch whose status word is already set (an earlier CTA or launch timed out) does no work:
// it keeps a failure from costing one time limit per CTA.
__device__ __forceinline__ bool status_is_set(const int32_t* status) {
  return status != nullptr && *reinterpret_cast<const volatile int32_t*>(status) != 0;
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0,
                                            int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
// One lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
// Groups of MMAs in one asm block.  A shared-memory descriptor is its tile's base descriptor plus a
// constant in the low word (the address field counts 16-byte units; shared-memory addresses stay
// below its 256 KB range) over a common high word, so a step costs two adds and the MMA.
// S = Q K^T at head_dim 128: 8 k-steps, both operands K-major tiles of 128 rows (16 KB slabs).
__device__ __forceinline__ void qk_block8(uint32_t d_tmem, uint32_t q_lo, uint32_t k_lo, uint32_t hi, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred pt, pf;\n\t.reg .b32 ta, tb;\n\t.reg .b64 da, db;\n\t"
      "setp.eq.u32 pt, %3, %3;\n\tsetp.ne.u32 pf, %3, %3;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pf;\n\t"
      "add.u32 ta, %1, %5;\n\tadd.u32 tb, %2, %5;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 ta, %1, %6;\n\tadd.u32 tb, %2, %6;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 ta, %1, %7;\n\tadd.u32 tb, %2, %7;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 ta, %1, %8;\n\tadd.u32 tb, %2, %8;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 ta, %1, %9;\n\tadd.u32 tb, %2, %9;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 ta, %1, %10;\n\tadd.u32 tb, %2, %10;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 ta, %1, %11;\n\tadd.u32 tb, %2, %11;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t"
      "}"
      ::"r"(d_tmem), "r"(q_lo), "r"(k_lo), "r"(hi), "r"(idesc),
        "n"(((1 >> 2) * (128 * 128) + (1 & 3) * 32) >> 4), "n"(((2 >> 2) * (128 * 128) + (2 & 3) * 32) >> 4), "n"(((3 >> 2) * (128 * 128) + (3 & 3) * 32) >> 4), "n"(((4 >> 2) * (128 * 128) + (4 & 3) * 32) >> 4), "n"(((5 >> 2) * (128 * 128) + (5 & 3) * 32) >> 4), "n"(((6 >> 2) * (128 * 128) + (6 & 3) * 32) >> 4), "n"(((7 >> 2) * (128 * 128) + (7 & 3) * 32) >> 4)
      : "memory");
}
// O += P V for 64 key rows: 4 k-steps, A = P from TMEM (8 columns per step), B = V MN-major (2 KB per step).
__device__ __forceinline__ void pv_block4(uint32_t d_tmem, uint32_t p_tmem, uint32_t v_lo, uint32_t hi, uint32_t idesc,
                                          uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred pt, pa;\n\t.reg .b32 ta, tb;\n\t.reg .b64 db;\n\t"
      "setp.eq.u32 pt, %3, %3;\n\tsetp.ne.b32 pa, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, pa;\n\t"
      "add.u32 ta, %1, 8;\n\tadd.u32 tb, %2, 128;\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "add.u32 ta, %1, 16;\n\tadd.u32 tb, %2, 256;\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "add.u32 ta, %1, 24;\n\tadd.u32 tb, %2, 384;\n\tmov.b64 db, {tb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n\t"
      "}"
      ::"r"(d_tmem), "r"(p_tmem), "r"(v_lo), "r"(hi), "r"(idesc), "r"(acc)
      : "memory");
}
#define XDIT_R32(a, o) \
  "=r"(a[o + 0]), "=r"(a[o + 1]), "=r"(a[o + 2]), "=r"(a[o + 3]), "=r"(a[o + 4]), "=r"(a[o + 5]), "=r"(a[o + 6]), \
  "=r"(a[o + 7]), "=r"(a[o + 8]), "=r"(a[o + 9]), "=r"(a[o + 10]), "=r"(a[o + 11]), "=r"(a[o + 12]),                \
  "=r"(a[o + 13]), "=r"(a[o + 14]), "=r"(a[o + 15]), "=r"(a[o + 16]), "=r"(a[o + 17]), "=r"(a[o + 18]),              \
  "=r"(a[o + 19]), "=r"(a[o + 20]), "=r"(a[o + 21]), "=r"(a[o + 22]), "=r"(a[o + 23]), "=r"(a[o + 24]),              \
  "=r"(a[o + 25]), "=r"(a[o + 26]), "=r"(a[o + 27]), "=r"(a[o + 28]), "=r"(a[o + 29]), "=r"(a[o + 30]), "=r"(a[o + 31])
#define XDIT_W32(a, o) \
  "r"(a[o + 0]), "r"(a[o + 1]), "r"(a[o + 2]), "r"(a[o + 3]), "r"(a[o + 4]), "r"(a[o + 5]), "r"(a[o + 6]),    \
  "r"(a[o + 7]), "r"(a[o + 8]), "r"(a[o + 9]), "r"(a[o + 10]), "r"(a[o + 11]), "r"(a[o + 12]), "r"(a[o + 13]), \
  "r"(a[o + 14]), "r"(a[o + 15]), "r"(a[o + 16]), "r"(a[o + 17]), "r"(a[o + 18]), "r"(a[o + 19]),             \
  "r"(a[o + 20]), "r"(a[o + 21]), "r"(a[o + 22]), "r"(a[o + 23]), "r"(a[o + 24]), "r"(a[o + 25]),             \
  "r"(a[o + 26]), "r"(a[o + 27]), "r"(a[o + 28]), "r"(a[o + 29]), "r"(a[o + 30]), "r"(a[o + 31])
// 32 lanes x 32 consecutive columns -> 32 registers per thread (thread i = lane base + i)
#define XDIT_TMEM_LD32(a, o, taddr)                                                                      \
  asm volatile(                                                                                          \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                          \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                           \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"          \
      : XDIT_R32(a, o) : "r"(taddr) : "memory")
#define XDIT_TMEM_ST32(a, o, taddr)                                                                      \
  asm volatile(                                                                                          \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "                                                   \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                           \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"                 \
      ::XDIT_W32(a, o), "r"(taddr) : "memory")
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// same instruction, but volatile: the compiler keeps a run of these in program order, which is how
// the softmax loop forces a batch of independent ex2 to be issued back to back
__device__ __forceinline__ float ex2_ordered(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// packed fp32 pairs (one 64-bit register): halves the issue slots of the softmax arithmetic
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t x, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(x));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// Shared-memory matrix descriptors (sm_100 format: version 1 at bit 46, 128-byte swizzle = 2 at
// bits 61-63, offsets in 16-byte units).
// K-major operand (Q, K): rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (V: N = head_dim contiguous, K = key rows): 64-element groups of N are one
// slab apart (leading offset), 8-row groups of K are 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(kSlabBytes >> 4) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: D fp32, A/B bf16 (1) or fp16 (0), M = 128.
__device__ __forceinline__ uint32_t make_idesc(bool bf16, bool b_mn_major, int n) {
  const uint32_t fmt = bf16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kTile >> 4) << 24);
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

struct ChunkLoc {
  int src, seg, row0, valid;
};
__device__ __forceinline__ ChunkLoc kv_chunk(const Sm100Args& a, int c) {
  ChunkLoc r;
  if (c < a.k_chunks_main) {
    r.src = 0;
    r.seg = c / a.k_cps;
    r.row0 = (c - r.seg * a.k_cps) * kChunk;
    r.valid = min(kChunk, a.k_seg_len - r.row0);
  } else if (c < a.kv_chunks) {
    r.src = 1;
    r.seg = 0;
    r.row0 = (c - a.k_chunks_main) * kChunk;
    r.valid = min(kChunk, a.k2_len - r.row0);
  } else {  // past the end: a box that is entirely out of range reads zeros
    r.src = 0;
    r.seg = 0;
    r.row0 = ((a.k_seg_len + kChunk - 1) / kChunk) * kChunk;
    r.valid = 0;
  }
  return r;
}

template <int SLABS, int NSTAGE>
struct SmemLayout {
  static constexpr int kQTileBytes = SLABS * kSlabBytes;
  static constexpr int kStageBytes = SLABS * kSlabBytes;
  static constexpr int kQOff = 0;
  static constexpr int kKvOff = 2 * kQTileBytes;
  static constexpr int kBarOff = kKvOff + NSTAGE * kStageBytes;
  // barriers: q_full[2], kv_full[NSTAGE], kv_empty[NSTAGE], s_full[2], p_full[2][2], o_full[2], drain
  static constexpr int kNumBars = 2 + 2 * NSTAGE + 2 + 4 + 2 + 1;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;  // slack to align the base to 1024 bytes
};

// ---------------------------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------------------------
template <int SLABS, int NSTAGE, bool BF16>
__global__ void __launch_bounds__(kThreads, 1) attn_fwd_sm100_kernel(const __grid_constant__ Sm100Args a) {
  using L = SmemLayout<SLABS, NSTAGE>;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - raw);

  const uint32_t q_smem = base + L::kQOff;
  const uint32_t kv_smem = base + L::kKvOff;
  const uint32_t bar0 = base + L::kBarOff;
  auto bar_q_full = [&](int t) { return bar0 + 8u * t; };
  auto bar_kv_full = [&](int s) { return bar0 + 8u * (2 + s); };
  auto bar_kv_empty = [&](int s) { return bar0 + 8u * (2 + NSTAGE + s); };
  auto bar_s_full = [&](int t) { return bar0 + 8u * (2 + 2 * NSTAGE + t); };
  // P of a key tile is published in two halves of 64 key columns, one barrier each (a waiter on
  // an mbarrier may fall at most one phase behind, so the halves cannot share one barrier)
  auto bar_p_full = [&](int t, int half) { return bar0 + 8u * (4 + 2 * NSTAGE + 2 * t + half); };
  auto bar_o_full = [&](int t) { return bar0 + 8u * (8 + 2 * NSTAGE + t); };
  const uint32_t bar_drain = bar0 + 8u * (10 + 2 * NSTAGE);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::kMiscOff + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x / a.pairs, pair = blockIdx.x - split * a.pairs, h = blockIdx.y, b = blockIdx.z;
  // key tiles [jt0, jt0 + n_tiles) of the a.n_kv_tiles belong to this CTA (all of them without a split)
  const int jt0 = (int)((int64_t)split * a.n_kv_tiles / a.kv_splits);
  const int n_tiles = (int)((int64_t)(split + 1) * a.n_kv_tiles / a.kv_splits) - jt0;
  // query tile t of this CTA covers query chunks 4*pair + 2t and 4*pair + 2t + 1
  const bool tile_on[2] = {4 * pair < a.q_chunks, 4 * pair + 2 < a.q_chunks};

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_q_full(t), 1);
      mbar_init(bar_s_full(t), 1);
      mbar_init(bar_p_full(t, 0), 128);
      mbar_init(bar_p_full(t, 1), 128);
      mbar_init(bar_o_full(t), 1);
    }
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
    }
    mbar_init(bar_drain, 1);
    *abort_flag = status_is_set(a.status) ? -1 : 0;  // -1: skip all work (an earlier failure is pending)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool skip = *abort_flag != 0;  // same value for every thread: written before the barrier above

  if (skip) {
    // nothing to do: fall through to the teardown, which frees TMEM
  } else if (warp >= 8) {
    // warps 8-11 hand registers to the softmax warps: per scheduler 2 x 232 + 40 <= 512
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 9) {
    // ======================= TMA producer =======================
    if (lane == 0) {
      int issued = 0;  // ring items armed so far
      bool ok = true;
      for (int t = 0; t < 2 && ok; ++t) {
        if (!tile_on[t]) continue;
        mbar_arrive_expect_tx(bar_q_full(t), L::kQTileBytes);
        for (int c = 0; c < 2; ++c) {
          const int qc = 4 * pair + 2 * t + c;
          int seg = 0, row0 = ((a.q_seg_len + kChunk - 1) / kChunk) * kChunk;  // out of range -> zeros
          if (qc < a.q_chunks) {
            seg = qc / a.q_cps;
            row0 = (qc - seg * a.q_cps) * kChunk;
          }
          for (int s = 0; s < SLABS; ++s)
            tma_load_5d(q_smem + t * L::kQTileBytes + s * kSlabBytes + c * kBoxBytes, &a.tm_q, bar_q_full(t),
                        s * 64, row0, seg, h, b);
        }
      }
      const int n_items = 2 * n_tiles;
      for (int i = 0; i < n_items && ok; ++i) {
        const int stage = i % NSTAGE;
        if (a.selftest_stall) { ok = false; break; }  // nothing is armed: the MMA warp's wait on stage 0 runs out
        if (i >= NSTAGE) ok = mbar_wait(bar_kv_empty(stage), ((i / NSTAGE) - 1) & 1, abort_flag, a.wait_limit_ns, 100 + stage);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_kv_full(stage), L::kStageBytes);
        const int j = i >> 1;
        const bool is_v = i & 1;
        for (int c = 0; c < 2; ++c) {
          const ChunkLoc loc = kv_chunk(a, 2 * (jt0 + j) + c);
          const CUtensorMap* tm = loc.src ? (is_v ? &a.tm_v2 : &a.tm_k2) : (is_v ? &a.tm_v : &a.tm_k);
          for (int s = 0; s < SLABS; ++s)
            tma_load_5d(kv_smem + stage * L::kStageBytes + s * kSlabBytes + c * kBoxBytes, tm, bar_kv_full(stage),
                        s * 64, loc.row0, loc.seg, h, b);
        }
        issued = i + 1;
      }
      if (!ok) {
        // drain: every armed stage must have received its bytes before the CTA may leave
        const int first = issued > NSTAGE ? issued - NSTAGE : 0;
        for (int i = first; i < issued; ++i) {
          const uint32_t bar = bar_kv_full(i % NSTAGE), par = (i / NSTAGE) & 1;
          for (int it = 0; it < (1 << 20) && !mbar_try_wait(bar, par); ++it) __nanosleep(64);
        }
        for (int t = 0; t < 2; ++t)
          if (tile_on[t])
            for (int it = 0; it < (1 << 20) && !mbar_try_wait(bar_q_full(t), 0); ++it) __nanosleep(64);
      }
    }
    } else if (warp == 8) {
    // ======================= MMA issuer =======================
    // The whole warp runs this role converged and one elected lane issues the tcgen05 instructions:
    // descriptors, TMEM addresses and barrier addresses are then warp-uniform values which the
    // compiler can keep in uniform registers, where tcgen05.mma / tcgen05.commit take their operands.
    // (Inside a single-lane branch every operand is first moved over from a vector register, and
    // that traffic, not the tensor pipe, set the pace of S = Q K^T.)
    {
      const bool leader = elect_one();
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t idesc_qk = make_idesc(BF16, false, kTile);
      const uint32_t idesc_pv = make_idesc(BF16, true, a.dv_n);
      const int dk16 = a.dk16;
      const bool two = tile_on[1];  // tile 0 exists in every launched CTA
      bool ok = true;
      const uint32_t kdesc_hi = (uint32_t)(desc_kmajor(0) >> 32), vdesc_hi = (uint32_t)(desc_mnmajor(0) >> 32);
      const uint32_t q_lo = (uint32_t)desc_kmajor(q_smem);
      const uint32_t kv_lo = (uint32_t)desc_kmajor(kv_smem);
      // the low words of the K-major and MN-major forms differ in the leading-offset field only
      constexpr uint32_t v_lo_delta = (uint32_t)((kSlabBytes >> 4) - 1) << 16;
      auto wait_all = [&](uint32_t bar, uint32_t parity, int code) {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, a.wait_limit_ns, code));
      };
      // S_t = Q_t K^T (call from the elected lane only)
      auto issue_qk = [&](int t, int stage) {
        const uint32_t qa = q_lo + (uint32_t)(t * (L::kQTileBytes >> 4));
        const uint32_t kb = kv_lo + (uint32_t)(stage * (L::kStageBytes >> 4));
        const uint32_t d = tmem_u + t * kTile;
        if (dk16 == 8) {
          qk_block8(d, qa, kb, kdesc_hi, idesc_qk);
        } else {
          for (int ks = 0; ks < dk16; ++ks) {
            const uint32_t off = ((ks >> 2) * kSlabBytes + (ks & 3) * 32) >> 4;
            tc_mma_ss(d, ((uint64_t)kdesc_hi << 32) | (qa + off), ((uint64_t)kdesc_hi << 32) | (kb + off), idesc_qk,
                      ks > 0);
          }
        }
      };
      // O_t += P_t[:, 64*half : 64*half+64] V[64*half : 64*half+64, :]   (4 steps of 16 key rows)
      auto issue_pv_half = [&](int t, int stage, int half, bool first_tile) {
        const uint32_t vb = kv_lo + v_lo_delta + (uint32_t)(stage * (L::kStageBytes >> 4)) + half * (4 * 2048 >> 4);
        pv_block4(tmem_u + 256 + t * kTile, tmem_u + t * kTile + half * 32, vb, vdesc_hi, idesc_pv,
                  (first_tile && half == 0) ? 0u : 1u);
      };
      // prologue: S_t(0) = Q_t K(0)^T
      ok = wait_all(bar_kv_full(0), 0, 200);
      for (int t = 0; t < 2 && ok; ++t) {
        if (t == 1 && !two) continue;
        ok = wait_all(bar_q_full(t), 0, 201 + t);
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          issue_qk(t, 0);
          tc_commit(bar_s_full(t));
        }
      }
      if (ok && leader) tc_commit(bar_kv_empty(0));
      // ring cursors: V(j) is item 2j+1, K(j+1) item 2j+2
      int sv = 1 % NSTAGE, pv = 0, sk = 2 % NSTAGE, pk = 0;
      auto advance2 = [&](int& st, int& ph) {
        st += 2;
        if (st >= NSTAGE) { st -= NSTAGE; ph ^= 1; }
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const bool more = j + 1 < n_tiles;
        ok = wait_all(bar_kv_full(sv), pv, 210);
        for (int t = 0; t < 2 && ok; ++t) {
          if (t == 1 && !two) continue;
          const bool last_tile = two ? t == 1 : true;
          // P arrives in two halves (64 key columns each): the first half of O += P V runs while
          // the softmax group still computes the second half
          ok = wait_all(bar_p_full(t, 0), j & 1, 220 + t);
          if (!ok) break;
          tc_fence_after();
          if (leader) issue_pv_half(t, sv, 0, j == 0);
          if (more && t == 0) {
            // K(j+1) has long arrived; taking the wait here keeps it out of the single-lane region below
            ok = wait_all(bar_kv_full(sk), pk, 230);
            if (!ok) break;
          }
          ok = wait_all(bar_p_full(t, 1), j & 1, 222 + t);
          if (!ok) break;
          tc_fence_after();
          if (leader) {
            issue_pv_half(t, sv, 1, j == 0);
            if (last_tile) tc_commit(bar_kv_empty(sv));  // V(j) is free once both tiles' PV retire
            if (more) {
              issue_qk(t, sk);
              // completes after every MMA issued so far, i.e. it also tells the softmax group that
              // O_t holds the sum up to key tile j
              tc_commit(bar_s_full(t));
              if (last_tile) tc_commit(bar_kv_empty(sk));
            } else {
              tc_commit(bar_o_full(t));
            }
          }
        }
        if (!ok) break;
        advance2(sv, pv);
        advance2(sk, pk);
      }
      if (!ok) {
        // drain the tensor pipe before TMEM is released
        if (leader) tc_commit(bar_drain);
        if (lane == 0)
          for (int it = 0; it < (1 << 20) && !mbar_try_wait(bar_drain, 0); ++it) __nanosleep(64);
        __syncwarp();
      }
    }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ======================= softmax + epilogue =======================
    const int t = warp >> 2;         // query tile of this warp group
    const int wq = warp & 3;         // TMEM lane quarter this warp may touch
    const int row = wq * 32 + lane;  // query row inside the tile
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_base + t * kTile;
    const uint32_t tmem_o = tmem_base + lane_base + 256 + t * kTile;
    bool ok = true;
    float m_run = -INFINITY;  // running reference maximum, in scaled log2 units
    float l_run = 0.f;
    const float sl2 = a.scale_log2;
    // valid key columns of the next chunk, tracked without divisions
    int cidx = 2 * jt0, cpos = (2 * jt0 < a.k_chunks_main) ? (2 * jt0) % a.k_cps : 0;
    auto next_valid = [&]() -> int {
      int v;
      if (cidx < a.k_chunks_main) {
        v = (cpos == a.k_cps - 1) ? a.k_tail : kChunk;
        if (++cpos == a.k_cps) cpos = 0;
      } else if (cidx < a.kv_chunks) {
        v = (cidx == a.kv_chunks - 1) ? a.k2_tail : kChunk;
      } else {
        v = 0;
      }
      ++cidx;
      return v;
    };
    // One key tile for this thread's query row.  MASKED is a compile-time switch so that full
    // tiles carry no masking instructions at all.
    auto softmax_tile = [&](auto masked_tag, int j, int v0, int v1) -> bool {
      constexpr bool MASKED = decltype(masked_tag)::value;
      tc_fence_after();
      uint32_t s[128];
      XDIT_TMEM_LD32(s, 0, tmem_s + 0);
      XDIT_TMEM_LD32(s, 32, tmem_s + 32);
      XDIT_TMEM_LD32(s, 64, tmem_s + 64);
      XDIT_TMEM_LD32(s, 96, tmem_s + 96);
      tmem_wait_ld();
      if constexpr (MASKED) {
#pragma unroll
        for (int c = 0; c < 128; ++c) {
          const bool dead = (c < 64) ? (c >= v0) : (c - 64 >= v1);
          if (dead) s[c] = 0xff800000u;  // -inf
        }
      }
      float mx0 = max3(__uint_as_float(s[0]), __uint_as_float(s[1]), __uint_as_float(s[2]));
      float mx1 = max3(__uint_as_float(s[3]), __uint_as_float(s[4]), __uint_as_float(s[5]));
      float mx2 = max3(__uint_as_float(s[6]), __uint_as_float(s[7]), __uint_as_float(s[8]));
      float mx3 = max3(__uint_as_float(s[9]), __uint_as_float(s[10]), __uint_as_float(s[11]));
#pragma unroll
      for (int c = 12; c < 124; c += 8) {
        mx0 = max3(mx0, __uint_as_float(s[c]), __uint_as_float(s[c + 1]));
        mx1 = max3(mx1, __uint_as_float(s[c + 2]), __uint_as_float(s[c + 3]));
        mx2 = max3(mx2, __uint_as_float(s[c + 4]), __uint_as_float(s[c + 5]));
        mx3 = max3(mx3, __uint_as_float(s[c + 6]), __uint_as_float(s[c + 7]));
      }
      mx0 = max3(mx0, __uint_as_float(s[124]), __uint_as_float(s[125]));
      mx1 = max3(mx1, __uint_as_float(s[126]), __uint_as_float(s[127]));
      const float mt = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;
      if (j == 0) {
        m_run = mt;
      } else {
        // Lazy rescale: keep the old reference maximum unless some row of this warp grew by
        // more than 2^8; exp2 of at most 8 is safe in fp32 and in the 16-bit P.  S_t(j) being
        // complete implies that O_t += P V of tile j-1 has retired, so O may be touched here.
        const bool grow = mt > m_run + 8.f;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m_run, mt);
          const float alpha = ex2(m_run - m_new);
          for (int c0 = 0; c0 < a.dv_n; c0 += 32) {
            uint32_t o[32];
            XDIT_TMEM_LD32(o, 0, tmem_o + c0);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
            XDIT_TMEM_ST32(o, 0, tmem_o + c0);
          }
          tmem_wait_st();
          l_run *= alpha;
          m_run = m_new;
        }
      }
      // P = 2^(s*scale - m), handed to the tensor core in two halves of 64 key columns.
      const uint64_t sl2_2 = f2_pack(sl2, sl2), negm_2 = f2_pack(-m_run, -m_run);
      // Software-pipelined in blocks of 16 columns: the 16 ex2 of block b+1 are issued before the
      // results of block b are consumed.  A warp issues in order, so without this every pair
      // would wait out the special-function unit's latency before the next one starts.
      uint64_t acc4[4] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
      uint32_t pk[64];
      float pcur[16], pnext[16];
      auto stage_ab = [&](int blk, float* p) {
        uint64_t x2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          x2[i] = f2_fma(f2_pack(__uint_as_float(s[16 * blk + 2 * i]), __uint_as_float(s[16 * blk + 2 * i + 1])),
                         sl2_2, negm_2);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float x0, x1;
          f2_unpack(x2[i], x0, x1);
          p[2 * i] = ex2_ordered(x0);
          p[2 * i + 1] = ex2_ordered(x1);
        }
      };
      auto stage_c = [&](int blk, const float* p) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          acc4[i & 3] = f2_add(acc4[i & 3], f2_pack(p[2 * i], p[2 * i + 1]));
          pk[8 * blk + i] = pack2<BF16>(p[2 * i], p[2 * i + 1]);
        }
      };
      stage_ab(0, pcur);
#pragma unroll
      for (int blk = 0; blk < 8; ++blk) {
        if (blk + 1 < 8) stage_ab(blk + 1, pnext);
        stage_c(blk, pcur);
#pragma unroll
        for (int i = 0; i < 16; ++i) pcur[i] = pnext[i];
        if (blk == 3 || blk == 7) {
          const int half = blk >> 2;
          XDIT_TMEM_ST32(pk, 32 * half, tmem_s + 32 * half);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(bar_p_full(t, half));
        }
      }
      {
        float a0, a1;
        f2_unpack(f2_add(f2_add(acc4[0], acc4[1]), f2_add(acc4[2], acc4[3])), a0, a1);
        l_run += a0 + a1;
      }
      return true;
    };
    if (tile_on[t]) {
      for (int j = 0; j < n_tiles; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full(t), j & 1, abort_flag, a.wait_limit_ns, 300 + t));
        if (!ok) break;
        const int v0 = next_valid(), v1 = next_valid();
        if (v0 < kChunk || v1 < kChunk) softmax_tile(std::true_type{}, j, v0, v1);
        else softmax_tile(std::false_type{}, j, v0, v1);
      }
      // ---------------- epilogue ----------------
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_o_full(t), 0, abort_flag, a.wait_limit_ns, 320 + t));
      if (ok) {
        tc_fence_after();
        const int qc = 4 * pair + 2 * t + (row >> 6);
        int seg = 0, trow = 0;
        bool live = qc < a.q_chunks;
        if (live) {
          seg = qc / a.q_cps;
          trow = (qc - seg * a.q_cps) * kChunk + (row & 63);
          live = trow < a.q_seg_len;
        }
        const int64_t flat = ((int64_t)b * a.H + h) * a.sq_total + (int64_t)seg * a.q_seg_len + trow;
        const float inv_l = 1.f / l_run;
        float lse = (m_run + log2f(l_run)) * 0.6931471805599453f;
        float w = 0.f;
        const bool merge = a.acc_in != 0;
        if (merge && live) {
          const float la = a.lse_acc[flat];
          if (!(la == -INFINITY && lse == -INFINITY)) {
            w = 1.f / (1.f + __expf(la - lse));            // sigmoid(lse - la)
            const float y = la - lse;                        // lse <- la - logsigmoid(la - lse)
            lse = la - (fminf(y, 0.f) - log1pf(__expf(-fabsf(y))));
          }
        }
        if (a.kv_splits > 1) {
          // partial result of this CTA's share of the keys: normalised fp32 rows and their log-sum-exp; the
          // merge kernel that follows on the stream writes the output
          float* prow = a.part_o + ((int64_t)split * a.part_rows + flat) * a.D;
          for (int c0 = 0; c0 < a.dv_n; c0 += 32) {
            uint32_t o[32];
            XDIT_TMEM_LD32(o, 0, tmem_o + c0);
            tmem_wait_ld();
            if (live) {
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                const int col = c0 + 4 * g;
                if (col < a.D)
                  *reinterpret_cast<float4*>(prow + col) =
                      make_float4(__uint_as_float(o[4 * g]) * inv_l, __uint_as_float(o[4 * g + 1]) * inv_l,
                                  __uint_as_float(o[4 * g + 2]) * inv_l, __uint_as_float(o[4 * g + 3]) * inv_l);
              }
            }
          }
          if (live) a.part_lse[(int64_t)split * a.part_rows + flat] = lse;
        } else {
        unsigned char* orow = nullptr;
        if (!a.acc_out) {
          // one base per query segment when the rows go to their source ranks' buffers, else one tensor
          unsigned char* obase = a.out ? reinterpret_cast<unsigned char*>(a.out) + 2 * seg * a.out_stride_seg
                                       : reinterpret_cast<unsigned char*>(a.out_seg[seg]);
          orow = obase + 2 * (b * a.out_stride_b + h * a.out_stride_h + trow * a.out_stride_row);
        }
        float* arow = a.o_acc ? a.o_acc + flat * a.D : nullptr;
        for (int c0 = 0; c0 < a.dv_n; c0 += 32) {
          uint32_t o[32];
          XDIT_TMEM_LD32(o, 0, tmem_o + c0);
          tmem_wait_ld();
          if (live) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = c0 + 8 * g;
              if (col < a.D) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(o[8 * g + e]) * inv_l;
                if (merge) {
                  const float4 a0 = *reinterpret_cast<const float4*>(arow + col);
                  const float4 a1 = *reinterpret_cast<const float4*>(arow + col + 4);
                  const float oa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] = oa[e] - w * (oa[e] - v[e]);
                }
                if (a.acc_out) {
                  *reinterpret_cast<float4*>(arow + col) = make_float4(v[0], v[1], v[2], v[3]);
                  *reinterpret_cast<float4*>(arow + col + 4) = make_float4(v[4], v[5], v[6], v[7]);
                } else {
                  uint4 pkd;
                  pkd.x = pack2<BF16>(v[0], v[1]);
                  pkd.y = pack2<BF16>(v[2], v[3]);
                  pkd.z = pack2<BF16>(v[4], v[5]);
                  pkd.w = pack2<BF16>(v[6], v[7]);
                  *reinterpret_cast<uint4*>(orow + 2 * col) = pkd;
                }
              }
            }
          }
        }
        if (live) {
          if (a.acc_out) a.lse_acc[flat] = lse;
          else if (a.lse) a.lse[flat] = lse;
        }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  // Rows stored into peer GPUs' memory: one system-scope fence per CTA, after the barrier that
  // orders every thread's stores before it.
  if (threadIdx.x == 0 && !a.out && !a.acc_out) __threadfence_system();
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag > 0) {
    if (a.status) atomicCAS(a.status, 0, *abort_flag);
    if (a.status_host) {  // host-visible copy, read by the next xdit_attn_fwd call without a synchronise
      *reinterpret_cast<volatile int32_t*>(a.status_host) = *abort_flag;
      __threadfence_system();
    }
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !p) return nullptr;
    fn = (EncodeTiledFn)p;
  }
  return fn;
}

// Encoded maps are kept in a small direct-mapped cache keyed by everything the encoding depends on
// (address, extents, strides, dtype): a layer loop that re-uses its buffers, or a graph capture that
// re-runs the same call, pays for cuTensorMapEncodeTiled once.  A tensor map holds no device state,
// so an entry stays valid for as long as the same address means the same tensor to the caller.
struct MapKey {
  const void* ptr;
  int64_t st[4];
  int32_t seg_len, nseg, dtype, B, H, D;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && st[0] == o.st[0] && st[1] == o.st[1] && st[2] == o.st[2] && st[3] == o.st[3] &&
           seg_len == o.seg_len && nseg == o.nseg && dtype == o.dtype && B == o.B && H == o.H && D == o.D;
  }
};
constexpr int kMapCacheSize = 256;
struct MapCache {
  std::mutex mu;
  bool used[kMapCacheSize] = {};
  MapKey key[kMapCacheSize];
  CUtensorMap map[kMapCacheSize];
};
MapCache& map_cache() {
  static MapCache c;
  return c;
}
inline uint32_t map_hash(const MapKey& k) {
  uint64_t h = (uint64_t)(uintptr_t)k.ptr * 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < 4; ++i) h = (h ^ (uint64_t)k.st[i]) * 0x100000001B3ull;
  h = (h ^ (uint64_t)(uint32_t)k.seg_len ^ ((uint64_t)(uint32_t)k.nseg << 32)) * 0x100000001B3ull;
  h = (h ^ (uint64_t)(uint32_t)k.D ^ ((uint64_t)(uint32_t)k.H << 16) ^ ((uint64_t)(uint32_t)k.B << 40) ^
       ((uint64_t)(uint32_t)k.dtype << 60)) * 0x100000001B3ull;
  return (uint32_t)(h >> 40) % kMapCacheSize;
}

int encode_seq_map_uncached(CUtensorMap* tm, const xdit_seq& s, int dtype, int B, int H, int D);

// 5-D map (d, row, segment, head, batch); a TMA box is 64 elements x 64 rows.
int encode_seq_map(CUtensorMap* tm, const xdit_seq& s, int dtype, int B, int H, int D) {
  MapKey k;
  memset(&k, 0, sizeof(k));
  k.ptr = s.ptr;
  k.st[0] = s.stride_row; k.st[1] = s.stride_seg; k.st[2] = s.stride_h; k.st[3] = s.stride_b;
  k.seg_len = s.seg_len; k.nseg = s.nseg; k.dtype = dtype; k.B = B; k.H = H; k.D = D;
  const uint32_t slot = map_hash(k);
  MapCache& c = map_cache();
  {
    std::lock_guard<std::mutex> lk(c.mu);
    if (c.used[slot] && c.key[slot] == k) { *tm = c.map[slot]; return XDIT_OK; }
  }
  const int rc = encode_seq_map_uncached(tm, s, dtype, B, H, D);
  if (rc) return rc;
  std::lock_guard<std::mutex> lk(c.mu);
  c.used[slot] = true; c.key[slot] = k; c.map[slot] = *tm;
  return XDIT_OK;
}

int encode_seq_map_uncached(CUtensorMap* tm, const xdit_seq& s, int dtype, int B, int H, int D) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return XDIT_E_DRIVER; }
  const uint64_t es = 2;
  cuuint64_t dims[5] = {(cuuint64_t)D, (cuuint64_t)s.seg_len, (cuuint64_t)s.nseg, (cuuint64_t)H, (cuuint64_t)B};
  int64_t st[4] = {s.stride_row, s.stride_seg, s.stride_h, s.stride_b};
  cuuint64_t strides[4];
  for (int i = 0; i < 4; ++i) {
    // a dimension of extent 1 is never stepped; give it a harmless legal stride
    int64_t v = (dims[i + 1] > 1) ? st[i] : (st[i] > 0 && st[i] % 8 == 0 ? st[i] : (int64_t)((D + 7) / 8 * 8));
    strides[i] = (cuuint64_t)v * es;
  }
  cuuint32_t box[5] = {64, (cuuint32_t)kChunk, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(tm, dtype == XDIT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
                  const_cast<void*>(s.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (D=%d seg_len=%d nseg=%d strides %lld %lld %lld %lld)",
              (int)r, D, s.seg_len, s.nseg, (long long)s.stride_row, (long long)s.stride_seg,
              (long long)s.stride_h, (long long)s.stride_b);
    return XDIT_E_DRIVER;
  }
  return XDIT_OK;
}

bool seq_ok(const xdit_seq& s, int B, int H, int D, const char* name) {
  if (((uintptr_t)s.ptr) & 15) { set_error("tcgen05 path: %s pointer is not 16-byte aligned", name); return false; }
  if (s.stride_row < 0 || (s.seg_len > 1 && (s.stride_row % 8 || s.stride_row < D))) { set_error("tcgen05 path: %s row stride %lld", name, (long long)s.stride_row); return false; }
  if (s.nseg > 1 && (s.stride_seg % 8 || s.stride_seg <= 0)) { set_error("tcgen05 path: %s segment stride", name); return false; }
  if (H > 1 && (s.stride_h % 8 || s.stride_h <= 0)) { set_error("tcgen05 path: %s head stride", name); return false; }
  if (B > 1 && (s.stride_b % 8 || s.stride_b <= 0)) { set_error("tcgen05 path: %s batch stride", name); return false; }
  return true;
}

// Merge of the key splits' partial results into the output: one warp per query row, lane l owns columns
// 4l..4l+3.  out = sum_s w_s O_s / sum_s w_s with w_s = exp(lse_s - max lse), the log-sum-exp of the whole
// row is max + log(sum w): the formula of the ring merge for any number of partials.
template <bool BF16>
__global__ void __launch_bounds__(256) split_merge_kernel(const __grid_constant__ Sm100Args a) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp0; row < a.part_rows; row += nwarps) {
    float ls[4], m = -INFINITY;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      ls[s] = s < a.kv_splits ? a.part_lse[(int64_t)s * a.part_rows + row] : -INFINITY;
      m = fmaxf(m, ls[s]);
    }
    float wsum = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int col = 4 * lane;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      if (s < a.kv_splits) {
        const float w = __expf(ls[s] - m);
        wsum += w;
        if (col < a.D) {
          const float4 o = *reinterpret_cast<const float4*>(a.part_o + ((int64_t)s * a.part_rows + row) * a.D + col);
          acc[0] = fmaf(w, o.x, acc[0]); acc[1] = fmaf(w, o.y, acc[1]);
          acc[2] = fmaf(w, o.z, acc[2]); acc[3] = fmaf(w, o.w, acc[3]);
        }
      }
    }
    const float inv = 1.f / wsum;
    const int64_t bh = row / a.sq_total;
    const int rs = (int)(row - bh * a.sq_total);
    const int b = (int)(bh / a.H), h = (int)(bh - (int64_t)b * a.H);
    const int seg = rs / a.q_seg_len, trow = rs - seg * a.q_seg_len;
    if (col < a.D) {
      unsigned char* obase = a.out ? reinterpret_cast<unsigned char*>(a.out) + 2 * seg * a.out_stride_seg
                                   : reinterpret_cast<unsigned char*>(a.out_seg[seg]);
      unsigned char* orow = obase + 2 * (b * a.out_stride_b + h * a.out_stride_h + trow * a.out_stride_row);
      uint2 pk;
      pk.x = pack2<BF16>(acc[0] * inv, acc[1] * inv);
      pk.y = pack2<BF16>(acc[2] * inv, acc[3] * inv);
      *reinterpret_cast<uint2*>(orow + 2 * col) = pk;
    }
    if (lane == 0 && a.lse) a.lse[row] = m + __logf(wsum);
  }
  if (!a.out) {  // rows stored into peer GPUs' memory: one system-scope fence per CTA
    __syncthreads();
    if (threadIdx.x == 0) __threadfence_system();
  }
}

// How many CTAs per pair of query tiles the keys of a call are split over: as many as fit the GPU's SMs
// beside each other (one wave), at most 4, every split at least four key tiles long, and only what the
// scratch can hold.  54 CTAs (a Flux shard at Ulysses degree 8) become 108 of half the length.  Launches of
// more than one wave are left alone: 216 CTAs (two waves) as 432 halves in three short waves measured
// slower (149 against 138 us), the partial results' traffic and the merge eat the gain.
int choose_kv_splits(const xdit_attn_params& p, int sms, int n_kv_tiles, int ctas, int64_t part_rows, int64_t scratch_bytes) {
  if (p.acc_in || p.acc_out || ctas <= 0) return 1;
  int want = sms / ctas;
  if (want > 4) want = 4;
  if (want > n_kv_tiles / 4) want = n_kv_tiles / 4;
  while (want > 1 && scratch_bytes >= 0 && (int64_t)want * part_rows * (p.D + 1) * 4 > scratch_bytes) --want;
  return want < 2 ? 1 : want;
}

template <int SLABS, int NSTAGE, bool BF16>
int launch_inst(const Sm100Args& a, dim3 grid, cudaStream_t stream) {
  using L = SmemLayout<SLABS, NSTAGE>;
  {
    // the attribute is per device; set once per device, under a lock (calls may come from several threads)
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      e = cudaFuncSetAttribute(attn_fwd_sm100_kernel<SLABS, NSTAGE, BF16>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
      if (e != cudaSuccess) return cuda_fail(e, "attn_fwd_sm100 smem attribute");
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
  }
  attn_fwd_sm100_kernel<SLABS, NSTAGE, BF16><<<grid, kThreads, L::kDynamic, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "attn_fwd_sm100_kernel launch");
  if (a.kv_splits > 1) {
    // a few CTAs per SM striding over the rows: with per-segment bases every CTA ends with a system fence
    int sms = 0;
    if (check_device(&sms) != XDIT_OK || sms <= 0) sms = 148;
    int64_t blocks = (a.part_rows * 32 + 255) / 256;
    if (blocks > (int64_t)sms * 4) blocks = (int64_t)sms * 4;
    split_merge_kernel<BF16><<<(int)blocks, 256, 0, stream>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "split_merge_kernel launch");
  }
  return XDIT_OK;
}

}  // namespace

int attn_sm100_applicable(const xdit_attn_params& p) {
  if (p.dtype != XDIT_BF16 && p.dtype != XDIT_F16) { set_error("tcgen05 path: dtype is not bf16/fp16"); return 0; }
  if (p.D % 8 || p.D < 8 || p.D > 128) { set_error("tcgen05 path: head_dim %d (multiple of 8 up to 128)", p.D); return 0; }
  if (p.causal) { set_error("tcgen05 path: causal masking is served by the CUDA-core kernel"); return 0; }
  if (!seq_ok(p.q, p.B, p.H, p.D, "q") || !seq_ok(p.k, p.B, p.H, p.D, "k") || !seq_ok(p.v, p.B, p.H, p.D, "v")) return 0;
  if (p.k2.ptr && (!seq_ok(p.k2, p.B, p.H, p.D, "k2") || !seq_ok(p.v2, p.B, p.H, p.D, "v2"))) return 0;
  if (!p.acc_out) {
    if (p.out_segments) {
      for (int g = 0; g < p.q.nseg; ++g)
        if (((uintptr_t)p.out_segments[g]) & 15) { set_error("tcgen05 path: out_segments pointer alignment"); return 0; }
    } else if (((uintptr_t)p.out) & 15) { set_error("tcgen05 path: out pointer alignment"); return 0; }
    if (p.out_stride_row % 8 || (p.q.nseg > 1 && !p.out_segments && p.out_stride_seg % 8) || (p.H > 1 && p.out_stride_h % 8) ||
        (p.B > 1 && p.out_stride_b % 8)) { set_error("tcgen05 path: out strides"); return 0; }
  }
  if ((p.acc_in || p.acc_out) && ((((uintptr_t)p.o_acc) & 15) || (p.D % 4))) { set_error("tcgen05 path: o_acc alignment"); return 0; }
  return 1;
}

int launch_attn_sm100(const xdit_attn_params& p, cudaStream_t stream) {
  Sm100Args a;
  memset(&a, 0, sizeof(a));
  int rc;
  if ((rc = encode_seq_map(&a.tm_q, p.q, p.dtype, p.B, p.H, p.D))) return rc;
  if ((rc = encode_seq_map(&a.tm_k, p.k, p.dtype, p.B, p.H, p.D))) return rc;
  if ((rc = encode_seq_map(&a.tm_v, p.v, p.dtype, p.B, p.H, p.D))) return rc;
  if (p.k2.ptr) {
    if ((rc = encode_seq_map(&a.tm_k2, p.k2, p.dtype, p.B, p.H, p.D))) return rc;
    if ((rc = encode_seq_map(&a.tm_v2, p.v2, p.dtype, p.B, p.H, p.D))) return rc;
  } else {
    a.tm_k2 = a.tm_k;
    a.tm_v2 = a.tm_v;
  }
  a.q_seg_len = p.q.seg_len;
  a.q_cps = (p.q.seg_len + kChunk - 1) / kChunk;
  a.q_chunks = a.q_cps * p.q.nseg;
  a.k_seg_len = p.k.seg_len;
  a.k_cps = (p.k.seg_len + kChunk - 1) / kChunk;
  a.k_chunks_main = a.k_cps * p.k.nseg;
  a.k2_len = p.k2.ptr ? p.k2.seg_len : 0;
  a.kv_chunks = a.k_chunks_main + (a.k2_len + kChunk - 1) / kChunk;
  a.n_kv_tiles = (a.kv_chunks + 1) / 2;
  a.k_tail = a.k_seg_len - (a.k_cps - 1) * kChunk;
  a.k2_tail = a.k2_len ? a.k2_len - ((a.k2_len + kChunk - 1) / kChunk - 1) * kChunk : 0;
  a.H = p.H;
  a.D = p.D;
  a.dk16 = (p.D + 15) / 16;
  a.dv_n = a.dk16 * 16;
  a.sq_total = p.q.nseg * p.q.seg_len;
  const float scale = p.softmax_scale > 0.f ? p.softmax_scale : 1.0f / sqrtf((float)p.D);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.out = p.out_segments ? nullptr : p.out;
  if (p.out_segments)
    for (int g = 0; g < p.q.nseg && g < XDIT_MAX_OUT_SEGMENTS; ++g) a.out_seg[g] = p.out_segments[g];
  a.out_stride_b = p.out_stride_b; a.out_stride_h = p.out_stride_h;
  a.out_stride_seg = p.out_stride_seg; a.out_stride_row = p.out_stride_row;
  a.lse = p.lse; a.o_acc = p.o_acc; a.lse_acc = p.lse_acc;
  a.acc_in = p.acc_in; a.acc_out = p.acc_out;
  a.status = p.status;
  a.status_host = p.status_host;
  a.wait_limit_ns = p.wait_limit_ns ? p.wait_limit_ns : kWaitLimitNs;
  a.selftest_stall = p.selftest_stall;
  a.pairs = (a.q_chunks + 3) / 4;
  a.kv_splits = 1;
  a.part_rows = (int64_t)p.B * p.H * a.sq_total;
  if (p.split_scratch && p.split_scratch_bytes > 0 && (((uintptr_t)p.split_scratch) & 15) == 0 && p.D % 4 == 0) {
    int sms = 0;
    if (check_device(&sms) == XDIT_OK && sms > 0) {
      a.kv_splits = choose_kv_splits(p, sms, a.n_kv_tiles, a.pairs * p.H * p.B, a.part_rows, p.split_scratch_bytes);
      if (a.kv_splits > 1) {
        a.part_o = reinterpret_cast<float*>(p.split_scratch);
        a.part_lse = a.part_o + (int64_t)a.kv_splits * a.part_rows * p.D;
      }
    }
  }
  dim3 grid(a.pairs * a.kv_splits, p.H, p.B);
  const bool bf16 = p.dtype == XDIT_BF16;
  if (p.D <= 64) {
    return bf16 ? launch_inst<1, 8, true>(a, grid, stream) : launch_inst<1, 8, false>(a, grid, stream);
  }
  return bf16 ? launch_inst<2, 5, true>(a, grid, stream) : launch_inst<2, 5, false>(a, grid, stream);
}

int64_t attn_sm100_split_scratch_bytes(const xdit_attn_params& p) {
  int sms = 0;
  if (check_device(&sms) != XDIT_OK || sms <= 0) return 0;
  const int q_cps = (p.q.seg_len + kChunk - 1) / kChunk, q_chunks = q_cps * p.q.nseg;
  const int k_cps = (p.k.seg_len + kChunk - 1) / kChunk;
  const int kv_chunks = k_cps * p.k.nseg + (p.k2.ptr ? (p.k2.seg_len + kChunk - 1) / kChunk : 0);
  const int64_t part_rows = (int64_t)p.B * p.H * p.q.nseg * p.q.seg_len;
  const int splits = choose_kv_splits(p, sms, (kv_chunks + 1) / 2, ((q_chunks + 3) / 4) * p.H * p.B, part_rows, -1);
  return splits > 1 ? (int64_t)splits * part_rows * (p.D + 1) * 4 : 0;
}

}  // namespace xdit

