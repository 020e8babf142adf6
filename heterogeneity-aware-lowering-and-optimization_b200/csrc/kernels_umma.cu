// NHWC implicit-GEMM convolution and GEMM on the Blackwell tensor cores (sm_100a).
//
//   D[M, K_out] = A[M, R*S*C] * B[K_out, R*S*C]^T       M = N*P*Q output pixels
//
// A is never materialised: a TMA load in im2col mode (cp.async.bulk.tensor.4d...im2col) gathers,
// for one filter tap (r,s) and one chunk of input channels, the 128 input pixels that feed 128
// consecutive output pixels, applying stride and zero padding in hardware.  A 1x1 / stride-1 /
// unpadded convolution and a plain GEMM use an ordinary tiled 2-d load instead.  B (filters
// repacked to [K_out][R*S][C]) comes through a tiled 3-d load, so the channel tail of a tap is
// zero-filled rather than running into the next tap.  Both land in shared memory in the
// 128/64/32-byte swizzled K-major layout that tcgen05.mma reads through shared-memory descriptors.
//
// One persistent CTA per SM walks its tiles (128 pixels x BN channels):
//   warp 0      producer: waits for a free stage, arms its mbarrier with the byte count, issues TMA
//   warp 1      allocates tensor memory, issues tcgen05.mma (one lane), commits to mbarriers
//   16 warps    staged epilogue: tcgen05.ld the fp32 / int32 accumulators (one TMEM lane = one output pixel per
//               thread), apply the fused epilogue, write 16-byte pieces into a ring of 128-row x 128-byte boxes
//   2 warps     feed the ring (TMA loads of residual boxes) and drain it (TMA stores, plain or through a 4-d map
//               of a head-permuted tensor)
//   (the direct variant, for fp32 / int32 outputs, runs 8 epilogue warps that store rows straight to global memory)
// Two accumulator buffers in tensor memory let the epilogue of tile i overlap the MMAs of tile i+1.
//
// The CTA-pair variant (clusters of two, tcgen05 cta_group::2) computes 256-row tiles across two SMs: each CTA
// loads its own rows of A and half of the filter tile, the first CTA issues the MMAs for both.
//
// Every mbarrier wait is bounded: when the limit expires the waiter records a code in the
// plan's status word, raises a CTA-wide abort flag, and every role falls through to the common
// exit where tensor memory is released.  The host reports ODLA_TIMEOUT.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "epilogue.cuh"

namespace b200 {

namespace {

constexpr int BM = 128;
// Epilogue organisation.  Staged kernels (results leave through the shared-memory ring) run 16 epilogue
// warps on 16-column chunks: four warps per scheduler hide the latency of each other's tensor-memory
// and shared-memory reads, and 16 columns keep a thread under 96 registers.  The direct kernel (fp32 /
// int32 outputs, rows stored straight to global memory) keeps 8 warps on 32-column chunks.
template <bool STAGED> struct EpiCfg {
  static constexpr int kWarps = STAGED ? 16 : 8;     // epilogue warps (a multiple of 4: one per TMEM lane quarter)
  static constexpr int kChunk = STAGED ? 16 : 32;    // accumulator columns per tcgen05.ld
  static constexpr int kLoaderWarp = 2 + kWarps;      // brings residual boxes into the staging ring
  static constexpr int kStorerWarp = 3 + kWarps;      // drains finished boxes with TMA stores
  static constexpr int kThreads = 32 * (4 + kWarps);
};
constexpr int kMaxRing = 8;
constexpr uint32_t kSpinLimit = 1u << 18;  // default number of attempts (up to 4 us each) before a wait gives up: about a second

struct UmmaParams {
  int M_total, K_out, C, R, S, P, Q;
  int stride_h, stride_w, pad_t, pad_l;
  int im2col;          // 1: im2col TMA for A, 0: tiled 2-d TMA
  int kbe;             // elements of K per stage
  int kb_bytes;        // bytes of K per stage: 128, 64 or 32 (= swizzle span)
  int chunks_per_tap;  // ceil(C / kbe)
  int num_kb;          // R*S*chunks_per_tap
  int bps;             // operand boxes (k-blocks) per pipeline stage
  int num_it;          // ceil(num_kb / bps): stage fills per tile
  int BN, stages, m_tiles, n_tiles, total_tiles;
  uint32_t idesc;      // tcgen05 instruction descriptor
  uint32_t desc_hi;    // upper 32 bits of the shared-memory matrix descriptors
  int acc_int;         // accumulators are int32
  int rows_per_batch;  // batched GEMM: output rows per B matrix (0 = one shared B)
  int b_n_major;       // batched GEMM: B boxes hold [k rows][64 columns] (MN-major operand) instead of [n rows][64 k]
  int b_kstep;         // descriptor advance of B per 32 bytes of K, in 16-byte units: 2 (K-major) or 128 (16 rows of 128 bytes)
  int staged;          // epilogue goes through a shared-memory tile and TMA stores
  int res_tma;         // the residual tile is brought into that tile by TMA
  int out_esz;         // bytes per output element
  int stage_boxes;     // 128-row x 128-byte boxes per output tile
  int ring_boxes;      // boxes in the staging ring (>= stage_boxes)
  int box_arrivals;    // epilogue warps that write into one box
  int epi_interleave;  // groups take every fourth chunk instead of a contiguous run
  int pair;            // 1: two CTAs of a cluster share each 256-row tile (tcgen05 cta_group::2), each loading half of B
  int bn_load;         // rows of B this CTA brings into shared memory per k-block (BN, or BN/2 in pair mode)
  int store_mode, store_S, store_NH;  // permuted store through a 4-d map (see UmmaConv)
  int epi_mode;        // kernel variant: 0 direct, 1 staged straight-line forms, 2 staged general form, 3 staged straight-line LeakyReLU form
  int fast_variant;    // mode 1: accumulator conversion (0 fp32, 1 int32 by conversion, 2 int32 by integer add) * 2 + residual
  int tmem_cols;
  uint32_t spin_limit;  // attempts before a bounded wait gives up
  int test_skip_stage;  // test hook: the producer of CTA 0 leaves the last stage of its first tile unarmed, so the MMA lane's wait runs out
  void* y;
  int* status;
  Epilogue ep;
};

// ---------------------------------------------------------------- PTX wrappers ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Same, but the thread may stay suspended in hardware for up to `ns` nanoseconds before the attempt
// reports failure (it resumes at once when the phase completes).  Long suspensions keep waiting warps
// from spending issue slots on polling while the epilogue warps of the same scheduler have work.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the limit expired or another role already aborted.
__device__ __forceinline__ bool mbar_wait_impl(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code, uint32_t limit);
// Debug builds add up, per wait site (and per epilogue group), the cycles block 0 spent waiting.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code, uint32_t limit) {
#ifdef UMMA_DEBUG_TS
  const long long t0 = clock64();
  const bool ok = mbar_wait_impl(bar, parity, abort_flag, status, code, limit);
  const int warp = threadIdx.x >> 5;
  const bool epi = code == 4 || code == 6;
  if (blockIdx.x == 0 && status && (!epi || ((threadIdx.x & 31) == 0 && ((warp - 2) & 3) == 0)))
    atomicAdd((unsigned long long*)status + 32 + code * 4 + (epi ? (warp - 2) >> 2 : 0), (unsigned long long)(clock64() - t0));
  return ok;
#else
  return mbar_wait_impl(bar, parity, abort_flag, status, code, limit);
#endif
}
__device__ __forceinline__ bool mbar_wait_impl(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code, uint32_t limit) {
  if (mbar_try_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait_suspend(bar, parity, 4000u)) return true;
    if ((i & 63) == 63 && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (status) { atomicCAS(status, 0, code); status[1] = (int)blockIdx.x; }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
               "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
               "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c, int w, int h, int n,
                                                   uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(
          smem_u32(dst)),
      "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// ---- CTA-pair (cta_group::2) forms.  Both CTAs of the pair issue their own loads; the byte counts land on
// the barrier of the pair's first CTA (`bar_cluster` is that barrier's shared::cluster address), whose MMA lane
// issues for both and signals barriers in both with a multicast commit.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
               "l"((uint64_t)map), "r"(bar_cluster), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
               "l"((uint64_t)map), "r"(bar_cluster), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster, int c, int w, int h, int n,
                                                        uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(
          smem_u32(dst)),
      "l"((uint64_t)map), "r"(bar_cluster), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
template <int CW> __device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t* r) {
  if (CW == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, naming the registers of the load it completes so that no read of them can be scheduled above it.
template <int N> __device__ __forceinline__ void tmem_ld_wait_regs(uint32_t (&r)[N]);
template <> __device__ __forceinline__ void tmem_ld_wait_regs<16>(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]),
                 "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_wait_regs<32>(uint32_t (&r)[32]) { tmem_ld_wait(); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#ifdef UMMA_DEBUG_TS
#define TS(i) do { if (blockIdx.x == 0 && p.status) { ((unsigned long long*)p.status)[4 + (i)] = gtime(); ((unsigned long long*)p.status)[20 + (i)] = (unsigned long long)clock64(); } } while (0)
#else
#define TS(i) do {} while (0)
#endif
// ------------------------------------------------------------------- epilogue ----
// One thread owns one output pixel (row) and CW consecutive channels held in v[] (registers: every
// index below is a compile-time constant after unrolling).
template <int CW>
__device__ __forceinline__ void load_vec(const float* __restrict__ src, int col0, int kmax, bool full, float (&out)[CW]) {
  if (full) {
#pragma unroll
    for (int q = 0; q < CW / 4; ++q) {
      float4 f = __ldg((const float4*)(src + col0) + q);
      out[4 * q] = f.x; out[4 * q + 1] = f.y; out[4 * q + 2] = f.z; out[4 * q + 3] = f.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < CW; ++j) out[j] = __ldg(src + min(col0 + j, kmax));
  }
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Where a thread's channel segment lives in the shared-memory staging box (128-byte swizzle:
// 16-byte piece j of row r sits at piece j ^ (r & 7)).
struct StagePos {
  uint32_t row_addr;  // shared address of the 128-byte box row
  int j0;             // first 16-byte piece of the segment inside the row
  int rxor;           // r & 7
};
__device__ __forceinline__ uint32_t stage_piece(const StagePos& sp, int q) { return sp.row_addr + (uint32_t)(((sp.j0 + q) ^ sp.rxor) << 4); }

// OUT: the output storage type when known at compile time (DT_F16 / DT_BF16 / DT_S8), or -1 to
// branch on it at run time.  STAGED: results go to the shared-memory staging box and the residual
// (res_smem) is read from it.  `pre`/`use_pre`: residual pieces already fetched into registers (direct
// epilogue).  One instantiation per combination keeps the instruction footprint of the epilogue small:
// with few resident warps an epilogue that overflows the instruction cache stalls on every fetch.
template <int OUT, bool STAGED, int CW>
__device__ __forceinline__ void epilogue_chunk(const UmmaParams& p, float (&v)[CW], int64_t row, int col0, int ncols, const uint4 (&pre)[4], bool use_pre,
                                               const StagePos& sp, bool res_smem_in) {
  const Epilogue& ep = p.ep;
  constexpr bool staged = STAGED;
  const bool res_smem = STAGED && res_smem_in;
  const int out_dt = OUT >= 0 ? OUT : ep.out_dt;
  const bool colsall = ncols == CW;
  const bool full = colsall;                                         // per-channel vectors can be read 16 bytes at a time: col0 is a multiple of CW
  const bool gvec = colsall && (p.K_out & 15) == 0;                  // the row segment in global memory is 16-byte aligned for every element size
  const bool gvec32 = (p.K_out & 3) == 0;                            // ... for 4-byte outputs rows of a multiple of 4 elements are enough
  const int kmax = p.K_out - 1;
  const int64_t base = row * p.K_out + col0;
  float rv[CW];
  const bool has_res = ep.res != nullptr;
  if (has_res) {
    const bool vec = res_smem || use_pre || gvec;
    if (vec && (ep.res_dt == DT_F16 || ep.res_dt == DT_BF16)) {
      constexpr int NQ = CW / 8;
      const uint4* rp = (const uint4*)((const uint16_t*)ep.res + base);
      uint4 u[NQ];
#pragma unroll
      for (int q = 0; q < NQ; ++q) u[q] = res_smem ? lds128(stage_piece(sp, q)) : (use_pre ? pre[q] : __ldg(rp + q));
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float2 f = ep.res_dt == DT_F16 ? __half22float2(((const __half2*)&u[q])[t]) : __bfloat1622float2(((const __nv_bfloat162*)&u[q])[t]);
          rv[q * 8 + 2 * t] = f.x;
          rv[q * 8 + 2 * t + 1] = f.y;
        }
      }
    } else if (vec && ep.res_dt == DT_S8) {
      constexpr int NQ = CW / 16;
      const uint4* rp = (const uint4*)((const int8_t*)ep.res + base);
      uint4 u[NQ];
#pragma unroll
      for (int q = 0; q < NQ; ++q) u[q] = res_smem ? lds128(stage_piece(sp, q)) : (use_pre ? pre[q] : __ldg(rp + q));
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const uint32_t* w = (const uint32_t*)&u[q];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
#pragma unroll
          for (int b = 0; b < 4; ++b) rv[q * 16 + t * 4 + b] = __fmul_rn((float)(signed char)(w[t] >> (8 * b)), ep.res_scale);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < CW; ++j) {
        float r = 0.f;
        if (j < ncols && row < p.M_total) {
          r = load_as_float(ep.res, ep.res_dt, base + j);
          if (ep.res_dt == DT_S8) r = __fmul_rn(r, ep.res_scale);
        }
        rv[j] = r;
      }
    }
  }
  float cv[CW];
  if (ep.mul) {
    load_vec<CW>(ep.mul, col0, kmax, full, cv);
#pragma unroll
    for (int j = 0; j < CW; ++j) v[j] = __fmul_rn(v[j], cv[j]);
  }
  if (ep.alpha != 1.f) {
#pragma unroll
    for (int j = 0; j < CW; ++j) v[j] = __fmul_rn(v[j], ep.alpha);
  }
  if (ep.add1) {
    load_vec<CW>(ep.add1, col0, kmax, full, cv);
#pragma unroll
    for (int j = 0; j < CW; ++j) v[j] = __fadd_rn(v[j], cv[j]);
  }
  if (ep.add2) {
    load_vec<CW>(ep.add2, col0, kmax, full, cv);
#pragma unroll
    for (int j = 0; j < CW; ++j) v[j] = __fadd_rn(v[j], cv[j]);
  }
  if (ep.add_full) {
#pragma unroll
    for (int j = 0; j < CW; ++j)
      if (j < ncols && row < p.M_total) v[j] = __fadd_rn(v[j], __fmul_rn(ep.beta_full, load_as_float(ep.add_full, ep.add_full_dt, base + j)));
  }
  if (ep.act != ACT_NONE && ep.act_first) {
#pragma unroll
    for (int j = 0; j < CW; ++j) v[j] = apply_act(ep.act, v[j], ep.act_a, ep.act_b);
  }
  if (has_res) {
#pragma unroll
    for (int j = 0; j < CW; ++j) v[j] = __fadd_rn(v[j], rv[j]);
  }
  if (ep.act != ACT_NONE && !ep.act_first) {
    if (ep.act == ACT_RELU) {
#pragma unroll
      for (int j = 0; j < CW; ++j) v[j] = fmaxf(v[j], 0.f);
    } else {
#pragma unroll
      for (int j = 0; j < CW; ++j) v[j] = apply_act(ep.act, v[j], ep.act_a, ep.act_b);
    }
  }
  // ---- store ----
  if (out_dt == DT_F16 || out_dt == DT_BF16) {
    constexpr int NQ = CW / 8;
    uint4 u[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      if (out_dt == DT_F16) {
        __half2* h = (__half2*)&u[q];
#pragma unroll
        for (int t = 0; t < 4; ++t) h[t] = __floats2half2_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1]);
      } else {
        __nv_bfloat162* h = (__nv_bfloat162*)&u[q];
#pragma unroll
        for (int t = 0; t < 4; ++t) h[t] = __floats2bfloat162_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1]);
      }
    }
    if (staged) {
#pragma unroll
      for (int q = 0; q < NQ; ++q) sts128(stage_piece(sp, q), u[q]);
    } else if (row < p.M_total) {
      uint16_t* out = (uint16_t*)p.y + base;
      if (gvec) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) ((uint4*)out)[q] = u[q];
      } else {
        const uint16_t* e = (const uint16_t*)u;
#pragma unroll
        for (int j = 0; j < CW; ++j) if (j < ncols) out[j] = e[j];
      }
    }
  } else if (out_dt == DT_S8) {
    constexpr int NQ = CW / 16;
    uint4 u[NQ];
    uint32_t* w = (uint32_t*)u;
#pragma unroll
    for (int t = 0; t < CW / 4; ++t) {
      uint32_t qb[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float t4 = ep.out_multiply ? __fmul_rn(v[t * 4 + b], ep.out_inv) : __fdiv_rn(v[t * 4 + b], ep.out_scale);
        qb[b] = (uint32_t)rne_sat_s8(t4);
      }
      // low bytes of the four results -> one word (three byte permutes)
      w[t] = __byte_perm(__byte_perm(qb[0], qb[1], 0x0040), __byte_perm(qb[2], qb[3], 0x0040), 0x5410);
    }
    if (staged) {
#pragma unroll
      for (int q = 0; q < NQ; ++q) sts128(stage_piece(sp, q), u[q]);
    } else if (row < p.M_total) {
      int8_t* out = (int8_t*)p.y + base;
      if (gvec) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) ((uint4*)out)[q] = u[q];
      } else {
        const int8_t* e = (const int8_t*)u;
#pragma unroll
        for (int j = 0; j < CW; ++j) if (j < ncols) out[j] = e[j];
      }
    }
  } else if (row < p.M_total) {  // DT_F32
    float* out = (float*)p.y + base;
    if (gvec32) {   // whole 16-byte pieces, then at most three single elements (ncols is a multiple of 4 here)
#pragma unroll
      for (int q = 0; q < CW / 4; ++q) if (4 * q + 3 < ncols) ((float4*)out)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < CW; ++j) if (j < ncols) out[j] = v[j];
    }
  }
}

// Two fp32 additions in one instruction (add.rn.f32x2, sm_100): same rounding as two __fadd_rn.
// CAUTION: an add.rn.f32x2 that consumes the result of a mul.rn.f32x2 is contracted into one fused multiply-add by
// the assembler in spite of the .rn qualifiers (measured: 27 % of random inputs differ in the last bit from
// mul-then-add; each instruction on its own, and a packed multiply followed by scalar __fadd_rn, are exact).  A sum
// whose operand comes from fmul2_rn therefore uses __fadd_rn.
__device__ __forceinline__ void fadd2_rn(float& a0, float& a1, float b0, float b1) {
  asm("{\n\t.reg .b64 x, y;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %3};\n\tadd.rn.f32x2 x, x, y;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "f"(b0), "f"(b1));
}
__device__ __forceinline__ void fmul2_rn(float& a0, float& a1, float b0, float b1) {
  asm("{\n\t.reg .b64 x, y;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %3};\n\tmul.rn.f32x2 x, x, y;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "f"(b0), "f"(b1));
}
// Exact conversions without the conversion pipe (its rate, a quarter of the ALU's, bounded the int8 epilogue):
//   int32 -> fp32 for |a| < 2^22: 0x4B400000 is 2^23 + 2^22 = 12582912.f, whose ulp is 1, so adding a to the bit pattern
//     gives 12582912 + a exactly and the subtraction is exact as well;
//   int8 -> fp32: the byte with its sign bit flipped (b + 128, 0..255) placed in the mantissa of 2^23 is 8388608 + 128 + b;
//   fp32 -> int8 with round-to-nearest-even and saturation: clamp to [-128, 127] (or [0, 127] under a ReLU), add
//     12582912.f -- the addition rounds to an integer, ties to even -- and take the low byte (two's complement).
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr float kMagic = 12582912.f;
__device__ __forceinline__ float s8_byte_to_float(uint32_t word_flipped, int b) {
  return __fadd_rn(__uint_as_float(__byte_perm(word_flipped, 0x4B000000u, 0x7540u + (uint32_t)b)), -8388736.f);
}
// The staged epilogue's chunk: 16 consecutive channels of one output row, residual read from and result
// written to the row's place in the staging box.  Only what a staged launch can need is here (the launcher
// sends everything else to the direct epilogue), so the loop around it stays small.
template <int OUT, bool ANYACT>
__device__ __forceinline__ void epilogue_chunk_staged(const UmmaParams& p, float (&v)[16], int col0, const StagePos& sp) {
  const Epilogue& ep = p.ep;
  const bool full = col0 + 16 <= p.K_out;  // the last chunk of a row may be cut short: its vectors are read with clamped indices
  const int kmax = p.K_out - 1;
  float cv[16];
  if (ep.mul) {
    load_vec<16>(ep.mul, col0, kmax, full, cv);
#pragma unroll
    for (int j = 0; j < 16; j += 2) fmul2_rn(v[j], v[j + 1], cv[j], cv[j + 1]);
  }
  if (ep.alpha != 1.f) {
#pragma unroll
    for (int j = 0; j < 16; j += 2) fmul2_rn(v[j], v[j + 1], ep.alpha, ep.alpha);
  }
  const bool after_mul = ep.mul != nullptr || ep.alpha != 1.f;  // v[] comes out of a packed multiplication
  if (ep.add1) {
    load_vec<16>(ep.add1, col0, kmax, full, cv);
    if (after_mul) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __fadd_rn(v[j], cv[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 16; j += 2) fadd2_rn(v[j], v[j + 1], cv[j], cv[j + 1]);
    }
  }
  if (ep.add2) {
    load_vec<16>(ep.add2, col0, kmax, full, cv);
    if (after_mul && !ep.add1) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __fadd_rn(v[j], cv[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 16; j += 2) fadd2_rn(v[j], v[j + 1], cv[j], cv[j + 1]);
    }
  }
  if (ANYACT && ep.act_first) apply_act_all<16>(ep.act, v, ep.act_a, ep.act_b);
  if (p.res_tma) {
    if (OUT == DT_S8) {
      const uint4 u = lds128(stage_piece(sp, 0));
      const uint32_t* w = (const uint32_t*)&u;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t wf = w[t] ^ 0x80808080u;
#pragma unroll
        for (int b = 0; b < 4; b += 2) {
          float r0 = s8_byte_to_float(wf, b), r1 = s8_byte_to_float(wf, b + 1);
          fmul2_rn(r0, r1, ep.res_scale, ep.res_scale);
          v[t * 4 + b] = __fadd_rn(v[t * 4 + b], r0);
          v[t * 4 + b + 1] = __fadd_rn(v[t * 4 + b + 1], r1);
        }
      }
    } else {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const uint4 u = lds128(stage_piece(sp, q));
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = OUT == DT_F16 ? __half22float2(((const __half2*)&u)[t]) : __bfloat1622float2(((const __nv_bfloat162*)&u)[t]);
          if (after_mul && !ep.add1 && !ep.add2) { v[q * 8 + 2 * t] = __fadd_rn(v[q * 8 + 2 * t], f.x); v[q * 8 + 2 * t + 1] = __fadd_rn(v[q * 8 + 2 * t + 1], f.y); }
          else fadd2_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1], f.x, f.y);
        }
      }
    }
  }
  if (ANYACT) {
    if (!ep.act_first) apply_act_all<16>(ep.act, v, ep.act_a, ep.act_b);
  }
  // (plain int8 outputs take their ReLU as the lower bound of the saturating clamp below)
  // (two-byte outputs take their ReLU after packing, two values per instruction: rounding is monotonic and keeps the sign)
  const bool relu_packed = !ANYACT && ep.act == ACT_RELU && OUT != DT_S8;
  if (OUT == DT_S8 && !ANYACT) {
    // requantisation by multiplication; the ReLU (if any) is the lower clamp: max(v, 0) * m == max(v * m, 0) for m > 0
    const float lo = ep.act == ACT_RELU && ep.out_inv > 0.f ? 0.f : -128.f;
    uint4 u;
    uint32_t* w = (uint32_t*)&u;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float q[4];
#pragma unroll
      for (int b = 0; b < 4; b += 2) {
        q[b] = v[t * 4 + b]; q[b + 1] = v[t * 4 + b + 1];
        fmul2_rn(q[b], q[b + 1], ep.out_inv, ep.out_inv);
        q[b] = fminf(fmaxf(q[b], lo), 127.f); q[b + 1] = fminf(fmaxf(q[b + 1], lo), 127.f);
        fadd2_rn(q[b], q[b + 1], kMagic, kMagic);  // (the clamp sits between the multiplication and this addition)
      }
      w[t] = __byte_perm(__byte_perm(__float_as_uint(q[0]), __float_as_uint(q[1]), 0x0040), __byte_perm(__float_as_uint(q[2]), __float_as_uint(q[3]), 0x0040), 0x5410);
    }
    sts128(stage_piece(sp, 0), u);
  } else if (OUT == DT_S8) {
    uint4 u;
    uint32_t* w = (uint32_t*)&u;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t qb[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float t4 = ep.out_multiply ? __fmul_rn(v[t * 4 + b], ep.out_inv) : __fdiv_rn(v[t * 4 + b], ep.out_scale);
        qb[b] = (uint32_t)rne_sat_s8(t4);
      }
      w[t] = __byte_perm(__byte_perm(qb[0], qb[1], 0x0040), __byte_perm(qb[2], qb[3], 0x0040), 0x5410);
    }
    sts128(stage_piece(sp, 0), u);
  } else {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint4 u;
      if (OUT == DT_F16) {
        __half2* h = (__half2*)&u;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          h[t] = __floats2half2_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1]);
          if (relu_packed) h[t] = __hmax2(h[t], __float2half2_rn(0.f));
        }
      } else {
        __nv_bfloat162* h = (__nv_bfloat162*)&u;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          h[t] = __floats2bfloat162_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1]);
          if (relu_packed) h[t] = __hmax2(h[t], __float2bfloat162_rn(0.f));
        }
      }
      sts128(stage_piece(sp, q), u);
    }
  }
}


// The staged epilogue of the common layer forms as straight-line code (MODE 1): every decision that does not depend on
// the data is a template parameter or was made on the host, because the general chunk above spends a fifth of its
// instructions on branches over the launch's configuration.  The launcher guarantees: full 16-column chunks, alpha = 1,
// exactly one per-channel addend (`addv`), a per-channel multiplier exactly when the accumulators are integers,
// activation none or ReLU after the residual, int8 outputs requantised by multiplication.
//   ACC 0: fp32 accumulators; 1: int32 -> fp32 by conversion; 2: int32 -> fp32 by the exact integer-add form (|acc| < 2^22)
//   RES: a residual tile of the output's type waits in the staging box
template <int OUT, int ACC, bool RES>
__device__ __forceinline__ void chunk_fast(const uint32_t (&r)[16], const float* __restrict__ mulv, const float* __restrict__ addv, float res_scale,
                                           float out_inv, float lo, uint32_t relu_floor, const StagePos& sp) {
  float v[16];
  if (ACC == 2) {
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      v[j] = __uint_as_float(r[j] + kMagicBits); v[j + 1] = __uint_as_float(r[j + 1] + kMagicBits);
      fadd2_rn(v[j], v[j + 1], -kMagic, -kMagic);
    }
  } else if (ACC == 1) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = (float)(int32_t)r[j];
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
  }
  float cv[16];
  if (ACC != 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) { const float4 f = __ldg((const float4*)mulv + q); cv[4 * q] = f.x; cv[4 * q + 1] = f.y; cv[4 * q + 2] = f.z; cv[4 * q + 3] = f.w; }
#pragma unroll
    for (int j = 0; j < 16; j += 2) fmul2_rn(v[j], v[j + 1], cv[j], cv[j + 1]);
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) { const float4 f = __ldg((const float4*)addv + q); cv[4 * q] = f.x; cv[4 * q + 1] = f.y; cv[4 * q + 2] = f.z; cv[4 * q + 3] = f.w; }
  if (ACC != 0) {  // the sum consumes a packed product: scalar additions (see fadd2_rn)
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __fadd_rn(v[j], cv[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 16; j += 2) fadd2_rn(v[j], v[j + 1], cv[j], cv[j + 1]);
  }
  if (OUT == DT_S8) {
    if (RES) {
      const uint4 u = lds128(stage_piece(sp, 0));
      const uint32_t* w = (const uint32_t*)&u;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t wf = w[t] ^ 0x80808080u;
#pragma unroll
        for (int b = 0; b < 4; b += 2) {
          float r0 = s8_byte_to_float(wf, b), r1 = s8_byte_to_float(wf, b + 1);
          fmul2_rn(r0, r1, res_scale, res_scale);
          v[t * 4 + b] = __fadd_rn(v[t * 4 + b], r0);
          v[t * 4 + b + 1] = __fadd_rn(v[t * 4 + b + 1], r1);
        }
      }
    }
    uint4 u;
    uint32_t* w = (uint32_t*)&u;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float q[4];
#pragma unroll
      for (int b = 0; b < 4; b += 2) {
        q[b] = v[t * 4 + b]; q[b + 1] = v[t * 4 + b + 1];
        fmul2_rn(q[b], q[b + 1], out_inv, out_inv);
        q[b] = fminf(fmaxf(q[b], lo), 127.f); q[b + 1] = fminf(fmaxf(q[b + 1], lo), 127.f);
        fadd2_rn(q[b], q[b + 1], kMagic, kMagic);  // (the clamp sits between the multiplication and this addition)
      }
      w[t] = __byte_perm(__byte_perm(__float_as_uint(q[0]), __float_as_uint(q[1]), 0x0040), __byte_perm(__float_as_uint(q[2]), __float_as_uint(q[3]), 0x0040), 0x5410);
    }
    sts128(stage_piece(sp, 0), u);
  } else {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint4 u;
      if (RES) {
        u = lds128(stage_piece(sp, q));
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = OUT == DT_F16 ? __half22float2(((const __half2*)&u)[t]) : __bfloat1622float2(((const __nv_bfloat162*)&u)[t]);
          fadd2_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1], f.x, f.y);   // v[] comes out of an addition here
        }
      }
      // ReLU after packing, two values per instruction: rounding is monotonic and keeps the sign; without a ReLU the
      // floor is -inf and the maximum changes nothing
      if (OUT == DT_F16) {
        __half2* h = (__half2*)&u;
        const __half2 fl = *(const __half2*)&relu_floor;
#pragma unroll
        for (int t = 0; t < 4; ++t) h[t] = __hmax2(__floats2half2_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1]), fl);
      } else {
        __nv_bfloat162* h = (__nv_bfloat162*)&u;
        const __nv_bfloat162 fl = *(const __nv_bfloat162*)&relu_floor;
#pragma unroll
        for (int t = 0; t < 4; ++t) h[t] = __hmax2(__floats2bfloat162_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1]), fl);
      }
      sts128(stage_piece(sp, q), u);
    }
  }
}
// One box's share of chunks for one epilogue warp, straight-line form.
template <int OUT, int ACC, bool RES>
__device__ __forceinline__ void box_fast(const UmmaParams& p, uint32_t taddr, int first, int last, int step, int n0, int bx, int chunks_per_box, StagePos sp,
                                         float lo, uint32_t relu_floor) {
  const float res_scale = p.ep.res_scale, out_inv = p.ep.out_inv;
  const float* mulv = p.ep.mul;
  const float* addv = p.ep.add1 ? p.ep.add1 : p.ep.add2;
  const int j_shift = OUT == DT_S8 ? 0 : 1;   // 16 columns are one (int8) or two (16-bit types) 16-byte pieces
#pragma unroll 1
  for (int ch = first; ch < last; ch += step) {
    const int col0 = n0 + ch * 16;
    if (col0 >= p.K_out) break;
    uint32_t r[16];
    tmem_ld16(taddr + (uint32_t)(ch * 16), r);
    tmem_ld_wait_regs<16>(r);
    sp.j0 = (ch - bx * chunks_per_box) << j_shift;
    chunk_fast<OUT, ACC, RES>(r, mulv + col0, addv + col0, res_scale, out_inv, lo, relu_floor, sp);
  }
}

// The Darknet layer form as straight-line code (MODE 3): fp32 accumulators, one per-channel addend, LeakyReLU with a
// slope in [0, 1], then (optionally) the residual tile, two-byte outputs.  For such a slope x < 0 ? fl(a*x) : x equals
// max(x, fl(a*x)): the product rounds monotonically and keeps the sign.
// GELU (erf form) without branches: erf by Abramowitz & Stegun 7.1.26 (absolute error 1.5e-7; the whole expression stays
// within 5e-7 of 0.5 x (1 + erf(x / sqrt 2)), a fraction of an fp16 or bf16 rounding step) -- the library erff takes two
// different paths by magnitude, which a warp's 32 rows then both execute.  Used only where the result is rounded to a
// two-byte type right after.
// Two values at a time with the packed fp32 instructions (fma / mul / add .f32x2): the polynomial and the
// scalings take half the issue slots; reciprocal, exponential, absolute value and sign transfer stay scalar.
__device__ __forceinline__ void ffma2(float& a0, float& a1, float b0, float b1, float c0, float c1) {   // a = a * b + c
  asm("{\n\t.reg .b64 x, y, z;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %3};\n\tmov.b64 z, {%4, %5};\n\tfma.rn.f32x2 x, x, y, z;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void gelu_erf_two_byte_pair(float& t0, float& t1) {
  float z0 = t0, z1 = t1;
  fmul2_rn(z0, z1, 0.70710678118654752440f, 0.70710678118654752440f);
  const float a0 = fabsf(z0), a1 = fabsf(z1);
  float d0 = a0, d1 = a1;
  ffma2(d0, d1, 0.3275911f, 0.3275911f, 1.0f, 1.0f);
  const float k0 = __fdividef(1.0f, d0), k1 = __fdividef(1.0f, d1);
  float p0 = k0, p1 = k1;
  ffma2(p0, p1, 1.061405429f, 1.061405429f, -1.453152027f, -1.453152027f);
  ffma2(p0, p1, k0, k1, 1.421413741f, 1.421413741f);
  ffma2(p0, p1, k0, k1, -0.284496736f, -0.284496736f);
  ffma2(p0, p1, k0, k1, 0.254829592f, 0.254829592f);
  fmul2_rn(p0, p1, -k0, -k1);                       // -(polynomial * k)
  float e0 = a0, e1 = a1;
  fmul2_rn(e0, e1, a0, a1);
  fmul2_rn(e0, e1, -1.4426950408889634f, -1.4426950408889634f);
  asm("ex2.approx.ftz.f32 %0, %0;" : "+f"(e0));
  asm("ex2.approx.ftz.f32 %0, %0;" : "+f"(e1));
  ffma2(p0, p1, e0, e1, 1.0f, 1.0f);                // 1 - polynomial * k * exp(-z^2)
  p0 = copysignf(p0, z0); p1 = copysignf(p1, z1);
  fadd2_rn(p0, p1, 1.0f, 1.0f);
  fmul2_rn(t0, t1, 0.5f, 0.5f);
  fmul2_rn(t0, t1, p0, p1);
}
// ACTF 0: LeakyReLU, 1: GELU (erf form)
template <int OUT, int ACTF, bool RES>
__device__ __forceinline__ void chunk_leaky(const uint32_t (&r)[16], const float* __restrict__ addv, float slope, const StagePos& sp) {
  float v[16], cv[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
#pragma unroll
  for (int q = 0; q < 4; ++q) { const float4 f = __ldg((const float4*)addv + q); cv[4 * q] = f.x; cv[4 * q + 1] = f.y; cv[4 * q + 2] = f.z; cv[4 * q + 3] = f.w; }
#pragma unroll
  for (int j = 0; j < 16; j += 2) {
    fadd2_rn(v[j], v[j + 1], cv[j], cv[j + 1]);
    if (ACTF == 0) {
      float t0 = v[j], t1 = v[j + 1];
      fmul2_rn(t0, t1, slope, slope);
      v[j] = fmaxf(v[j], t0); v[j + 1] = fmaxf(v[j + 1], t1);   // (a maximum between the product and any later sum: nothing to contract)
    } else {
      gelu_erf_two_byte_pair(v[j], v[j + 1]);
    }
  }
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint4 u;
    if (RES) {
      u = lds128(stage_piece(sp, q));
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = OUT == DT_F16 ? __half22float2(((const __half2*)&u)[t]) : __bfloat1622float2(((const __nv_bfloat162*)&u)[t]);
        fadd2_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1], f.x, f.y);
      }
    }
    if (OUT == DT_F16) {
      __half2* h = (__half2*)&u;
#pragma unroll
      for (int t = 0; t < 4; ++t) h[t] = __floats2half2_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1]);
    } else {
      __nv_bfloat162* h = (__nv_bfloat162*)&u;
#pragma unroll
      for (int t = 0; t < 4; ++t) h[t] = __floats2bfloat162_rn(v[q * 8 + 2 * t], v[q * 8 + 2 * t + 1]);
    }
    sts128(stage_piece(sp, q), u);
  }
}
template <int OUT, int ACTF, bool RES>
__device__ __forceinline__ void box_leaky(const UmmaParams& p, uint32_t taddr, int first, int last, int step, int n0, int bx, int chunks_per_box, StagePos sp) {
  const float slope = p.ep.act_a;
  const float* addv = p.ep.add1 ? p.ep.add1 : p.ep.add2;
#pragma unroll 1
  for (int ch = first; ch < last; ch += step) {
    const int col0 = n0 + ch * 16;
    if (col0 >= p.K_out) break;
    uint32_t r[16];
    tmem_ld16(taddr + (uint32_t)(ch * 16), r);
    tmem_ld_wait_regs<16>(r);
    sp.j0 = (ch - bx * chunks_per_box) << 1;
    chunk_leaky<OUT, ACTF, RES>(r, addv + col0, slope, sp);
  }
}

// The int8 form of a transformer's first feed-forward layer: int32 accumulators, per-channel multiplier and addend,
// GELU, requantisation by multiplication to int8.  ACC as in chunk_fast (1: conversion, 2: exact integer-add form).
template <int ACC>
__device__ __forceinline__ void chunk_gelu_s8(const uint32_t (&r)[16], const float* __restrict__ mulv, const float* __restrict__ addv, float out_inv, const StagePos& sp) {
  float v[16], cv[16];
  if (ACC == 2) {
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      v[j] = __uint_as_float(r[j] + kMagicBits); v[j + 1] = __uint_as_float(r[j + 1] + kMagicBits);
      fadd2_rn(v[j], v[j + 1], -kMagic, -kMagic);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = (float)(int32_t)r[j];
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) { const float4 f = __ldg((const float4*)mulv + q); cv[4 * q] = f.x; cv[4 * q + 1] = f.y; cv[4 * q + 2] = f.z; cv[4 * q + 3] = f.w; }
#pragma unroll
  for (int j = 0; j < 16; j += 2) fmul2_rn(v[j], v[j + 1], cv[j], cv[j + 1]);
#pragma unroll
  for (int q = 0; q < 4; ++q) { const float4 f = __ldg((const float4*)addv + q); cv[4 * q] = f.x; cv[4 * q + 1] = f.y; cv[4 * q + 2] = f.z; cv[4 * q + 3] = f.w; }
#pragma unroll
  for (int j = 0; j < 16; j += 2) {   // scalar sums after a packed product (see fadd2_rn)
    v[j] = __fadd_rn(v[j], cv[j]); v[j + 1] = __fadd_rn(v[j + 1], cv[j + 1]);
    gelu_erf_two_byte_pair(v[j], v[j + 1]);
  }
  uint4 u;
  uint32_t* w = (uint32_t*)&u;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    float q[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) q[b] = __fadd_rn(fminf(fmaxf(__fmul_rn(v[t * 4 + b], out_inv), -128.f), 127.f), kMagic);
    w[t] = __byte_perm(__byte_perm(__float_as_uint(q[0]), __float_as_uint(q[1]), 0x0040), __byte_perm(__float_as_uint(q[2]), __float_as_uint(q[3]), 0x0040), 0x5410);
  }
  sts128(stage_piece(sp, 0), u);
}
template <int ACC>
__device__ __forceinline__ void box_gelu_s8(const UmmaParams& p, uint32_t taddr, int first, int last, int step, int n0, int bx, int chunks_per_box, StagePos sp) {
  const float out_inv = p.ep.out_inv;
  const float* mulv = p.ep.mul;
  const float* addv = p.ep.add1 ? p.ep.add1 : p.ep.add2;
#pragma unroll 1
  for (int ch = first; ch < last; ch += step) {
    const int col0 = n0 + ch * 16;
    if (col0 >= p.K_out) break;
    uint32_t r[16];
    tmem_ld16(taddr + (uint32_t)(ch * 16), r);
    tmem_ld_wait_regs<16>(r);
    sp.j0 = ch - bx * chunks_per_box;
    chunk_gelu_s8<ACC>(r, mulv + col0, addv + col0, out_inv, sp);
  }
}

// --------------------------------------------------------------------- kernel ----
// MODE 3: staged epilogue, further straight-line forms: LeakyReLU before the optional residual (Darknet) or GELU, two-byte
//         outputs (box_leaky); int8 operands, GELU, requantised int8 output (box_gelu_s8).
// MODE 0: direct epilogue (any output type, rows written straight to global memory).
// MODE 1: staged epilogue, straight-line forms (box_fast): activation none / ReLU after the residual, one per-channel
//         addend, int8 requantisation by multiplication.
// MODE 2: staged epilogue, general form: every activation, activation before the residual, division requantisation,
//         any combination of per-channel vectors, a ragged last chunk.
// PAIR: CTA-pair variant (its cta_group::2 instructions make the kernel launchable only as clusters of two).
template <int OUT, int MODE, bool PAIR>
__global__ void __launch_bounds__(EpiCfg<MODE != 0>::kThreads, 1)
umma_conv_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmY,
                 const __grid_constant__ CUtensorMap tmR, const UmmaParams p) {
  constexpr bool STAGED = MODE != 0;
  constexpr int kPair = PAIR ? 1 : 0;
  constexpr int kEpilogueWarps = EpiCfg<STAGED>::kWarps, kLoaderWarp = EpiCfg<STAGED>::kLoaderWarp, kStorerWarp = EpiCfg<STAGED>::kStorerWarp;
  constexpr int CW = EpiCfg<STAGED>::kChunk;
  extern __shared__ uint8_t smem_raw[];
  if (threadIdx.x == 0) TS(7);
  // operand stages start on a 1024-byte boundary (the 128-byte swizzle repeats every 1024 bytes)
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stage_bytes = p.bps * (BM + p.bn_load) * p.kb_bytes;
  uint8_t* staging = smem + (size_t)p.stages * stage_bytes;   // 1024-byte aligned: stage sizes are multiples of 2 KiB
  uint8_t* ctrl = staging + (size_t)p.ring_boxes * 16384;
  uint64_t* full_bar = (uint64_t*)ctrl;            // [stages]
  uint64_t* empty_bar = full_bar + 16;             // [stages]
  uint64_t* tfull_bar = empty_bar + 16;            // [2]
  uint64_t* tempty_bar = tfull_bar + 2;            // [2]
  uint64_t* box_full = tempty_bar + 2;             // [ring] box is armed: free, and its residual (if any) has landed
  uint64_t* box_done = box_full + kMaxRing;        // [ring] every epilogue warp that owns part of the box has written it
  uint64_t* box_free = box_done + kMaxRing;        // [ring] the TMA store has finished reading the box
  uint32_t* tmem_slot = (uint32_t*)(box_free + kMaxRing);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    // in pair mode the epilogue warps of both CTAs release an accumulator on the first CTA's barrier
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], (uint32_t)(kEpilogueWarps << kPair)); }
    for (int b = 0; b < kMaxRing; ++b) { mbar_init(&box_full[b], 1); mbar_init(&box_done[b], (uint32_t)p.box_arrivals); mbar_init(&box_free[b], 1); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if constexpr (PAIR) cluster_sync_all();  // the peer's barriers exist before anything of this CTA can reach them
  if (warp == 1) {
    if constexpr (PAIR) {  // the same warp of both CTAs allocates the same columns in both tensor memories
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)p.tmem_cols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)p.tmem_cols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: everything above overlapped the previous kernel's tail; from here on
  // this kernel reads what that kernel wrote.  The next kernel may start its own prologue now.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) TS(0);

  const uint32_t a_box = (uint32_t)(BM * p.kb_bytes), b_box = (uint32_t)(p.bn_load * p.kb_bytes);
  // Tile walk: a unit (a CTA, or a CTA pair) takes every `tile_step`-th tile; in pair mode a tile is 256 rows and
  // this CTA owns the half given by its rank in the cluster.
  const int rank = PAIR ? (int)cluster_ctarank() : 0;
  const int tile_first = (int)(blockIdx.x >> kPair), tile_step = (int)(gridDim.x >> kPair);
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer ----
    // One lane runs this loop; it is kept free of divisions (filter tap, channel chunk, stage and
    // phase are running counters) because its instruction rate bounds the rate of k-blocks.
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = tile_first; tile < p.total_tiles && ok; tile += tile_step) {
        const int m0 = (((tile % p.m_tiles) << kPair) + rank) * BM, n0 = (tile / p.m_tiles) * p.BN;
        int w0 = 0, h0 = 0, img = 0;
        if (p.im2col) {
          const int pq = p.P * p.Q;
          img = m0 / pq;
          const int rem = m0 - img * pq;
          const int op = rem / p.Q, oq = rem - op * p.Q;
          w0 = oq * p.stride_w - p.pad_l;
          h0 = op * p.stride_h - p.pad_t;
        }
        int tap = 0, fr = 0, fs = 0, c0 = 0, left = p.num_kb;
        const int bidx = p.rows_per_batch ? m0 / p.rows_per_batch : 0;
        for (int it = 0; it < p.num_it; ++it) {
          if (!mbar_wait(empty_bar + s, ph ^ 1, abort_flag, p.status, 1, p.spin_limit)) { ok = false; break; }
          const int nb = left < p.bps ? left : p.bps;
          left -= nb;
          uint8_t* sa = smem + (size_t)s * stage_bytes;
          uint8_t* sb = sa + (size_t)p.bps * a_box;
          uint64_t* fb = full_bar + s;
          if constexpr (PAIR) {
            // the first CTA's barrier counts the bytes of both CTAs; only it is armed
            if (rank == 0) mbar_expect_tx(fb, 2u * (uint32_t)nb * (a_box + b_box));
            const uint32_t fbc = map_to_cta(smem_u32(fb), 0);
            const int nb0 = n0 + rank * p.bn_load;
            for (int j = 0; j < nb; ++j) {
              if (p.im2col) tma_load_im2col_4d_pair(sa, &tmA, fbc, c0, w0, h0, img, (uint16_t)fs, (uint16_t)fr);
              else tma_load_2d_pair(sa, &tmA, fbc, c0, m0);
              if (p.rows_per_batch) tma_load_3d_pair(sb, &tmB, fbc, c0, nb0, bidx);
              else tma_load_3d_pair(sb, &tmB, fbc, c0, tap, nb0);
              sa += a_box;
              sb += b_box;
              c0 += p.kbe;
              if (c0 >= p.C) {
                c0 = 0;
                ++tap;
                if (++fs == p.S) { fs = 0; if (++fr == p.R) fr = 0; }   // the next filter term walks the window again
              }
            }
            if (++s == p.stages) { s = 0; ph ^= 1; }
            continue;
          }
          // Test hook (never set by the planner): this stage is neither armed nor loaded, so its barrier can never
          // complete and the MMA lane's bounded wait reports a timeout; nothing faults and nothing spins for ever.
          const bool skip = p.test_skip_stage && blockIdx.x == 0 && tile == tile_first && it == p.num_it - 1;
          if (!skip) mbar_expect_tx(fb, (uint32_t)nb * (a_box + b_box));
          for (int j = 0; j < nb; ++j) {
            if (skip) {}
            else if (p.im2col) tma_load_im2col_4d(sa, &tmA, fb, c0, w0, h0, img, (uint16_t)fs, (uint16_t)fr);
            else tma_load_2d(sa, &tmA, fb, c0, m0);
            if (skip) {}
            else if (p.rows_per_batch) tma_load_3d(sb, &tmB, fb, p.b_n_major ? n0 : c0, p.b_n_major ? c0 : n0, bidx);
            else tma_load_3d(sb, &tmB, fb, c0, tap, n0);
            sa += a_box;
            sb += b_box;
            c0 += p.kbe;
            if (c0 >= p.C) {
              c0 = 0;
              ++tap;
              if (++fs == p.S) { fs = 0; if (++fr == p.R) fr = 0; }   // the next filter term walks the window again
            }
          }
          if (++s == p.stages) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) {
        // give copies already in flight a bounded chance to land before shared memory goes away
        for (int i = 0; i < p.stages; ++i)
          for (uint32_t k = 0; k < 4096; ++k)
            if (mbar_try_wait(&full_bar[i], 0) || mbar_try_wait(&full_bar[i], 1)) break;
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer ----
    if (rank == 0 && elect_one()) {  // in pair mode the first CTA's lane issues for both
      int s = 0;
      uint32_t ph = 0, tcount = 0;
      bool ok = true;
      const uint32_t smem_base = smem_u32(smem);
      const uint64_t desc_fixed = ((uint64_t)p.desc_hi << 32) | (1ull << 16);
      const int ksteps = p.kb_bytes >> 5;  // 32 bytes of K per instruction
      for (int tile = tile_first; tile < p.total_tiles && ok; tile += tile_step, ++tcount) {
        const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_flag, p.status, 2, p.spin_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * (uint32_t)p.BN;
        int left = p.num_kb;
        uint32_t accum = 0;
        for (int it = 0; it < p.num_it; ++it) {
          if (!mbar_wait(full_bar + s, ph, abort_flag, p.status, 3, p.spin_limit)) { ok = false; break; }
          tc_fence_after();
          const int nb = left < p.bps ? left : p.bps;
          left -= nb;
          uint32_t sa = smem_base + (uint32_t)s * (uint32_t)stage_bytes, sb = sa + (uint32_t)p.bps * a_box;
          for (int j = 0; j < nb; ++j) {
            const uint64_t da = desc_fixed | (uint64_t)((sa & 0x3FFFF) >> 4);
            const uint64_t db = desc_fixed | (uint64_t)((sb & 0x3FFFF) >> 4);
            for (int k = 0; k < ksteps; ++k) {
              if constexpr (PAIR) {
                if (p.acc_int) umma_i8_pair(tmem_d, da + 2 * k, db + 2 * k, p.idesc, accum);
                else umma_f16_pair(tmem_d, da + 2 * k, db + 2 * k, p.idesc, accum);
              } else {
                if (p.acc_int) umma_i8(tmem_d, da + 2 * k, db + 2 * k, p.idesc, accum);
                else umma_f16(tmem_d, da + 2 * k, db + (uint64_t)(p.b_kstep * k), p.idesc, accum);
              }
              accum = 1;
            }
            sa += a_box;
            sb += b_box;
          }
          if constexpr (PAIR) umma_commit_pair(empty_bar + s); else umma_commit(empty_bar + s);  // frees the stage once these MMAs have read it
          if (++s == p.stages) { s = 0; ph ^= 1; }
        }
        if (ok) { if constexpr (PAIR) umma_commit_pair(&tfull_bar[acc]); else umma_commit(&tfull_bar[acc]); }  // accumulator complete
        if (tcount == 0) TS(3);
      }
    }
  } else if (warp == kLoaderWarp) {
    // -------------------------------------------- staging ring: arm boxes (residual loads) ----
    if (STAGED && elect_one()) {
      const int cols_per_box = 128 / p.out_esz;
      int slot = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = tile_first; tile < p.total_tiles && ok; tile += tile_step) {
        const int m0 = (((tile % p.m_tiles) << kPair) + rank) * BM, n0 = (tile / p.m_tiles) * p.BN;
        for (int bx = 0; bx < p.stage_boxes; ++bx) {
          const int x0 = n0 + bx * cols_per_box;
          if (x0 >= p.K_out) break;
          if (!mbar_wait(box_free + slot, ph ^ 1, abort_flag, p.status, 5, p.spin_limit)) { ok = false; break; }
          if (p.res_tma) {
            mbar_expect_tx(box_full + slot, 16384u);
            tma_load_2d(staging + slot * 16384, &tmR, box_full + slot, x0, m0);
          } else {
            mbar_arrive(box_full + slot);
          }
          if (++slot == p.ring_boxes) { slot = 0; ph ^= 1; }
        }
      }
      if (!ok && p.res_tma) {
        // residual loads already in flight get a bounded chance to land before shared memory goes away
        for (int i = 0; i < p.ring_boxes; ++i)
          for (uint32_t k = 0; k < 4096; ++k)
            if (mbar_try_wait(&box_full[i], 0) || mbar_try_wait(&box_full[i], 1)) break;
      }
    }
  } else if (warp == kStorerWarp) {
    // ------------------------------------------------ staging ring: store finished boxes ----
    if (STAGED && elect_one()) {
      const int cols_per_box = 128 / p.out_esz;
      const uint32_t staging_u32 = smem_u32(staging);
      int slot = 0, prev = -1;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = tile_first; tile < p.total_tiles && ok; tile += tile_step) {
        const int m0 = (((tile % p.m_tiles) << kPair) + rank) * BM, n0 = (tile / p.m_tiles) * p.BN;
        for (int bx = 0; bx < p.stage_boxes; ++bx) {
          const int x0 = n0 + bx * cols_per_box;
          if (x0 >= p.K_out) break;
          // Nothing to send yet: use the wait to let the last store finish reading its box and hand that box back,
          // so that the next tile's epilogue never waits for this tile's boxes to be stored.
          if (prev >= 0 && !mbar_try_wait(box_done + slot, ph)) {
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            mbar_arrive(box_free + prev);
            prev = -1;
          }
          if (!mbar_wait(box_done + slot, ph, abort_flag, p.status, 7, p.spin_limit)) { ok = false; break; }
          if (p.store_mode == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"((uint64_t)&tmY),
                         "r"(staging_u32 + (uint32_t)slot * 16384u), "r"(x0), "r"(m0)
                         : "memory");
          } else {
            // the 128 rows of the box are one run of sequence positions of one batch element; its columns one head
            const int g = m0 / p.store_S, s0 = m0 - g * p.store_S;
            int c1, c2, c3;
            if (p.store_mode == 1) { c1 = s0; c2 = x0 / cols_per_box; c3 = g; }                                   // [B][NH][S][D]
            else { const int b = g / p.store_NH; c1 = g - b * p.store_NH; c2 = s0; c3 = b; }                      // [B][S][NH][D]
            asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"((uint64_t)&tmY),
                         "r"(staging_u32 + (uint32_t)slot * 16384u), "r"(0), "r"(c1), "r"(c2), "r"(c3)
                         : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          if (prev >= 0) {
            asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // every store but the newest has read its box
            mbar_arrive(box_free + prev);
          }
          prev = slot;
          if (++slot == p.ring_boxes) { slot = 0; ph ^= 1; }
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // stores complete before shared memory is released
    }
  } else {
    // ---------------------------------------------------------------- epilogue ----
    const int quarter = warp & 3;  // the TMEM lanes this warp may read: 32*quarter .. +31
    const int cgroup = (warp - 2) >> 2;  // the warps of a quarter take the 32-column chunks round-robin
    uint32_t tcount = 0;
    bool ok = true;
    constexpr int kGroups = kEpilogueWarps / 4;            // warps per TMEM lane quarter
    constexpr int kChunksPerWarp = 8 / kGroups;            // BN <= 256 -> at most 8 chunks of 32 columns
    const int r_in_tile = quarter * 32 + lane;
    const uint32_t staging_u32 = smem_u32(staging);
    if constexpr (STAGED) {
      // Per output tile the staging ring supplies stage_boxes boxes of 128 rows x 128 bytes; the
      // loader warp has already put the residual there, this warp overwrites its part of the box
      // with the result and the storer warp sends the box out.
      const int cols_per_box = 128 / p.out_esz, chunks_per_box = cols_per_box / CW;
      // Which 16-column chunks of a tile the four warps of a group (one per lane quarter) take: either a
      // contiguous run, so that a group fills and hands over a box (or its share of one) on its own while the
      // other groups work on other boxes, or every fourth chunk, so that all groups finish box after box together.
      const int n_chunks = p.BN / CW, per_group = n_chunks / kGroups;  // per group: 1, 2 or 4 chunks
      const int ch_lo = cgroup * per_group, ch_hi = ch_lo + per_group;
      int slot = 0;
      uint32_t ph = 0;
      // ReLU of the straight-line forms: the lower clamp of an int8 output, a packed floor for 16-bit outputs
      const bool fast_relu = p.ep.act == ACT_RELU;
      const float fast_lo = fast_relu ? 0.f : -128.f;
      const uint32_t fast_floor = fast_relu ? 0u : (OUT == DT_F16 ? 0xFC00FC00u : 0xFF80FF80u);
      for (int tile = tile_first; tile < p.total_tiles && ok; tile += tile_step, ++tcount) {
        const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
        const int n0 = (tile / p.m_tiles) * p.BN;
        if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, p.status, 4, p.spin_limit)) { ok = false; break; }
        tc_fence_after();
        if (tcount == 0 && threadIdx.x == 64) TS(4);
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * (uint32_t)p.BN;
        for (int bx = 0; bx < p.stage_boxes && ok; ++bx) {
          if (n0 + bx * cols_per_box >= p.K_out) break;
          int first, last, step;
          if (p.epi_interleave) { first = bx * chunks_per_box + cgroup; last = min((bx + 1) * chunks_per_box, n_chunks); step = kGroups; }
          else { first = max(ch_lo, bx * chunks_per_box); last = min(ch_hi, (bx + 1) * chunks_per_box); step = 1; }
          if (first < last) {
            if (!mbar_wait(box_full + slot, ph, abort_flag, p.status, 6, p.spin_limit)) { ok = false; break; }
            StagePos sp;
            sp.row_addr = staging_u32 + (uint32_t)slot * 16384u + (uint32_t)r_in_tile * 128u;
            sp.rxor = r_in_tile & 7;
            if constexpr (MODE == 1) {
              // straight-line forms, chosen once per launch on the host (p.fast_variant = ACC * 2 + RES)
              switch (p.fast_variant) {
                case 0: box_fast<OUT, 0, false>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp, fast_lo, fast_floor); break;
                case 1: box_fast<OUT, 0, true>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp, fast_lo, fast_floor); break;
                case 2: box_fast<OUT, 1, false>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp, fast_lo, fast_floor); break;
                case 3: box_fast<OUT, 1, true>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp, fast_lo, fast_floor); break;
                case 4: box_fast<OUT, 2, false>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp, fast_lo, fast_floor); break;
                default: box_fast<OUT, 2, true>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp, fast_lo, fast_floor); break;
              }
            } else if constexpr (MODE == 3) {
              if constexpr (OUT == DT_S8) {
                if (p.ep.acc_small) box_gelu_s8<2>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp);
                else box_gelu_s8<1>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp);
              }
              if constexpr (OUT == DT_F16 || OUT == DT_BF16) {
                if (p.ep.act == ACT_GELU_ERF) box_leaky<OUT, 1, false>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp);
                else if (p.ep.res) box_leaky<OUT, 0, true>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp);
                else box_leaky<OUT, 0, false>(p, taddr, first, last, step, n0, bx, chunks_per_box, sp);
              }
            } else {
#pragma unroll 1
            for (int ch = first; ch < last; ch += step) {
              const int col0 = n0 + ch * CW;
              if (col0 >= p.K_out) break;  // columns past K_out inside a chunk are computed and then clipped by the store
              uint32_t r[CW];
              tmem_ld<CW>(taddr + (uint32_t)(ch * CW), r);
              tmem_ld_wait_regs<CW>(r);
              float v[CW];
              if (p.acc_int) {
                if (p.ep.acc_small) {
#pragma unroll
                  for (int j = 0; j < CW; j += 2) {
                    v[j] = __uint_as_float(r[j] + kMagicBits); v[j + 1] = __uint_as_float(r[j + 1] + kMagicBits);
                    fadd2_rn(v[j], v[j + 1], -kMagic, -kMagic);
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < CW; ++j) v[j] = (float)(int32_t)r[j];
                }
              } else {
#pragma unroll
                for (int j = 0; j < CW; ++j) v[j] = __uint_as_float(r[j]);
              }
              sp.j0 = ((ch - bx * chunks_per_box) * CW * p.out_esz) >> 4;
              epilogue_chunk_staged<OUT, true>(p, v, col0, sp);
            }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the bulk-copy engine must see these writes
            __syncwarp();
            if (lane == 0) mbar_arrive(box_done + slot);
          }
          if (++slot == p.ring_boxes) { slot = 0; ph ^= 1; }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) { if (PAIR && rank) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0)); else mbar_arrive(&tempty_bar[acc]); }
        if (tcount == 0 && threadIdx.x == 64) TS(5);
      }
    } else {
      // Direct epilogue: rows go straight to global memory.  Residual rows can be fetched before the
      // accumulator is ready: they only depend on the tile.
      const bool res_vec = p.ep.res && (p.K_out & 15) == 0 && (p.ep.res_dt == DT_F16 || p.ep.res_dt == DT_BF16 || p.ep.res_dt == DT_S8);
      const int res_q = p.ep.res_dt == DT_S8 ? 2 : 4;       // 16-byte pieces per 32 channels
      const int res_esz = p.ep.res_dt == DT_S8 ? 1 : 2;
      for (int tile = tile_first; tile < p.total_tiles && ok; tile += tile_step, ++tcount) {
        const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
        const int m0 = (((tile % p.m_tiles) << kPair) + rank) * BM, n0 = (tile / p.m_tiles) * p.BN;
        const int64_t row = (int64_t)m0 + r_in_tile;
        uint4 pre[kChunksPerWarp][4] = {};
        bool pre_ok[kChunksPerWarp] = {};
#pragma unroll
        for (int i = 0; i < kChunksPerWarp; ++i) {
          const int c = (cgroup + kGroups * i) * 32, col0 = n0 + c;
          pre_ok[i] = res_vec && c < p.BN && row < p.M_total && col0 + 32 <= p.K_out;
          if (pre_ok[i]) {
            const uint4* rp = (const uint4*)((const char*)p.ep.res + (row * p.K_out + col0) * res_esz);
#pragma unroll
            for (int q = 0; q < 4; ++q) if (q < res_q) pre[i][q] = __ldg(rp + q);
          }
        }
        if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, p.status, 4, p.spin_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * (uint32_t)p.BN;
#pragma unroll
        for (int i = 0; i < kChunksPerWarp; ++i) {
          const int c = (cgroup + kGroups * i) * 32, col0 = n0 + c;
          if (c >= p.BN || col0 >= p.K_out) break;  // uniform across the warp
          uint32_t r[32];
          tmem_ld32(taddr + (uint32_t)c, r);
          tmem_ld_wait();
          const int ncols = min(32, p.K_out - col0);
          if (p.ep.out_dt == DT_S32) {
            if (row < p.M_total) {
              int32_t* out = (int32_t*)p.y + row * p.K_out + col0;
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < ncols) out[j] = (int32_t)r[j];
            }
          } else if (row < p.M_total) {
            float v[32];
            if (p.acc_int) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = (float)(int32_t)r[j];
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            }
            StagePos sp = {0, 0, 0};
            epilogue_chunk<OUT, false, 32>(p, v, row, col0, ncols, pre[i], pre_ok[i], sp, false);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) { if (PAIR && rank) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0)); else mbar_arrive(&tempty_bar[acc]); }
      }
    }
  }
  // ------------------------------------------------------------------ teardown ----
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TS(6);
  if constexpr (PAIR) cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
  }
}

// ------------------------------------------------------------ fused attention ----
// softmax(scale * Q K^T) V for heads of 128 positions x 64 channels (two-byte types): one CTA works on one head at a
// time and keeps the 128 x 128 scores in tensor memory -- they never reach global memory.  Roles: warp 0 brings Q, K, V
// in with TMA and sends the result out, warp 1 issues the two products, warps 2-5 (one TMEM lane quarter each, a thread
// per query row) do the soft-max between them and the final scaling.  Shared memory holds one head (no double buffer)
// and is reused inside the head -- the probabilities overwrite Q and K, the result accumulates over the scores' tensor
// memory columns, the result box overwrites V -- so that four CTAs share an SM and fill each other's gaps.  The probabilities go to the second product unnormalised
// (exp(s - max), rounded to the two-byte type) and the row sums divide the result, as in any online soft-max.
struct AttnParams {
  int tiles, NH, merge;          // heads in all; heads per batch element; 1: the result is stored [B][S][NH][D], 0: [B][NH][S][D]
  float scale_log2e;             // scale * log2(e)
  uint32_t idesc_s, idesc_o, desc_hi;
  uint32_t spin_limit;
  int bf16;
  int* status;
};
constexpr int kAttnS = 128, kAttnD = 64, kAttnThreads = 192;
constexpr uint32_t kAttnBox = 16384;   // 128 rows x 128 bytes

template <bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 4)
attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
            const __grid_constant__ CUtensorMap tmY, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                 // [128 rows][64] K-major
  uint8_t* sK = sQ + kAttnBox;        // [128 keys][64] K-major
  uint8_t* sV = sK + kAttnBox;        // [128 keys][64 channels]: the second product reads it MN-major
  uint8_t* sP = sQ;                   // two k-blocks of [128 rows][64 keys], written once the first product has read Q and K
  uint8_t* sY = sV;                   // result box, written once the second product has read V
  uint64_t* bars = (uint64_t*)(sV + kAttnBox);
  uint64_t *b_full = bars, *b_s = bars + 1, *b_p = bars + 2, *b_o = bars + 3, *b_e = bars + 4, *b_sf = bars + 5;
  uint32_t* tmem_slot = (uint32_t*)(bars + 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(b_full, 1); mbar_init(b_s, 1); mbar_init(b_p, 4); mbar_init(b_o, 1); mbar_init(b_e, 4); mbar_init(b_sf, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base;   // the result's 64 columns replace the first 64 of the scores

  if (warp == 0) {
    // ------------------------------------------------ loads and the result's store ----
    if (elect_one()) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++it) {
        // the previous head's products have finished reading Q, K, V and P
        if (it > 0 && !mbar_wait(b_o, (it - 1) & 1, abort_flag, p.status, 11, p.spin_limit)) break;
        mbar_expect_tx(b_full, 3u * kAttnBox);
        tma_load_2d(sQ, &tmQ, b_full, 0, tile * kAttnS);
        tma_load_2d(sK, &tmK, b_full, 0, tile * kAttnS);
        tma_load_2d(sV, &tmV, b_full, 0, tile * kAttnS);
        if (!mbar_wait(b_e, it & 1, abort_flag, p.status, 12, p.spin_limit)) break;
        if (p.merge) {
          const int b = tile / p.NH, h = tile - b * p.NH;
          asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"((uint64_t)&tmY), "r"(smem_u32(sY)), "r"(0),
                       "r"(h), "r"(0), "r"(b)
                       : "memory");
        } else {
          asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"((uint64_t)&tmY), "r"(smem_u32(sY)), "r"(0),
                       "r"(tile * kAttnS)
                       : "memory");
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        mbar_arrive(b_sf);
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      // copies that were armed but never consumed (an aborted run) get a bounded chance to land
      if (*abort_flag)
        for (uint32_t k = 0; k < 4096; ++k)
          if (mbar_try_wait(b_full, 0) || mbar_try_wait(b_full, 1)) break;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- the two products ----
    if (elect_one()) {
      const uint64_t fixed = ((uint64_t)p.desc_hi << 32) | (1ull << 16);
      const uint64_t dq = fixed | (uint64_t)((smem_u32(sQ) & 0x3FFFF) >> 4), dk = fixed | (uint64_t)((smem_u32(sK) & 0x3FFFF) >> 4);
      const uint64_t dv = fixed | (uint64_t)((smem_u32(sV) & 0x3FFFF) >> 4), dp = fixed | (uint64_t)((smem_u32(sP) & 0x3FFFF) >> 4);
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++it) {
        if (!mbar_wait(b_full, it & 1, abort_flag, p.status, 13, p.spin_limit)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16(tmem_s, dq + 2 * k, dk + 2 * k, p.idesc_s, k ? 1u : 0u);        // S = Q K^T, 64 deep
        umma_commit(b_s);
        if (!mbar_wait(b_p, it & 1, abort_flag, p.status, 14, p.spin_limit)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)   // O = P V, 128 deep: P advances 32 bytes per step inside a k-block, V sixteen rows
          umma_f16(tmem_o, dp + (uint64_t)((k >> 2) * (kAttnBox >> 4) + 2 * (k & 3)), dv + (uint64_t)(128 * k), p.idesc_o, k ? 1u : 0u);
        umma_commit(b_o);
      }
    }
  } else {
    // ------------------------------------------------ soft-max and the final scaling ----
    const int quarter = warp & 3, row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t p_row = smem_u32(sP) + (uint32_t)row * 128u, y_row = smem_u32(sY) + (uint32_t)row * 128u;
    const int rx = row & 7;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++it) {
      if (!mbar_wait(b_s, it & 1, abort_flag, p.status, 15, p.spin_limit)) break;
      tc_fence_after();
      float mx = -3.402823466e+38f;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t r[16];
        tmem_ld16(tmem_s + lane_addr + (uint32_t)(c * 16), r);
        tmem_ld_wait_regs<16>(r);
#pragma unroll
        for (int j = 0; j < 16; ++j) mx = fmaxf(mx, __uint_as_float(r[j]) * p.scale_log2e);
      }
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t r[16];
        tmem_ld16(tmem_s + lane_addr + (uint32_t)(c * 16), r);
        tmem_ld_wait_regs<16>(r);
        float e[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          e[j] = fmaf(__uint_as_float(r[j]), p.scale_log2e, -mx);
          asm("ex2.approx.ftz.f32 %0, %0;" : "+f"(e[j]));
          sum += e[j];
        }
        // keys c*16 .. c*16+15 are pieces (c & 3) * 2, +1 of this row in k-block c >> 2
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint4 u;
          uint32_t* w = (uint32_t*)&u;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            if (BF16) { __nv_bfloat162 h = __floats2bfloat162_rn(e[q * 8 + 2 * t], e[q * 8 + 2 * t + 1]); w[t] = *(uint32_t*)&h; }
            else { __half2 h = __floats2half2_rn(e[q * 8 + 2 * t], e[q * 8 + 2 * t + 1]); w[t] = *(uint32_t*)&h; }
          }
          sts128(p_row + (uint32_t)(c >> 2) * kAttnBox + (uint32_t)(((((c & 3) << 1) + q) ^ rx) << 4), u);
        }
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor cores read P through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(b_p);
      const float inv = __fdividef(1.0f, sum);
      if (!mbar_wait(b_o, it & 1, abort_flag, p.status, 16, p.spin_limit)) break;
      tc_fence_after();
      // the store of the previous head has finished reading the result box
      if (it > 0 && !mbar_wait(b_sf, (it - 1) & 1, abort_flag, p.status, 17, p.spin_limit)) break;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[16];
        tmem_ld16(tmem_o + lane_addr + (uint32_t)(c * 16), r);
        tmem_ld_wait_regs<16>(r);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint4 u;
          uint32_t* w = (uint32_t*)&u;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float a = __uint_as_float(r[q * 8 + 2 * t]) * inv, b = __uint_as_float(r[q * 8 + 2 * t + 1]) * inv;
            if (BF16) { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); w[t] = *(uint32_t*)&h; }
            else { __half2 h = __floats2half2_rn(a, b); w[t] = *(uint32_t*)&h; }
          }
          sts128(y_row + (uint32_t)((((c << 1) + q) ^ rx) << 4), u);
        }
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(b_e);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
  }
}

// ------------------------------------------------------------- host: tensor maps ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;
EncodeIm2colFn g_encode_im2col = nullptr;
bool load_driver_entry_points() {
  if (g_encode_tiled && g_encode_im2col) return true;
  void* f = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || !f) return false;
  g_encode_tiled = (EncodeTiledFn)f;
  f = nullptr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &f, cudaEnableDefault, &q) != cudaSuccess || !f) return false;
  g_encode_im2col = (EncodeIm2colFn)f;
  return true;
}
int elem_bytes(int dt) { return dt == DT_S8 ? 1 : 2; }
int storage_size_of(int dt) { return dt == DT_S8 || dt == DT_U8 ? 1 : (dt == DT_F16 || dt == DT_BF16 ? 2 : (dt == DT_S64 ? 8 : 4)); }
int pick_kb_bytes(int c_bytes) { return c_bytes > 64 ? 128 : (c_bytes > 32 ? 64 : 32); }
int pick_bn(int k_out) { return k_out <= 64 ? 64 : (k_out <= 128 ? 128 : 256); }

}  // namespace

struct UmmaLaunch {
  CUtensorMap tmA, tmB, tmY, tmR;
  UmmaParams p;
  int grid;
  size_t smem;
};

bool umma_conv_supported(const UmmaConv& c) {
  if (c.in_dt != DT_F16 && c.in_dt != DT_BF16 && c.in_dt != DT_S8) return false;
  int es = elem_bytes(c.in_dt);
  if (((int64_t)c.C * es) % 16 != 0) return false;   // TMA strides and channel coordinates must be 16-byte multiples
  if (c.C * es < 32) return false;
  if (c.K < 1 || c.R < 1 || c.S < 1 || c.R * c.S * (c.w_terms > 1 ? c.w_terms : 1) > 4096) return false;
  if (c.w_terms > 1 && c.w_batches > 0) return false;
  if (c.stride_h < 1 || c.stride_w < 1 || c.stride_h > 8 || c.stride_w > 8) return false;
  if (c.pad_t > 127 || c.pad_l > 127 || c.R > 128 || c.S > 128) return false;  // im2col corners are 8-bit
  if ((int64_t)c.N * c.P * c.Q >= (1ll << 31)) return false;
  if (c.H < 1 || c.W < 1 || c.P < 1 || c.Q < 1) return false;
  if (c.w_batches > 0 && (c.R != 1 || c.S != 1 || c.rows_per_batch <= 0 || c.rows_per_batch % 128 != 0)) return false;
  if (c.w_n_major && (c.w_batches <= 0 || es != 2 || c.K != 64 || c.C % 64 != 0)) return false;
  return true;
}

bool umma_store_perm_ok(const UmmaConv& c, const Epilogue& ep, const void* y) {
  if (c.store_mode != 1 && c.store_mode != 2) return false;
  const int oes = storage_size_of(ep.out_dt);
  if (!(ep.out_dt == DT_F16 || ep.out_dt == DT_BF16 || ep.out_dt == DT_S8) || c.store_D * oes != 128) return false;  // one head = one 128-byte box
  if (ep.res || ep.add_full || (uintptr_t)y % 16 != 0 || getenv("ODLA_B200_DIRECT_EPILOGUE")) return false;
  if (c.store_S <= 0 || c.store_S % 128 != 0 || c.store_NH <= 0 || c.R != 1 || c.S != 1) return false;
  const long long M = (long long)c.N * c.P * c.Q;
  if (c.store_mode == 1) return M % c.store_S == 0 && c.K == c.store_NH * c.store_D;
  return M % ((long long)c.store_S * c.store_NH) == 0 && c.K == c.store_D;
}

UmmaLaunch* umma_conv_prepare(const UmmaConv& c, const void* x, const void* w, void* y, const Epilogue& ep, int* status, int sms) {
  if (!umma_conv_supported(c) || !load_driver_entry_points()) return nullptr;
  auto* L = new UmmaLaunch();
  UmmaParams& p = L->p;
  const int es = elem_bytes(c.in_dt);
  p.M_total = c.N * c.P * c.Q; p.K_out = c.K; p.C = c.C; p.R = c.R; p.S = c.S; p.P = c.P; p.Q = c.Q;
  p.stride_h = c.stride_h; p.stride_w = c.stride_w; p.pad_t = c.pad_t; p.pad_l = c.pad_l;
  p.im2col = !(c.R == 1 && c.S == 1 && c.stride_h == 1 && c.stride_w == 1 && c.pad_t == 0 && c.pad_l == 0 && c.P == c.H && c.Q == c.W);
  p.kb_bytes = pick_kb_bytes(c.C * es);
  p.kbe = p.kb_bytes / es;
  p.chunks_per_tap = (c.C + p.kbe - 1) / p.kbe;
  const int terms = c.w_terms > 1 ? c.w_terms : 1;
  p.num_kb = c.R * c.S * terms * p.chunks_per_tap;
  p.BN = pick_bn(c.K);
  p.m_tiles = (p.M_total + BM - 1) / BM;
  // Few rows (small batches, the classifier): narrower tiles put more SMs to work on the same reduction; a tile's time
  // is dominated by its k-blocks, not by its width.
  // (a staged tile leaves in whole 128-byte boxes, so one-byte outputs keep at least 128 columns)
  if (!getenv("ODLA_B200_NO_BN_SHRINK")) {
    const int min_bn = storage_size_of(ep.out_dt) == 1 ? 128 : 64;
    while (p.BN > min_bn && 2 * p.m_tiles * ((c.K + p.BN - 1) / p.BN) <= sms) p.BN /= 2;
  }
  p.n_tiles = (c.K + p.BN - 1) / p.BN;
  p.total_tiles = p.m_tiles * p.n_tiles;
  // CTA pairs (tcgen05 cta_group::2): a pair computes 256 rows x BN columns and each CTA loads only half of the
  // filter tile.  That pays where operand traffic into shared memory is the limit -- two-byte operands and a long
  // reduction (measured: 12 or more k-blocks, e.g. a 768-deep transformer projection; at 8 a ResNet layer loses) -- and
  // costs where the epilogue is, because the pair's CTAs then wait for each other's accumulators.  Needs whole 256-row
  // tiles and an even grid.
  {
    // (the thresholds can be moved through the environment, which the tests use to run every shape on pairs)
    const int pair_min_bn = getenv("ODLA_B200_PAIR_MIN_BN") ? atoi(getenv("ODLA_B200_PAIR_MIN_BN")) : 128;
    const int pair_min_kb = getenv("ODLA_B200_PAIR_MIN_KB") ? atoi(getenv("ODLA_B200_PAIR_MIN_KB")) : 12;
    const bool pair_s8 = getenv("ODLA_B200_PAIR_S8") != nullptr;
    p.pair = ((c.in_dt != DT_S8 || pair_s8) && p.BN >= pair_min_bn && p.num_kb >= pair_min_kb && p.M_total % (2 * BM) == 0 && sms >= 2 &&
              c.w_batches == 0) ? 1 : 0;
    p.bn_load = p.pair ? p.BN / 2 : p.BN;
    if (p.pair) {
      p.m_tiles = p.M_total / (2 * BM);
      p.total_tiles = p.m_tiles * p.n_tiles;
    }
  }
  // Several k-blocks share one pipeline stage (one mbarrier round trip) when they are small: up to
  // 48 KB per stage, balanced over the tile's k-blocks.
  const int box_bytes = (BM + p.bn_load) * p.kb_bytes;
  int bps_max = (48 * 1024) / box_bytes;
  if (bps_max < 1) bps_max = 1;
  if (bps_max > 8) bps_max = 8;
  const int iters = (p.num_kb + bps_max - 1) / bps_max;
  p.bps = (p.num_kb + iters - 1) / iters;
  p.num_it = (p.num_kb + p.bps - 1) / p.bps;
  const int stage_bytes = p.bps * box_bytes;
  // Staged epilogue: the output tile goes through shared memory (128-byte-swizzled boxes of 128 rows)
  // and leaves with TMA stores; the residual tile arrives the same way when its element size equals
  // the output's.  Needs 16-byte-multiple rows in global memory and a 1/2-byte output type.
  p.out_esz = storage_size_of(ep.out_dt);
  // The residual of a staged launch always comes through the staging box, so it must have the output's type.
  const bool res_ok = !ep.res || (ep.res_dt == ep.out_dt && (uintptr_t)ep.res % 16 == 0);
  const int64_t y_cols = c.y_pitch > 0 ? c.y_pitch : c.K;  // row pitch of y in elements
  p.staged = (ep.out_dt == DT_F16 || ep.out_dt == DT_BF16 || ep.out_dt == DT_S8) && (y_cols * p.out_esz) % 16 == 0 && !ep.add_full && res_ok &&
             (c.y_pitch == 0 || (c.y_pitch >= c.K && !ep.res && c.store_mode == 0)) &&
             ((uintptr_t)y % 16 == 0) && !getenv("ODLA_B200_DIRECT_EPILOGUE");
  p.stage_boxes = p.staged ? (p.BN * p.out_esz + 127) / 128 : 0;
  p.res_tma = p.staged && ep.res;
  const bool plain_act = !ep.act_first && (ep.act == ACT_NONE || ep.act == ACT_RELU) && (ep.out_dt != DT_S8 || (ep.out_multiply && ep.out_inv > 0.f));
  // what the straight-line epilogue assumes (see chunk_fast); everything else takes the general staged form
  const bool fast_ok = plain_act && c.K % 16 == 0 && ep.alpha == 1.f && ((ep.add1 != nullptr) != (ep.add2 != nullptr)) &&
                       ((ep.mul != nullptr) == (c.in_dt == DT_S8)) && (ep.out_dt != DT_S8 || c.in_dt == DT_S8) && !getenv("ODLA_B200_GENERAL_EPILOGUE");
  // the Darknet form (see chunk_leaky): LeakyReLU with a slope in [0, 1] straight after the per-channel addend, a
  // residual (if any) after the activation, fp32 accumulators, two-byte outputs
  // (the same kernel carries the GELU form of a transformer's first feed-forward layer: no residual there)
  const bool act_form = (ep.act == ACT_LEAKY && ep.act_a >= 0.f && ep.act_a <= 1.f && (!ep.res || ep.act_first)) ||
                        (ep.act == ACT_GELU_ERF && !ep.res && !getenv("ODLA_B200_EXACT_ERF"));
  const bool leaky_ok = act_form && c.K % 16 == 0 && ep.alpha == 1.f &&
                        ((ep.add1 != nullptr) != (ep.add2 != nullptr)) && !ep.mul && c.in_dt != DT_S8 && (ep.out_dt == DT_F16 || ep.out_dt == DT_BF16) &&
                        !getenv("ODLA_B200_GENERAL_EPILOGUE");
  // ... and its int8 form: int8 operands, multiplier + addend, GELU, requantised int8 output
  const bool gelu_s8_ok = ep.act == ACT_GELU_ERF && !ep.res && c.in_dt == DT_S8 && ep.out_dt == DT_S8 && ep.mul && ep.out_multiply && ep.out_inv > 0.f &&
                          c.K % 16 == 0 && ep.alpha == 1.f && ((ep.add1 != nullptr) != (ep.add2 != nullptr)) &&
                          !getenv("ODLA_B200_EXACT_ERF") && !getenv("ODLA_B200_GENERAL_EPILOGUE");
  p.epi_mode = !p.staged ? 0 : (fast_ok ? 1 : ((leaky_ok || gelu_s8_ok) ? 3 : 2));
  p.fast_variant = (c.in_dt == DT_S8 ? (ep.acc_small ? 2 : 1) : 0) * 2 + (ep.res ? 1 : 0);
  // Shared memory: pipeline stages first (up to 4, or what one tile needs), then as many staging
  // boxes as fit (at least one tile's worth, at most 8) so residual loads run ahead of the epilogue
  // and stores drain behind it; what is left goes back to the pipeline.
  // A memory-bound layer needs enough bytes in flight per SM to cover the latency of HBM (about 64 KB at 6.5 TB/s
  // over 148 SMs): boxes armed ahead carry the residual loads, stages armed ahead the operand loads, so neither is
  // limited to what one tile needs.
  const int budget = 224 * 1024;
  int want_stages = p.num_it + 1 < 4 ? p.num_it + 1 : 4;
  if (want_stages < 2) want_stages = 2;
  p.ring_boxes = 0;
  if (p.staged) {
    int ring_want = ep.res ? 4 * p.stage_boxes : 2 * p.stage_boxes;
    if (ring_want < 4) ring_want = 4;
    if (getenv("ODLA_B200_RING")) ring_want = atoi(getenv("ODLA_B200_RING"));
    p.ring_boxes = (budget - want_stages * stage_bytes) / 16384;
    if (p.ring_boxes > kMaxRing) p.ring_boxes = kMaxRing;
    if (p.ring_boxes > ring_want) p.ring_boxes = ring_want;
    if (p.ring_boxes < p.stage_boxes) p.ring_boxes = p.stage_boxes;
    if (p.ring_boxes < 2) p.ring_boxes = 2;  // the store of box i frees box i-1
  }
  {
    // 16 epilogue warps = 4 groups; a group owns BN/64 consecutive 16-column chunks, a box holds 128/out_esz/16
    const int per_group = p.BN / 64, per_box = 128 / p.out_esz / 16;
    const int groups_per_box = per_box / per_group < 4 ? per_box / per_group : 4;
    p.box_arrivals = 4 * (groups_per_box < 1 ? 1 : groups_per_box);
    // Contiguous runs let the groups work on different boxes at once, which pays when boxes need no residual and
    // the CTA has many tiles to stream through; otherwise finishing box after box gets the first store out sooner.
    p.epi_interleave = ep.res != nullptr || (p.total_tiles << p.pair) < 16 * sms;
    if (getenv("ODLA_B200_EPI_INTERLEAVE")) p.epi_interleave = atoi(getenv("ODLA_B200_EPI_INTERLEAVE"));
    if (p.epi_interleave) p.box_arrivals = 16;
  }
  p.stages = (budget - p.ring_boxes * 16384) / stage_bytes;
  if (p.stages > 8) p.stages = 8;
  {
    // stages beyond one tile's worth let the producer run into the following tiles (the stage ring spans tiles)
    int cap = p.num_it + 1 > 6 ? p.num_it + 1 : 6;
    if (getenv("ODLA_B200_STAGE_CAP")) cap = atoi(getenv("ODLA_B200_STAGE_CAP")) + p.num_it;
    if (p.stages > cap) p.stages = cap;
  }
  if (p.stages < 2) p.stages = 2;
  p.acc_int = c.in_dt == DT_S8;
  p.store_mode = c.store_mode; p.store_S = c.store_S; p.store_NH = c.store_NH;
  if (p.store_mode && (!p.staged || !umma_store_perm_ok(c, ep, y))) { delete L; return nullptr; }
  if (c.y_pitch > 0 && !p.staged) { delete L; return nullptr; }  // the direct epilogue writes rows of K elements
  p.rows_per_batch = c.w_batches > 0 ? c.rows_per_batch : 0;
  p.tmem_cols = 2 * p.BN;  // 128, 256 or 512: powers of two >= 32
  const uint32_t fmt = c.in_dt == DT_BF16 ? 1u : (c.in_dt == DT_S8 ? 1u : 0u);      // bf16 / signed 8-bit / f16
  const uint32_t cfmt = p.acc_int ? 2u : 1u;                                        // s32 / f32 accumulators
  p.idesc = (cfmt << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)((BM << p.pair) >> 4) << 24);
  // B stored [k][n]: the instruction reads it MN-major (descriptor bit 16).  A box is then 64 k-rows of 128 bytes: the
  // 8-row group pitch (SBO) is the same 1024 bytes, and 32 bytes of K are 16 rows = 2048 bytes further on.
  p.b_n_major = c.w_n_major ? 1 : 0;
  p.b_kstep = p.b_n_major ? (16 * 128) >> 4 : 2;
  if (p.b_n_major) {
    if (p.BN != 64 || p.kb_bytes != 128 || p.pair) { delete L; return nullptr; }
    p.idesc |= 1u << 16;
  }
  const uint32_t layout = p.kb_bytes == 128 ? 2u : (p.kb_bytes == 64 ? 4u : 6u);    // swizzle mode of the operand tiles
  const uint32_t sbo = (uint32_t)(8 * p.kb_bytes) >> 4;                             // 8-row group pitch, 16-byte units
  p.desc_hi = sbo | (1u << 14) | (layout << 29);                                    // bits 32-45 SBO, 46-47 version 1, 61-63 layout
  p.y = y; p.status = status; p.ep = ep;
  p.spin_limit = kSpinLimit;
  p.test_skip_stage = 0;
  // Test hooks for the time-out path (tests/test_conv_umma_gpu.py): a short limit and one deliberately unarmed stage.
  if (const char* e = getenv("ODLA_B200_TEST_SPIN_LIMIT")) { const long v = atol(e); if (v >= 64 && v <= (1l << 18)) p.spin_limit = (uint32_t)v; }
  if (getenv("ODLA_B200_TEST_SKIP_STAGE") && !p.pair) p.test_skip_stage = 1;
  L->grid = p.pair ? (2 * p.total_tiles < (sms & ~1) ? 2 * p.total_tiles : (sms & ~1)) : (p.total_tiles < sms ? p.total_tiles : sms);
  L->smem = (size_t)p.stages * stage_bytes + (size_t)p.ring_boxes * 16384 + 1024 /*alignment slack*/ + 1024 /*barriers*/;
  if (L->smem > 227 * 1024) { delete L; return nullptr; }

  const CUtensorMapDataType dt = c.in_dt == DT_S8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : (c.in_dt == DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  const CUtensorMapSwizzle sw = p.kb_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (p.kb_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  CUresult r;
  if (p.im2col) {
    cuuint64_t dims[4] = {(cuuint64_t)c.C, (cuuint64_t)c.W, (cuuint64_t)c.H, (cuuint64_t)c.N};
    cuuint64_t strides[3] = {(cuuint64_t)c.C * es, (cuuint64_t)c.W * c.C * es, (cuuint64_t)c.H * c.W * c.C * es};
    if (c.x_w_stride) { strides[0] = (cuuint64_t)c.x_w_stride; strides[1] = (cuuint64_t)c.x_h_stride; strides[2] = (cuuint64_t)c.x_n_stride; }
    // The box of filter-window origins: from -pad to the last origin that still yields an output.
    int lower[2] = {-c.pad_l, -c.pad_t};
    // The last origin is (Q-1)*stride - pad; the upper corner is that position relative to W-1 (H-1).
    int upper[2] = {(c.Q - 1) * c.stride_w - c.pad_l - (c.W - 1), (c.P - 1) * c.stride_h - c.pad_t - (c.H - 1)};
    if (upper[0] < -128 || upper[0] > 127 || upper[1] < -128 || upper[1] > 127) { delete L; return nullptr; }
    cuuint32_t estr[4] = {1, (cuuint32_t)c.stride_w, (cuuint32_t)c.stride_h, 1};
    r = g_encode_im2col(&L->tmA, dt, 4, (void*)x, dims, strides, lower, upper, (cuuint32_t)p.kbe, (cuuint32_t)BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
      // Drivers up to 13.1 encode small im2col tensors (< 128 KiB) with a flag that makes the load
      // misbehave; CUTLASS clears bit 21 of the second descriptor word in that case
      // (cute/atom/copy_traits_sm90_im2col.hpp), and so does this library.
      int drv = 0;
      cudaDriverGetVersion(&drv);
      const int64_t span = c.x_w_stride ? (int64_t)c.N * c.x_n_stride : (int64_t)c.N * c.H * c.W * c.C * es;
      if (drv <= 13010 && span < 131072) ((uint64_t*)&L->tmA)[1] &= ~(1ull << 21);
    }
  } else {
    cuuint64_t dims[2] = {(cuuint64_t)c.C, (cuuint64_t)p.M_total};
    cuuint64_t strides[1] = {(cuuint64_t)c.C * es};
    cuuint32_t box[2] = {(cuuint32_t)p.kbe, (cuuint32_t)BM};
    cuuint32_t estr[2] = {1, 1};
    r = g_encode_tiled(&L->tmA, dt, 2, (void*)x, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    if (!c.x_w_stride) fprintf(stderr, "[odla_b200] tensor map (A) encode failed: %d\n", (int)r);  // overlapping strides are an optional fast path
    delete L;
    return nullptr;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)c.C, (cuuint64_t)(c.R * c.S * terms), (cuuint64_t)c.K};
    cuuint64_t strides[2] = {(cuuint64_t)c.C * es, (cuuint64_t)c.R * c.S * terms * c.C * es};
    cuuint32_t box[3] = {(cuuint32_t)p.kbe, 1, (cuuint32_t)p.bn_load};
    if (c.w_batches > 0) {  // [batches][K][C]: the box spans BN rows of one matrix
      dims[1] = (cuuint64_t)c.K; dims[2] = (cuuint64_t)c.w_batches;
      strides[1] = (cuuint64_t)c.K * c.C * es;
      box[1] = (cuuint32_t)p.BN; box[2] = 1;
    }
    if (c.w_n_major) {      // [batches][C][K]: the box spans kbe rows (of the reduction) by all 64 columns
      dims[0] = (cuuint64_t)c.K; dims[1] = (cuuint64_t)c.C;
      strides[0] = (cuuint64_t)c.K * es;
      box[0] = (cuuint32_t)c.K; box[1] = (cuuint32_t)p.kbe;
    }
    cuuint32_t estr[3] = {1, 1, 1};
    r = g_encode_tiled(&L->tmB, dt, 3, (void*)w, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) { fprintf(stderr, "[odla_b200] tensor map (B) encode failed: %d\n", (int)r); delete L; return nullptr; }
  if (p.staged) {
    const CUtensorMapDataType odt = p.out_esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
    cuuint64_t dims[2] = {(cuuint64_t)y_cols, (cuuint64_t)p.M_total};
    cuuint64_t strides[1] = {(cuuint64_t)y_cols * p.out_esz};
    cuuint32_t box[2] = {(cuuint32_t)(128 / p.out_esz), (cuuint32_t)BM};
    cuuint32_t estr[2] = {1, 1};
    if (p.store_mode) {
      const cuuint64_t D = (cuuint64_t)c.store_D, S = (cuuint64_t)c.store_S, NH = (cuuint64_t)c.store_NH;
      const cuuint64_t Bn = (cuuint64_t)p.M_total / (S * (p.store_mode == 1 ? 1 : NH));
      cuuint64_t d4[4] = {D, p.store_mode == 1 ? S : NH, p.store_mode == 1 ? NH : S, Bn};
      cuuint64_t s4[3] = {D * p.out_esz, d4[1] * D * p.out_esz, d4[1] * d4[2] * D * p.out_esz};
      cuuint32_t b4[4] = {(cuuint32_t)D, p.store_mode == 1 ? (cuuint32_t)BM : 1u, p.store_mode == 1 ? 1u : (cuuint32_t)BM, 1};
      cuuint32_t e4[4] = {1, 1, 1, 1};
      r = g_encode_tiled(&L->tmY, odt, 4, y, d4, s4, b4, e4, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else
    r = g_encode_tiled(&L->tmY, odt, 2, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS && p.res_tma)
      r = g_encode_tiled(&L->tmR, odt, 2, (void*)ep.res, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "[odla_b200] tensor map (output/residual) encode failed: %d\n", (int)r); delete L; return nullptr; }
  }
  if (!p.staged) L->tmY = L->tmA;
  if (!p.res_tma) L->tmR = L->tmA;
  static bool attr_set[16] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 16 && !attr_set[dev]) {
#define B2_SMEM(O, M)                                                                                                              \
  (cudaFuncSetAttribute(umma_conv_kernel<O, M, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess && \
   cudaFuncSetAttribute(umma_conv_kernel<O, M, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess)
    bool ok = B2_SMEM(DT_F16, 1) && B2_SMEM(DT_BF16, 1) && B2_SMEM(DT_S8, 1) && B2_SMEM(DT_F16, 2) && B2_SMEM(DT_BF16, 2) && B2_SMEM(DT_S8, 2) && B2_SMEM(DT_F16, 3) && B2_SMEM(DT_BF16, 3) && B2_SMEM(DT_S8, 3) && B2_SMEM(-1, 0);
#undef B2_SMEM
    if (!ok) { cudaGetLastError(); delete L; return nullptr; }
    attr_set[dev] = true;
  }
  return L;
}

int umma_conv_run(UmmaLaunch* L, cudaStream_t stream) {
  if (!L) return -1;
  if (L->p.total_tiles <= 0) return 0;
  const UmmaParams& p = L->p;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)L->grid);
  cfg.blockDim = dim3(p.staged ? EpiCfg<true>::kThreads : EpiCfg<false>::kThreads);
  cfg.dynamicSmemBytes = L->smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  static const bool pdl = !getenv("ODLA_B200_NO_PDL");
  int na = 0;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (p.pair) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t le;
#define B2_LAUNCH(O, M)                                                                                   \
  le = p.pair ? cudaLaunchKernelEx(&cfg, umma_conv_kernel<O, M, true>, L->tmA, L->tmB, L->tmY, L->tmR, p) \
              : cudaLaunchKernelEx(&cfg, umma_conv_kernel<O, M, false>, L->tmA, L->tmB, L->tmY, L->tmR, p)
  if (p.epi_mode == 0) B2_LAUNCH(-1, 0);
  else if (p.epi_mode == 1) { if (p.ep.out_dt == DT_F16) B2_LAUNCH(DT_F16, 1); else if (p.ep.out_dt == DT_BF16) B2_LAUNCH(DT_BF16, 1); else B2_LAUNCH(DT_S8, 1); }
  else if (p.epi_mode == 3) { if (p.ep.out_dt == DT_F16) B2_LAUNCH(DT_F16, 3); else if (p.ep.out_dt == DT_BF16) B2_LAUNCH(DT_BF16, 3); else B2_LAUNCH(DT_S8, 3); }
  else { if (p.ep.out_dt == DT_F16) B2_LAUNCH(DT_F16, 2); else if (p.ep.out_dt == DT_BF16) B2_LAUNCH(DT_BF16, 2); else B2_LAUNCH(DT_S8, 2); }
#undef B2_LAUNCH
  if (le != cudaSuccess) { fprintf(stderr, "[odla_b200] umma_conv launch failed: %s\n", cudaGetErrorString(le)); cudaGetLastError(); return -2; }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { fprintf(stderr, "[odla_b200] umma_conv launch failed: %s\n", cudaGetErrorString(e)); return -2; }
  return 0;
}
void umma_conv_destroy(UmmaLaunch* L) { delete L; }

// ---- fused attention: host side ----
struct AttnLaunch {
  CUtensorMap tmQ, tmK, tmV, tmY;
  AttnParams p;
  int grid;
  size_t smem;
  bool bf16;
};
bool attn_supported(int dt, int64_t S, int64_t D) { return (dt == DT_F16 || dt == DT_BF16) && S == kAttnS && D == kAttnD; }
AttnLaunch* attn_prepare(int dt, const void* q, const void* k, const void* v, void* y, int64_t batch, int heads, float scale, bool merge_heads, int* status,
                         int sms) {
  if (!attn_supported(dt, kAttnS, kAttnD) || batch * heads <= 0 || batch * heads * kAttnS >= (1ll << 31) || !load_driver_entry_points()) return nullptr;
  if ((uintptr_t)q % 16 || (uintptr_t)k % 16 || (uintptr_t)v % 16 || (uintptr_t)y % 16) return nullptr;
  auto* L = new AttnLaunch();
  AttnParams& p = L->p;
  p.tiles = (int)(batch * heads); p.NH = heads; p.merge = merge_heads ? 1 : 0;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.bf16 = dt == DT_BF16; L->bf16 = dt == DT_BF16;
  const uint32_t fmt = dt == DT_BF16 ? 1u : 0u;
  p.idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(kAttnS >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  p.idesc_o = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(kAttnD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);   // B (= V) is MN-major
  p.desc_hi = ((uint32_t)(8 * 128) >> 4) | (1u << 14) | (2u << 29);
  p.spin_limit = kSpinLimit;
  p.status = status;
  L->grid = p.tiles < 4 * sms ? p.tiles : 4 * sms;
  L->smem = 3 * (size_t)kAttnBox + 1024 /*alignment slack*/ + 256 /*barriers*/;
  const CUtensorMapDataType tdt = dt == DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint64_t rows = (cuuint64_t)p.tiles * kAttnS;
  cuuint64_t dims[2] = {(cuuint64_t)kAttnD, rows};
  cuuint64_t strides[1] = {(cuuint64_t)kAttnD * 2};
  cuuint32_t box[2] = {(cuuint32_t)kAttnD, (cuuint32_t)kAttnS};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = CUDA_SUCCESS;
  const void* src[3] = {q, k, v};
  CUtensorMap* maps[3] = {&L->tmQ, &L->tmK, &L->tmV};
  for (int i = 0; i < 3 && r == CUDA_SUCCESS; ++i)
    r = g_encode_tiled(maps[i], tdt, 2, (void*)src[i], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) {
    if (merge_heads) {   // [B][S][NH][D]: a head's 128 rows lie NH * D elements apart
      cuuint64_t d4[4] = {(cuuint64_t)kAttnD, (cuuint64_t)heads, (cuuint64_t)kAttnS, (cuuint64_t)batch};
      cuuint64_t s4[3] = {(cuuint64_t)kAttnD * 2, (cuuint64_t)heads * kAttnD * 2, (cuuint64_t)kAttnS * heads * kAttnD * 2};
      cuuint32_t b4[4] = {(cuuint32_t)kAttnD, 1, (cuuint32_t)kAttnS, 1};
      cuuint32_t e4[4] = {1, 1, 1, 1};
      r = g_encode_tiled(&L->tmY, tdt, 4, y, d4, s4, b4, e4, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
      r = g_encode_tiled(&L->tmY, tdt, 2, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
  }
  if (r != CUDA_SUCCESS) { fprintf(stderr, "[odla_b200] tensor map (attention) encode failed: %d\n", (int)r); delete L; return nullptr; }
  if (cudaFuncSetAttribute(attn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L->smem) != cudaSuccess ||
      cudaFuncSetAttribute(attn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L->smem) != cudaSuccess) {
    cudaGetLastError(); delete L; return nullptr;
  }
  return L;
}
int attn_run(AttnLaunch* L, cudaStream_t stream) {
  if (!L) return -1;
  if (L->p.tiles <= 0) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)L->grid);
  cfg.blockDim = dim3(kAttnThreads);
  cfg.dynamicSmemBytes = L->smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  static const bool pdl = !getenv("ODLA_B200_NO_PDL");
  int na = 0;
  if (pdl) { attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[na].val.programmaticStreamSerializationAllowed = 1; ++na; }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t le = L->bf16 ? cudaLaunchKernelEx(&cfg, attn_kernel<true>, L->tmQ, L->tmK, L->tmV, L->tmY, L->p)
                           : cudaLaunchKernelEx(&cfg, attn_kernel<false>, L->tmQ, L->tmK, L->tmV, L->tmY, L->p);
  if (le != cudaSuccess) { fprintf(stderr, "[odla_b200] attention launch failed: %s\n", cudaGetErrorString(le)); cudaGetLastError(); return -2; }
  return 0;
}
void attn_destroy(AttnLaunch* L) { delete L; }

}  // namespace b200
