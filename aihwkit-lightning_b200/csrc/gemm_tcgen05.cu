// bf16 GEMMs of the analog linear path on the Blackwell tensor cores (sm_100a): operands are
// brought into shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), multiplied by
// tcgen05.mma with fp32 accumulators in tensor memory (TMEM), and drained by tcgen05.ld.
//
// Two persistent, warp-specialised kernels (one CTA per SM):
//
//  * fwd_tc_kernel   out[m,n] = sum_t stage_t( xq[m, tile t] . w_mod[n, tile t] ) + bias[n]
//      128x128 output block per CTA iteration.  The K loop is cut at the analog-tile
//      boundaries; each analog tile accumulates into one of two TMEM accumulators, and while
//      the tensor core works on tile t+1 sixteen epilogue warps run tile t's output stage
//      (rounding, output noise, ADC quantisation, clamp, clamp-mask bits) and add it to a
//      running sum that also lives in TMEM.
//  * bwd_tc_kernel   C[i, lo_t + j] = sum_l (g * keep_t)(i,l) * B(l, lo_t + j)
//      dgrad (C = grad_x, A = g, B = w_mod) and wgrad (C = grad_w, A = g^T, B = xq) in one
//      template: 128x256 output block, the operands that are contiguous along the output
//      dimension are fed as MN-major tiles, and four warps apply the ADC clamp mask of the
//      analog tile to the staged gradient tile before the MMA reads it.
//
// Every wait on an mbarrier is bounded (wall-clock limit); a wait that gives up raises a
// device error word, makes the CTA drain its copies in flight, free its TMEM and return.
// No TMA multicast and no thread-block clusters are used.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "analog_math.cuh"
#include "device_fast.cuh"
#include "internal.h"

namespace al {

__device__ uint32_t g_tc_error_word = 0;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle span
constexpr int kThreads = 384;          // 12 warps
constexpr uint64_t kTimeoutNs = 2000000000ull;

// forward kernel
constexpr int F_BN = 128;
constexpr int F_STAGES = 6;
constexpr int FP_STAGES = 5;   // CTA pairs: 64 KiB of shared memory hold the running sum
constexpr int FP_SUM_BYTES = BM * 2 * F_BN * 2;
constexpr int F_A_BYTES = BM * BK * 2;     // 16 KiB
constexpr int F_B_BYTES = F_BN * BK * 2;   // 16 KiB
constexpr int F_STAGE_BYTES = F_A_BYTES + F_B_BYTES;
constexpr int F_EPI_WARPS = 16;
constexpr int kFwdThreads = (4 + F_EPI_WARPS) * 32;  // producer, MMA, two idle, 16 epilogue warps
// backward kernel
constexpr int B_BN = 256;
constexpr int B_STAGES = 4;
constexpr int B_A_BYTES = BM * BK * 2;     // 16 KiB
constexpr int B_B_BYTES = B_BN * BK * 2;   // 32 KiB
constexpr int B_STAGE_BYTES = B_A_BYTES + B_B_BYTES;
constexpr int B_BOX_BYTES = 64 * BK * 2;   // one 64x64 MN-major box: 8 KiB
constexpr int B_EPI_WARPS = 4;
constexpr int B_XFORM_THREADS = 128;   // per group; each group handles one stage at a time
constexpr int B_XFORM_GROUPS = 4;
constexpr int kBwdThreads = (8 + 4 * B_XFORM_GROUPS) * 32;

// backward kernel on CTA pairs: a 256 x 256 tile per pair, each CTA stages its 128 rows of A and
// its 128 columns of B, so a stage is 32 KiB and six of them fit
constexpr int P_BN = 256;
constexpr int P_BN_CTA = 128;
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = BM * BK * 2;         // 16 KiB
constexpr int P_B_BYTES = P_BN_CTA * BK * 2;   // 16 KiB
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;

constexpr int kTmemCols = 512;

enum ErrCode : uint32_t {
  kErrProducer = 1u, kErrMma = 2u, kErrEpilogue = 4u, kErrTransform = 8u, kErrDrain = 16u
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Arrival that publishes nothing: the caller wrote no data the waiter reads.
__device__ __forceinline__ void mbar_arrive_relaxed(uint64_t* bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
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
// Bounded wait.  Returns false when the wait gave up (time limit, or another role aborted).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 31u) == 31u) {
      if (*abort_flag) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kTimeoutNs) return false;
    }
  }
}
__device__ __forceinline__ void raise_error(uint32_t code, volatile uint32_t* abort_flag) {
  *abort_flag = 1u;
  atomicOr(&g_tc_error_word, code);
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate, issued by one thread
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// ---- CTA pairs (cta_group::2): two CTAs of a cluster drive one 256-row MMA ------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `saddr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrival on an mbarrier of any CTA of the cluster (address from mapa_u32)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// wait side of a barrier that CTAs of the whole cluster arrive on
__device__ __forceinline__ bool mbar_try_cluster(uint64_t* bar, uint32_t parity) {
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
// TMA tile load of a CTA pair: lands in this CTA's shared memory, completes bytes on the
// mbarrier at `bar_cluster_addr`, which may live in either CTA of the pair.  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// commit of the pair's MMAs: one arrival on the barrier at this offset in every CTA of cta_mask
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(cta_mask)
      : "memory");
}
// D[tmem of both CTAs] (+)= A[256 rows, 128 per CTA] * B[256 columns, 128 per CTA]
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
#define AL_TMEM_REGS32(r)                                                                                   \
  r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7], r[8], r[9], r[10], r[11], r[12], r[13], r[14], r[15],     \
      r[16], r[17], r[18], r[19], r[20], r[21], r[22], r[23], r[24], r[25], r[26], r[27], r[28], r[29],     \
      r[30], r[31]
// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base lane + i), 32 columns
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t r[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t r[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
        "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (128-byte swizzle, descriptor version 1 of sm_100).
// K-major: rows of 128 bytes (64 bf16 along K), 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// MN-major: rows of 128 bytes hold 64 consecutive M/N elements of one k; 8-k groups are 1024
// bytes apart (stride offset) and the next 64 M/N elements start `lbo_bytes` further (leading
// offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t saddr, uint32_t lbo_bytes) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
         ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of tcgen05.mma.kind::f16: fp32 accumulator, bf16 A and B.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
}

// 16-column variants of the TMEM load / store
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t r[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t r[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(taddr)
      : "memory");
}

// Round-to-nearest-even to bf16 precision on the integer ALU.  The cvt.rn.bf16.f32 instruction
// runs on the quarter-rate conversion pipe, which the per-tile output stage (six roundings per
// element in reference-rounding mode) would saturate.  Same result as the cvt for every finite
// value and for infinities; NaNs are patched by the caller.
template <int RD>
__device__ __forceinline__ float rnd_alu(float v) {
  if (RD == kBF16) {
    uint32_t u = __float_as_uint(v);
    u += 0x7fffu + ((u >> 16) & 1u);
    return __uint_as_float(u & 0xffff0000u);
  }
  return v;
}
// round-half-even to an integer with two additions (exact for |x| < 2^22)
__device__ __forceinline__ float rint_magic(float x) {
  const float r = __fsub_rn(__fadd_rn(x, 12582912.0f), 12582912.0f);
  return fabsf(x) < 4194304.0f ? r : x;
}
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// 8-column (packed bf16x2 running sum) variants of the TMEM load / store
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t r[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t r[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};"
               ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(taddr)
               : "memory");
}

struct Barriers {
  uint64_t full[8];
  uint64_t ready[8];
  uint64_t empty[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t mma_done;
  uint32_t tmem_slot;
  uint32_t abort_flag;
};

__device__ __forceinline__ uint8_t* align_1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
}

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
struct FwdTcParams {
  int32_t small_adc_codes;  // |ADC code| provably below 2^38: unguarded add-based rint is exact
  int32_t tile_w;      // width of every analog tile (all equal on this path)
  int32_t ksteps;      // ceil(tile_w / 64)
  int32_t num_mb, num_nb;
  FwdEpilogueParams ep;
  NoiseKeys noise;     // output-noise stream of this call, prepared on the host
  void* out;
};

// MODE >= 0: the output stage is fixed at compile time (bit 0 output noise from the internal
// generator, bit 1 ADC quantisation, bit 2 clamp; reference rounding, per-tile scalar scales,
// rounding on, small ADC codes).  MODE < 0: every switch is read at run time.
//
// PAIR: launched as clusters of two CTAs that share one tcgen05.mma.cta_group::2 of 256 x 256
// per k-step (an MMA that is 256 columns wide runs the tensor cores at their full rate, one of
// 128 columns does not).  CTA `rank` owns rows [256 mb + 128 rank, +128) of the block: it stages
// those rows of the inputs and 128 of the block's 256 weight rows, holds its 128 x 256 half of
// the accumulator and runs the output stage on it.  The two accumulator buffers fill the tensor
// memory, so the running sum over the analog tiles (bf16x2) lives in shared memory, which leaves
// five pipeline stages.  Only the packed bf16 output stage exists in this form (the host sends
// per-channel scales and fp32 rounding to single CTAs).  The leader (rank 0) issues the MMAs;
// `full` collects both CTAs' copies in the leader, `empty` and `acc_full` are signalled in both
// CTAs by the leader's multicast commits, `acc_empty` collects both CTAs' epilogue warps in the
// leader.
template <int RD, int MODE, bool PAIR>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
              const FwdTcParams p) {
  constexpr int kStages = PAIR ? FP_STAGES : F_STAGES;
  constexpr int kBRows = F_BN;                                 // weight rows this CTA stages
  constexpr int kStageBytes = F_STAGE_BYTES;
  constexpr int kBlockRows = PAIR ? 2 * BM : BM;               // rows of the outputs per work item
  constexpr int kBN = PAIR ? 2 * F_BN : F_BN;                  // columns of the outputs per work item
  constexpr int kSumBytes = PAIR ? FP_SUM_BYTES : 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* stage_base = align_1024(smem_raw);
  uint8_t* sum_base = stage_base + kStages * kStageBytes;      // PAIR: [128 rows][256 bf16], 16-byte chunks swizzled
  Barriers* bars = reinterpret_cast<Barriers*>(sum_base + kSumBytes);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const FwdEpilogueParams& ep = p.ep;
  const int T = ep.T;
  const int num_tiles = p.num_mb * p.num_nb;  // num_mb counts blocks of kBlockRows rows
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int row_off = (int)rank * BM;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], PAIR ? 2 * F_EPI_WARPS : F_EPI_WARPS);
    }
    mbar_init(&bars->mma_done, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    if (PAIR) tmem_alloc_pair(&bars->tmem_slot, kTmemCols);
    else tmem_alloc(&bars->tmem_slot, kTmemCols);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_slot;

  if (warp == 0) {
    // ---- TMA producer ------------------------------------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = worker; tile < num_tiles && ok; tile += n_workers) {
        const int mb = tile / p.num_nb, nb = tile % p.num_nb;
        for (int t = 0; t < T && ok; ++t) {
          for (int ks = 0; ks < p.ksteps; ++ks, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            if (!mbar_wait(&bars->empty[s], ph ^ 1u, abort_flag)) {
              raise_error(kErrProducer, abort_flag);
              ok = false;
              break;
            }
            uint8_t* sa = stage_base + s * kStageBytes;
            if (PAIR) {
              // both CTAs' copies complete on the leader's barrier
              if (leader) mbar_expect_tx(&bars->full[s], 2 * kStageBytes);
              const uint32_t bar = mapa_u32(smem_u32(&bars->full[s]), 0);
              tma_load_3d_pair(sa, &map_a, bar, ks * BK, t, mb * kBlockRows + row_off);
              tma_load_3d_pair(sa + F_A_BYTES, &map_b, bar, ks * BK, t, nb * kBN + (int)rank * kBRows);
            } else {
              mbar_expect_tx(&bars->full[s], kStageBytes);
              tma_load_3d(sa, &map_a, &bars->full[s], ks * BK, t, mb * BM);
              tma_load_3d(sa + F_A_BYTES, &map_b, &bars->full[s], ks * BK, t, nb * F_BN);
            }
          }
        }
      }
      // drain: the last copies issued must have landed before the CTA may exit (the leader's
      // barrier covers its peer's copies; both CTAs meet at the end of the kernel)
      if (leader) {
        const uint32_t n_back = it < (uint32_t)kStages ? it : (uint32_t)kStages;
        for (uint32_t j = it - n_back; j < it; ++j) {
          const int s = j % kStages;
          const uint32_t ph = (j / kStages) & 1u;
          uint64_t t0 = globaltimer_ns();
          while (!mbar_try(&bars->full[s], ph)) {
            if (globaltimer_ns() - t0 > kTimeoutNs) {
              raise_error(kErrDrain, abort_flag);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer --------------------------------------------------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(kBlockRows, kBN, 0, 0);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = worker; tile < num_tiles && ok; tile += n_workers) {
        for (int t = 0; t < T && ok; ++t, ++acc_it) {
          const int b = acc_it & 1u;
          const uint32_t aph = (acc_it >> 1) & 1u;
          if (!mbar_wait(&bars->acc_empty[b], aph ^ 1u, abort_flag)) {
            raise_error(kErrMma, abort_flag);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(b * kBN);
          for (int ks = 0; ks < p.ksteps; ++ks, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            if (!mbar_wait(&bars->full[s], ph, abort_flag)) {
              raise_error(kErrMma, abort_flag);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(stage_base + s * kStageBytes);
            const uint64_t da = desc_k_major(sa), db = desc_k_major(sa + F_A_BYTES);
#pragma unroll
            for (int k4 = 0; k4 < BK / 16; ++k4) {
              if (PAIR) umma_bf16_pair(d_tmem, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (ks | k4) != 0 ? 1u : 0u);
              else umma_bf16(d_tmem, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (ks | k4) != 0 ? 1u : 0u);
            }
            if (PAIR) umma_commit_pair(&bars->empty[s], 3);  // frees the stage in both CTAs
            else umma_commit(&bars->empty[s]);
          }
          if (ok) {
            if (PAIR) umma_commit_pair(&bars->acc_full[b], 3);
            else umma_commit(&bars->acc_full[b]);
          }
        }
      }
      // all MMAs issued by this thread must have retired before TMEM is freed
      if (PAIR) umma_commit_pair(&bars->mma_done, 1);
      else umma_commit(&bars->mma_done);
      uint64_t t0 = globaltimer_ns();
      while (!mbar_try(&bars->mma_done, 0)) {
        if (globaltimer_ns() - t0 > kTimeoutNs) {
          raise_error(kErrDrain, abort_flag);
          break;
        }
      }
    }
  } else if (warp >= 4) {
    // ---- epilogue: per-tile output stage, running sum in TMEM ---------------------------
    // 16 warps: warp & 3 selects the TMEM lane quadrant (rows), (warp - 4) >> 2 the kCols columns.
    constexpr int kCols = kBN / 4;
    const int quad = warp & 3;
    const int col0 = ((warp - 4) >> 2) * kCols;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const int M = ep.M, N = ep.N;
    constexpr bool kFixed = MODE >= 0;
    const bool has_noise = kFixed ? (MODE & 1) != 0 : ep.has_noise != 0;
    const bool has_adc = kFixed ? (MODE & 2) != 0 : ep.has_adc != 0;
    const bool has_bound = kFixed ? (MODE & 4) != 0 : ep.has_bound != 0;
    const bool replay = kFixed ? false : ep.out_noise != nullptr;
    const bool no_round = kFixed ? false : ep.no_rounding != 0;
    const bool small_codes = kFixed ? true : p.small_adc_codes != 0;
    const bool per_channel = kFixed ? false : (ep.w_amax != nullptr && (ep.noise_pc || ep.bound_pc));
    // Output noise with nothing non-linear between the tiles (no ADC, no clamp): the T independent
    // Gaussian terms s_t * xi_t of an output add up to one Gaussian of variance sum_t s_t^2, so
    // one draw per output at the last tile replaces T draws -- same distribution up to the bf16
    // rounding of the partial sums, an eighth of the generator work on an 8-tile layer.  Replayed
    // noise (parity runs) never takes this route: it is applied tile by tile as given.
    constexpr bool kMergedNoise = kFixed && MODE == 1;
    float noise_var = 0.0f;
    TileEpilogueCfg cfg;
    cfg.has_noise = ep.has_noise; cfg.has_bound = ep.has_bound; cfg.has_adc = ep.has_adc;
    cfg.no_rounding = ep.no_rounding; cfg.noise_coef = ep.noise_coef; cfg.out_bound = ep.out_bound;
    cfg.out_res = ep.out_res;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int tile = worker; tile < num_tiles && ok; tile += n_workers) {
      const int mb = tile / p.num_nb, nb = tile % p.num_nb;
      const int m = mb * kBlockRows + row_off + quad * 32 + lane;
      const bool row_ok = m < M;
      const int n_first = nb * kBN + col0;
      for (int t = 0; t < T && ok; ++t, ++acc_it) {
        const int b = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        // constants of this (row, analog tile): fetched and derived before waiting for the
        // accumulator, so that the load latency and the division overlap the tile's MMAs
        float ir = 0.0f;
        if (row_ok) {
          if (ep.ir_mode == AL_IR_DYNAMIC) ir = Elem<kBF16>::load(ep.ir_rows, (int64_t)t * M + m);
          else if (ep.ir_mode == AL_IR_STATIC) ir = Elem<kBF16>::load(ep.ir_rows, t);
        }
        const float t_max = ep.w_tile_max ? ep.w_tile_max[t] : 0.0f;
        float sc = rnd<RD>(fmul(t_max, rnd<RD>(fmul(ep.noise_coef, ir))));
        bool noise_now = has_noise;
        if (kMergedNoise) {
          noise_var = t == 0 ? sc * sc : fmaf(sc, sc, noise_var);
          noise_now = t == T - 1;
          sc = sqrtf(noise_var);
        }
        const float bound = rnd<RD>(fmul(rnd<RD>(fmul(ir, ep.out_bound)), t_max));
        const float step = has_adc ? quant_step<RD>(bound, ep.out_res) : 1.0f;
        const float stepc = step < kTiny ? kTiny : step;
        const float rstep = __frcp_rn(stepc);
        if (!mbar_wait(&bars->acc_full[b], aph, abort_flag)) {
          if (lane == 0) raise_error(kErrEpilogue, abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t keep_bits = 0;
        // eight consecutive elements share one generator call (N is a multiple of 8 on this path)
        const uint64_t row_group8 = (((uint64_t)t * M + (row_ok ? m : 0)) * N) >> 3;
        const bool packed = RD == kBF16 && !per_channel;  // bf16x2 arithmetic, bf16x2 running sum
        const __nv_bfloat162 sc2 = __float2bfloat162_rn(sc), step2 = __float2bfloat162_rn(step);
        const __nv_bfloat162 bound2 = __float2bfloat162_rn(bound), nbound2 = __float2bfloat162_rn(-bound);
        const __nv_bfloat162 zero2 = __float2bfloat162_rn(0.0f);
        const uint64_t nstepc2 = f32x2_pack(-stepc, -stepc), rstep2 = f32x2_pack(rstep, rstep);
        const uint64_t magic2 = f32x2_pack(12582912.0f, 12582912.0f), nmagic2 = f32x2_pack(-12582912.0f, -12582912.0f);
        // this thread's row of the shared-memory running sum (PAIR): chunk c of 8 columns sits at
        // 16 * (c ^ (row & 7)), so the eight rows a quarter-warp reads hit distinct banks
        const int srow = quad * 32 + lane;
        const uint32_t sum_row = smem_u32(sum_base) + (uint32_t)srow * (uint32_t)(kBN * 2);
#pragma unroll 1
        for (int h = 0; h < kCols / 16; ++h) {
          const int cc = col0 + h * 16;
          const int nh = n_first + h * 16;
          const int n0 = n_first + (h >> 1) * 32;  // the 32 columns whose mask word this half belongs to
          if ((h & 1) == 0) keep_bits = 0;
          uint32_t accr[16], sumr[16];
          tmem_ld16(tmem_base + lane_base + (uint32_t)(b * kBN + cc), accr);
          if (t > 0) {
            if (PAIR) {
#pragma unroll
              for (int v = 0; v < 2; ++v) {
                const uint32_t addr = sum_row + (uint32_t)((((cc >> 3) + v) ^ (srow & 7)) << 4);
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(sumr[4 * v]), "=r"(sumr[4 * v + 1]), "=r"(sumr[4 * v + 2]), "=r"(sumr[4 * v + 3])
                             : "r"(addr) : "memory");
              }
            } else if (packed) {
              tmem_ld8(tmem_base + lane_base + (uint32_t)(2 * F_BN + (cc >> 1)), sumr);
            } else {
              tmem_ld16(tmem_base + lane_base + (uint32_t)(2 * F_BN + cc), sumr);
            }
          }
          tmem_wait_ld();
          float z[16];
          if (noise_now) {
#pragma unroll
            for (int g8 = 0; g8 < 2; ++g8) {
              const int nq = nh + g8 * 8;
              if (replay) {
                const uint64_t idx = ((uint64_t)t * M + (row_ok ? m : 0)) * N + (nq < N ? nq : 0);
                const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(ep.out_noise) + idx);
                const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  z[g8 * 8 + 2 * q] = __uint_as_float(rw[q] << 16);
                  z[g8 * 8 + 2 * q + 1] = __uint_as_float(rw[q] & 0xffff0000u);
                }
              } else {
                normal8_keyed(p.noise, row_group8 + (uint32_t)((nq < N ? nq : 0) >> 3), &z[g8 * 8]);
              }
            }
          }
          if (packed) {
            if (t == 0) {
#pragma unroll
              for (int pr = 0; pr < 8; ++pr) sumr[pr] = 0u;  // +0.0 in both halves
            }
            uint32_t kept = 0;  // bit 2*pr (low half) and bit 16 + 2*pr + 1 (high half): element kept
#pragma unroll
            for (int pr = 0; pr < 8; ++pr) {
              // element 2*pr in the low half, 2*pr+1 in the high half
              __nv_bfloat162 o2 = __floats2bfloat162_rn(__uint_as_float(accr[2 * pr]), __uint_as_float(accr[2 * pr + 1]));
              if (noise_now) {
                const __nv_bfloat162 z2 = __floats2bfloat162_rn(z[2 * pr], z[2 * pr + 1]);
                o2 = __hadd2_rn(o2, __hmul2_rn(sc2, z2));
              }
              if (has_adc) {
                // both elements of the pair side by side in fp32x2 arithmetic
                float q_lo, q_hi;
                f32x2_unpack(f32x2_div_rcp(f32x2_pack(__low2float(o2), __high2float(o2)), nstepc2, rstep2), &q_lo, &q_hi);
                const __nv_bfloat162 q2 = __floats2bfloat162_rn(q_lo, q_hi);
                float c_lo = __low2float(q2), c_hi = __high2float(q2);
                if (!no_round) {
                  // bf16-valued codes: the unguarded add-based rint is exact below 2^38
                  if (small_codes) {
                    f32x2_unpack(f32x2_add(f32x2_add(f32x2_pack(c_lo, c_hi), magic2), nmagic2), &c_lo, &c_hi);
                  } else {
                    c_lo = rint_magic(c_lo);
                    c_hi = rint_magic(c_hi);
                  }
                }
                // an integer-rounded bf16 value is a bf16 value: packing is a bit move
                const uint32_t c2 = __byte_perm(__float_as_uint(c_lo), __float_as_uint(c_hi), 0x7632);
                o2 = __hmul2_rn(as_bf162(c2), step2);
              }
              if (has_bound) {
                // kept <=> the clamp leaves the value unchanged (false for NaN, like the reference's
                // -bound <= o <= bound)
                const __nv_bfloat162 c2 = __hmin2_nan(__hmax2_nan(o2, nbound2), bound2);
                kept |= __heq2_mask(c2, o2) & ((1u << (2 * pr)) | (1u << (17 + 2 * pr)));
                o2 = c2;
              }
              sumr[pr] = as_u32(__hadd2_rn(as_bf162(sumr[pr]), o2));
            }
            if (!has_bound) kept = 0xffffffffu;
            keep_bits |= ((kept | (kept >> 16)) & 0xffffu) << ((h & 1) * 16);
          } else if (!per_channel) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float acc = __uint_as_float(accr[j]);
              float o = rnd_alu<RD>(acc);
              if (has_noise) o = rnd_alu<RD>(fadd(o, rnd_alu<RD>(fmul(sc, rnd_alu<RD>(z[j])))));
              bool keep = true;
              if (has_adc) {
                float code = rnd_alu<RD>(fdiv_rcp(o, stepc, rstep));
                if (!no_round) code = rint_magic(code);
                o = rnd_alu<RD>(fmul(code, step));
              }
              if (has_bound) {
                keep = fabsf(o) <= bound;
                o = fminf(fmaxf(o, -bound), bound);
              }
              float sum = t == 0 ? fadd(0.0f, o) : rnd_alu<RD>(fadd(__uint_as_float(sumr[j]), o));
              if (acc != acc) sum = acc;  // the integer rounding above does not preserve NaN
              sumr[j] = __float_as_uint(sum);
              keep_bits |= (keep ? 1u : 0u) << ((h & 1) * 16 + j);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int n = nh + j;
              const float cmax = n < N ? Elem<kBF16>::load(ep.w_amax, (int64_t)t * N + n) : 0.0f;
              bool keep;
              const float o = tile_epilogue<RD>(__uint_as_float(accr[j]), ir, ep.noise_pc ? cmax : t_max,
                                                ep.bound_pc ? cmax : t_max, has_noise ? rnd<RD>(z[j]) : 0.0f,
                                                cfg, &keep);
              sumr[j] = __float_as_uint(t == 0 ? fadd(0.0f, o) : rnd<RD>(fadd(__uint_as_float(sumr[j]), o)));
              keep_bits |= (keep ? 1u : 0u) << ((h & 1) * 16 + j);
            }
          }
          if (t < T - 1) {
            if (PAIR) {
#pragma unroll
              for (int v = 0; v < 2; ++v) {
                const uint32_t addr = sum_row + (uint32_t)((((cc >> 3) + v) ^ (srow & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(sumr[4 * v]),
                             "r"(sumr[4 * v + 1]), "r"(sumr[4 * v + 2]), "r"(sumr[4 * v + 3]) : "memory");
              }
            } else if (packed) {
              tmem_st8(tmem_base + lane_base + (uint32_t)(2 * F_BN + (cc >> 1)), sumr);
            } else {
              tmem_st16(tmem_base + lane_base + (uint32_t)(2 * F_BN + cc), sumr);
            }
          } else if (row_ok) {
            // final: bias, convert, store 16 bf16 = 32 bytes of this row
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.out) + (int64_t)m * N + nh;
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              if (nh + v * 8 < N) {
                uint32_t w4[4];
                if (packed) {
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 s2 = as_bf162(sumr[v * 4 + e]);
                    if (ep.bias) {
                      const uint32_t b2 = *reinterpret_cast<const uint32_t*>(
                          reinterpret_cast<const uint16_t*>(ep.bias) + nh + v * 8 + 2 * e);
                      s2 = __hadd2_rn(s2, as_bf162(b2));
                    }
                    w4[e] = as_u32(s2);
                  }
                } else {
                  float f[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    f[e] = __uint_as_float(sumr[v * 8 + e]);
                    if (ep.bias) f[e] = fadd(rnd<RD>(f[e]), Elem<kBF16>::load(ep.bias, nh + v * 8 + e));
                  }
#pragma unroll
                  for (int e = 0; e < 4; ++e) w4[e] = pack_bf16x2_rn(f[2 * e], f[2 * e + 1]);
                }
                *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
              }
            }
          }
          if ((h & 1) && ep.keep_mask != nullptr && row_ok && (n0 >> 5) < ep.mask_words)
            ep.keep_mask[((int64_t)t * ep.mask_words + (n0 >> 5)) * M + m] = keep_bits;  // lanes = consecutive rows
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&bars->acc_empty[b]), 0));
          else mbar_arrive(&bars->acc_empty[b]);
        }
      }
    }
  }

  // (pairs) nothing of this CTA's shared or tensor memory may go while the peer can still signal
  // or use it: both CTAs meet before the tensor memory is released
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  tc_fence_after();
  if (warp == 1) {
    if (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// backward (dgrad / wgrad)
// ---------------------------------------------------------------------------------------------
struct BwdTcParams {
  int32_t I;           // rows of C (M for dgrad, N for wgrad)
  int32_t L;           // reduction length (N for dgrad, M for wgrad)
  int32_t K;           // row stride of C
  int32_t M;           // rows of the mask
  int32_t T;           // analog tiles that carry their own mask (1 when there is no mask)
  int32_t tile_w;      // width of a tile (K when there is no mask)
  int32_t num_ib, num_jb, lsteps;
  const uint32_t* keep_mask;
  int32_t mask_words;
  void* c_out;
};

// A heavily clamped 128-byte row of a staged A tile: rewrite its 16-byte chunks under the
// expanded keep mask (bit j = keep element j).
__device__ __forceinline__ void rewrite_row_masked(uint32_t row_addr, int sw, uint64_t keep) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t kb = (uint32_t)(keep >> (8 * c)) & 0xffu;
    if (kb == 0xffu) continue;
    const uint32_t addr = row_addr + (uint32_t)((c ^ sw) << 4);
    uint32_t v[4];
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr) : "memory");
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t two = (kb >> (2 * j)) & 3u;
      v[j] &= (two & 1u) * 0x0000ffffu + (two >> 1) * 0xffff0000u;
    }
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]),
                 "r"(v[3]) : "memory");
  }
}

template <bool WGRAD>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
              const BwdTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* stage_base = align_1024(smem_raw);
  Barriers* bars = reinterpret_cast<Barriers*>(stage_base + B_STAGES * B_STAGE_BYTES);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool masked = p.keep_mask != nullptr;
  const int num_work = p.num_ib * p.T * p.num_jb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < B_STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->ready[s], B_XFORM_THREADS / 32);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], B_EPI_WARPS);
    }
    mbar_init(&bars->mma_done, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&bars->tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_slot;

  if (warp == 0) {
    // ---- TMA producer ------------------------------------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const int ib = w / (p.T * p.num_jb);
        const int rem = w % (p.T * p.num_jb);
        const int t = rem / p.num_jb, jb = rem % p.num_jb;
        const int j0 = t * p.tile_w + jb * B_BN;
        for (int ls = 0; ls < p.lsteps; ++ls, ++it) {
          const int s = it % B_STAGES;
          const uint32_t ph = (it / B_STAGES) & 1u;
          if (!mbar_wait(&bars->empty[s], ph ^ 1u, abort_flag)) {
            raise_error(kErrProducer, abort_flag);
            ok = false;
            break;
          }
          uint8_t* sa = stage_base + s * B_STAGE_BYTES;
          uint8_t* sb = sa + B_A_BYTES;
          const int l0 = ls * BK;
          mbar_expect_tx(&bars->full[s], B_STAGE_BYTES);
          if (WGRAD) {
            // A = g^T: two MN-major boxes [64 rows of m] x [64 n]
            tma_load_2d(sa, &map_a, &bars->full[s], ib * BM, l0);
            tma_load_2d(sa + B_BOX_BYTES, &map_a, &bars->full[s], ib * BM + 64, l0);
          } else {
            // A = g: K-major [128 rows of m] x [64 n]
            tma_load_2d(sa, &map_a, &bars->full[s], l0, ib * BM);
          }
#pragma unroll
          for (int c = 0; c < B_BN / 64; ++c)
            tma_load_2d(sb + c * B_BOX_BYTES, &map_b, &bars->full[s], j0 + c * 64, l0);
        }
      }
      const uint32_t n_back = it < (uint32_t)B_STAGES ? it : (uint32_t)B_STAGES;
      for (uint32_t j = it - n_back; j < it; ++j) {
        const int s = j % B_STAGES;
        const uint32_t ph = (j / B_STAGES) & 1u;
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try(&bars->full[s], ph)) {
          if (globaltimer_ns() - t0 > kTimeoutNs) {
            raise_error(kErrDrain, abort_flag);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer --------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, B_BN, WGRAD ? 1 : 0, 1);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++acc_it) {
        const int b = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        if (!mbar_wait(&bars->acc_empty[b], aph ^ 1u, abort_flag)) {
          raise_error(kErrMma, abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * B_BN);
        for (int ls = 0; ls < p.lsteps; ++ls, ++it) {
          const int s = it % B_STAGES;
          const uint32_t ph = (it / B_STAGES) & 1u;
          // the transform warps vouch for a stage on `ready` before its copy has landed when
          // the stage has nothing to zero, so both barriers gate the MMA
          if (!mbar_wait(&bars->full[s], ph, abort_flag) ||
              (masked && !mbar_wait(&bars->ready[s], ph, abort_flag))) {
            raise_error(kErrMma, abort_flag);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + s * B_STAGE_BYTES);
          const uint32_t sb = sa + B_A_BYTES;
          const uint64_t da = WGRAD ? desc_mn_major(sa, B_BOX_BYTES) : desc_k_major(sa);
          const uint64_t db = desc_mn_major(sb, B_BOX_BYTES);
          // one MMA consumes 16 k: 32 bytes along a K-major row, 16 rows (2048 bytes) of an MN-major box
          constexpr uint64_t a_step = WGRAD ? (2048u >> 4) : (32u >> 4);
          constexpr uint64_t b_step = 2048u >> 4;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)
            umma_bf16(d_tmem, da + a_step * k4, db + b_step * k4, idesc, (ls | k4) != 0 ? 1u : 0u);
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[b]);
      }
      umma_commit(&bars->mma_done);
      uint64_t t0 = globaltimer_ns();
      while (!mbar_try(&bars->mma_done, 0)) {
        if (globaltimer_ns() - t0 > kTimeoutNs) {
          raise_error(kErrDrain, abort_flag);
          break;
        }
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ---- epilogue: TMEM -> bf16 -> global ------------------------------------------------
    const int quad = warp & 3;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++acc_it) {
      const int ib = w / (p.T * p.num_jb);
      const int rem = w % (p.T * p.num_jb);
      const int t = rem / p.num_jb, jb = rem % p.num_jb;
      const int j0 = t * p.tile_w + jb * B_BN;
      const int j_end = min((t + 1) * p.tile_w, p.K);
      const int i = ib * BM + quad * 32 + lane;
      const int b = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      if (!mbar_wait(&bars->acc_full[b], aph, abort_flag)) {
        if (lane == 0) raise_error(kErrEpilogue, abort_flag);
        ok = false;
        break;
      }
      tc_fence_after();
      uint16_t* dst_row = reinterpret_cast<uint16_t*>(p.c_out) + (int64_t)i * p.K;
#pragma unroll 1
      for (int c = 0; c < B_BN / 32; ++c) {
        const int jc = j0 + c * 32;
        if (jc >= j_end) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_base + (uint32_t)(b * B_BN + c * 32), r);
        tmem_wait_ld();
        if (i < p.I) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (jc + v * 8 < j_end) {
              uint4 pk = make_uint4(
                  pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1])),
                  pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3])),
                  pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5])),
                  pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7])));
              *reinterpret_cast<uint4*>(dst_row + jc + v * 8) = pk;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[b]);
    }
  } else if (warp >= 8 && masked && (int)blockIdx.x < num_work) {
    // ---- mask transform: zero the gradient entries the tile's ADC clamp blocked ---------
    // B_XFORM_GROUPS groups of 128 threads take the stage-iterations round robin, so that
    // the fix-up of consecutive stages overlaps.  Within a group thread r owns one 128-byte
    // row of the staged A tile and the two mask words that cover it.
    const int grp = (warp - 8) >> 2;
    const int r = threadIdx.x - (8 + 4 * grp) * 32;  // 0..127
    const int row_in_box = WGRAD ? (r & 63) : r;
    const int box = WGRAD ? (r >> 6) : 0;
    const int total = ((num_work - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x) * p.lsteps;
    // Mask words are [T][word][M].  The fetch stream walks (work item, l-step) with a cursor
    // instead of dividing per turn, and its loads are unconditional: indices past an edge
    // are clamped to the last valid row / word.  What a clamped word may zero lies in rows or
    // columns that the TMA copy filled with zeros anyway, and a load that nothing selects on
    // does not stall the warp at the point of issue.
    const int m_last = p.M - 1, w_last = p.mask_words - 1;
    int f_w = (int)blockIdx.x + (grp / p.lsteps) * (int)gridDim.x, f_ls = grp % p.lsteps;
    const uint32_t* f_lo = p.keep_mask;  // dgrad: word 0 of (t, row); wgrad: row 0 of (t, word)
    const uint32_t* f_hi = p.keep_mask;
    auto seek_item = [&]() {
      if (f_w >= num_work) return;  // past the end: keep pointing at valid memory
      const int ib = f_w / (p.T * p.num_jb);
      const int t = (f_w % (p.T * p.num_jb)) / p.num_jb;
      const uint32_t* tile = p.keep_mask + (int64_t)t * p.mask_words * p.M;
      if (WGRAD) {
        const int w0 = (ib * BM + box * 64) >> 5;
        f_lo = tile + (int64_t)min(w0, w_last) * p.M;
        f_hi = tile + (int64_t)min(w0 + 1, w_last) * p.M;
      } else {
        f_lo = tile + min(ib * BM + r, m_last);
        f_hi = f_lo;
      }
    };
    seek_item();
    auto fetch = [&](uint32_t* lo, uint32_t* hi) {
      if (WGRAD) {
        const int m = min(f_ls * BK + row_in_box, m_last);
        *lo = f_lo[m];
        *hi = f_hi[m];
      } else {
        *lo = f_lo[(int64_t)min(2 * f_ls, w_last) * p.M];
        *hi = f_hi[(int64_t)min(2 * f_ls + 1, w_last) * p.M];
      }
      f_ls += B_XFORM_GROUPS;
      if (f_ls >= p.lsteps) {
        do {
          f_ls -= p.lsteps;
          f_w += (int)gridDim.x;
        } while (f_ls >= p.lsteps);
        seek_item();
      }
    };
    constexpr int kScanLimit = 6;  // blocked entries per row up to which single stores beat a rewrite
    uint8_t* const row_base = stage_base + box * B_BOX_BYTES + row_in_box * 128;
    const int sw = r & 7;  // 128-byte swizzle: 16-byte chunk index is XORed with row % 8
    // one stage-iteration of this thread's row; false = the wait gave up
    auto process = [&](int it, uint32_t lo, uint32_t hi) -> bool {
      const int s = it % B_STAGES;
      const uint32_t ph = ((uint32_t)it / B_STAGES) & 1u;
      uint64_t zeros = ~((uint64_t)lo | ((uint64_t)hi << 32));
      // A parity wait tells phases apart only one phase deep, and a warp that had nothing to
      // zero on the stage's previous use never looked at `full` then: first wait until that
      // previous use has been consumed (normally long past), which puts `full` and `ready`
      // of this stage in the phase of this use.
      bool okw = true;
      if (lane == 0) {
        okw = mbar_wait(&bars->empty[s], ph ^ 1u, abort_flag);
        if (!okw) raise_error(kErrTransform, abort_flag);
      }
      if (!__shfl_sync(0xffffffffu, okw, 0)) return false;
      if (!__any_sync(0xffffffffu, zeros != 0ull)) {
        // Nothing to zero in this warp's rows: it vouches for the stage before the copy has
        // landed, which takes this hand-off off the TMA -> MMA critical path, and it
        // publishes no data, so the arrival is a relaxed one.
        if (lane == 0) mbar_arrive_relaxed(&bars->ready[s]);
        return true;
      }
      if (!mbar_wait(&bars->full[s], ph, abort_flag)) {
        raise_error(kErrTransform, abort_flag);
        return false;
      }
      if (zeros != 0ull) {
        const uint32_t row_addr = smem_u32(row_base + s * B_STAGE_BYTES);
        if (__popcll(zeros) <= kScanLimit) {
          // one 2-byte store of zero per blocked element (typically one or two per row)
          while (zeros != 0ull) {
            const int pos = __ffsll((long long)zeros) - 1;  // n - n0 of the blocked element
            zeros &= zeros - 1ull;
            const uint32_t addr = row_addr + (uint32_t)((((pos >> 3) ^ sw) << 4) + ((pos & 7) << 1));
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)0) : "memory");
          }
        } else {
          rewrite_row_masked(row_addr, sw, ~zeros);
        }
        fence_proxy_async_smem();
      }
      // one arrival per warp: 128 arrivals on one mbarrier would serialise in shared memory
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ready[s]);
      return true;
    };
    // The mask words run kAhead turns ahead of their use in a ring of registers (the loop is
    // unrolled by the ring size so that every slot is a fixed register): a turn never waits
    // for a load it issued itself.
    constexpr int kRing = 4, kAhead = 3;
    uint32_t lo[kRing], hi[kRing];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) fetch(&lo[u], &hi[u]);
    bool ok = true;
    for (int base = grp; base < total && ok; base += kRing * B_XFORM_GROUPS) {
#pragma unroll
      for (int u = 0; u < kRing; ++u) {
        const int it = base + u * B_XFORM_GROUPS;
        if (it < total && ok) {
          fetch(&lo[(u + kAhead) % kRing], &hi[(u + kAhead) % kRing]);
          ok = process(it, lo[u], hi[u]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// backward (dgrad / wgrad) on CTA pairs
// ---------------------------------------------------------------------------------------------
// Same GEMM as bwd_tc_kernel with one tcgen05.mma.cta_group::2 of 256 x 256 x 16 per k-step.
// CTA `rank` of the pair owns rows [256 ib + 128 rank, +128) of C: it stages those rows of A and
// columns [128 rank, +128) of the B block, holds its half of the accumulator in its own tensor
// memory and writes its rows of C.  Each CTA therefore stages 32 KiB per 64-deep k-step instead of
// 48 KiB, which buys two more pipeline stages and takes a third off the L2 -> shared-memory
// traffic per flop.
//
// Barriers.  `empty`, `acc_full`: one copy per CTA, signalled in both by the leader's multicast
// commit.  `acc_empty`, `ready`, `mma_done`: used in the leader (rank 0) only; the other CTA
// arrives on them through the cluster address.  `full`: without a mask the leader's barrier
// collects the bytes of both CTAs' copies and gates the MMA; with a mask each CTA's copies
// complete on its own barrier, its transform warps fix the A tile up and then vouch for the
// stage on the leader's `ready`, which gates the MMA.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try_cluster(bar, parity)) return true;
    if ((spin & 31u) == 31u) {
      if (*abort_flag) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kTimeoutNs) return false;
    }
  }
}

template <bool WGRAD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kBwdThreads, 1)
bwd_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const BwdTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* stage_base = align_1024(smem_raw);
  Barriers* bars = reinterpret_cast<Barriers*>(stage_base + P_STAGES * P_STAGE_BYTES);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const bool masked = p.keep_mask != nullptr;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int num_work = p.num_ib * p.T * p.num_jb;  // num_ib counts 256-row blocks here
  const int row_off = (int)rank * BM;               // this CTA's rows inside the pair's block

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->ready[s], 2 * (B_XFORM_THREADS / 32));
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 2 * B_EPI_WARPS);
    }
    mbar_init(&bars->mma_done, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc_pair(&bars->tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_slot;

  if (warp == 0) {
    // ---- TMA producer (both CTAs) --------------------------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (int w = pair; w < num_work && ok; w += n_pairs) {
        const int ib = w / (p.T * p.num_jb);
        const int rem = w % (p.T * p.num_jb);
        const int t = rem / p.num_jb, jb = rem % p.num_jb;
        const int i0 = ib * (2 * BM) + row_off;
        const int j0 = t * p.tile_w + jb * P_BN + (int)rank * P_BN_CTA;
        for (int ls = 0; ls < p.lsteps; ++ls, ++it) {
          const int s = it % P_STAGES;
          const uint32_t ph = (it / P_STAGES) & 1u;
          if (!mbar_wait_cluster(&bars->empty[s], ph ^ 1u, abort_flag)) {
            raise_error(kErrProducer, abort_flag);
            ok = false;
            break;
          }
          uint8_t* sa = stage_base + s * P_STAGE_BYTES;
          uint8_t* sb = sa + P_A_BYTES;
          const int l0 = ls * BK;
          uint32_t bar;
          if (masked) {
            mbar_expect_tx(&bars->full[s], P_STAGE_BYTES);
            bar = smem_u32(&bars->full[s]);
          } else {
            if (leader) mbar_expect_tx(&bars->full[s], 2 * P_STAGE_BYTES);
            bar = mapa_u32(smem_u32(&bars->full[s]), 0);
          }
          if (WGRAD) {
            tma_load_2d_pair(sa, &map_a, bar, i0, l0);
            tma_load_2d_pair(sa + B_BOX_BYTES, &map_a, bar, i0 + 64, l0);
          } else {
            tma_load_2d_pair(sa, &map_a, bar, l0, i0);
          }
#pragma unroll
          for (int c = 0; c < P_BN_CTA / 64; ++c)
            tma_load_2d_pair(sb + c * B_BOX_BYTES, &map_b, bar, j0 + c * 64, l0);
        }
      }
      // drain: copies that complete on this CTA's own barrier must have landed before it exits;
      // copies that complete on the leader's barrier are covered by the leader's drain and the
      // cluster barrier at the end
      if (masked || leader) {
        const uint32_t n_back = it < (uint32_t)P_STAGES ? it : (uint32_t)P_STAGES;
        for (uint32_t j = it - n_back; j < it; ++j) {
          const int s = j % P_STAGES;
          const uint32_t ph = (j / P_STAGES) & 1u;
          uint64_t t0 = globaltimer_ns();
          while (!mbar_try_cluster(&bars->full[s], ph)) {
            if (globaltimer_ns() - t0 > kTimeoutNs) {
              raise_error(kErrDrain, abort_flag);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (leader only) --------------------------------------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(2 * BM, P_BN, WGRAD ? 1 : 0, 1);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int w = pair; w < num_work && ok; w += n_pairs, ++acc_it) {
        const int b = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        if (!mbar_wait_cluster(&bars->acc_empty[b], aph ^ 1u, abort_flag)) {
          raise_error(kErrMma, abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * P_BN);
        for (int ls = 0; ls < p.lsteps; ++ls, ++it) {
          const int s = it % P_STAGES;
          const uint32_t ph = (it / P_STAGES) & 1u;
          if (!mbar_wait_cluster(masked ? &bars->ready[s] : &bars->full[s], ph, abort_flag)) {
            raise_error(kErrMma, abort_flag);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + s * P_STAGE_BYTES);
          const uint32_t sb = sa + P_A_BYTES;
          const uint64_t da = WGRAD ? desc_mn_major(sa, B_BOX_BYTES) : desc_k_major(sa);
          const uint64_t db = desc_mn_major(sb, B_BOX_BYTES);
          constexpr uint64_t a_step = WGRAD ? (2048u >> 4) : (32u >> 4);
          constexpr uint64_t b_step = 2048u >> 4;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)
            umma_bf16_pair(d_tmem, da + a_step * k4, db + b_step * k4, idesc, (ls | k4) != 0 ? 1u : 0u);
          umma_commit_pair(&bars->empty[s], 3);  // frees the stage in both CTAs
        }
        if (ok) umma_commit_pair(&bars->acc_full[b], 3);
      }
      umma_commit_pair(&bars->mma_done, 1);
      uint64_t t0 = globaltimer_ns();
      while (!mbar_try_cluster(&bars->mma_done, 0)) {
        if (globaltimer_ns() - t0 > kTimeoutNs) {
          raise_error(kErrDrain, abort_flag);
          break;
        }
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ---- epilogue (both CTAs): own half of the accumulator -> bf16 -> own rows of C --------
    const int quad = warp & 3;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int w = pair; w < num_work && ok; w += n_pairs, ++acc_it) {
      const int ib = w / (p.T * p.num_jb);
      const int rem = w % (p.T * p.num_jb);
      const int t = rem / p.num_jb, jb = rem % p.num_jb;
      const int j0 = t * p.tile_w + jb * P_BN;
      const int j_end = min((t + 1) * p.tile_w, p.K);
      const int i = ib * (2 * BM) + row_off + quad * 32 + lane;
      const int b = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      if (!mbar_wait_cluster(&bars->acc_full[b], aph, abort_flag)) {
        if (lane == 0) raise_error(kErrEpilogue, abort_flag);
        ok = false;
        break;
      }
      tc_fence_after();
      uint16_t* dst_row = reinterpret_cast<uint16_t*>(p.c_out) + (int64_t)i * p.K;
#pragma unroll 1
      for (int c = 0; c < P_BN / 32; ++c) {
        const int jc = j0 + c * 32;
        if (jc >= j_end) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_base + (uint32_t)(b * P_BN + c * 32), r);
        tmem_wait_ld();
        if (i < p.I) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (jc + v * 8 < j_end) {
              uint4 pk = make_uint4(
                  pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1])),
                  pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3])),
                  pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5])),
                  pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7])));
              *reinterpret_cast<uint4*>(dst_row + jc + v * 8) = pk;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars->acc_empty[b]), 0));
    }
  } else if (warp >= 8 && masked && pair < num_work) {
    // ---- mask transform (both CTAs, own A tile): see bwd_tc_kernel -------------------------
    const int grp = (warp - 8) >> 2;
    const int r = threadIdx.x - (8 + 4 * grp) * 32;  // 0..127
    const int row_in_box = WGRAD ? (r & 63) : r;
    const int box = WGRAD ? (r >> 6) : 0;
    const int total = ((num_work - pair + n_pairs - 1) / n_pairs) * p.lsteps;
    const int m_last = p.M - 1, w_last = p.mask_words - 1;
    int f_w = pair + (grp / p.lsteps) * n_pairs, f_ls = grp % p.lsteps;
    const uint32_t* f_lo = p.keep_mask;
    const uint32_t* f_hi = p.keep_mask;
    auto seek_item = [&]() {
      if (f_w >= num_work) return;
      const int ib = f_w / (p.T * p.num_jb);
      const int t = (f_w % (p.T * p.num_jb)) / p.num_jb;
      const int i0 = ib * (2 * BM) + row_off;
      const uint32_t* tile = p.keep_mask + (int64_t)t * p.mask_words * p.M;
      if (WGRAD) {
        const int w0 = (i0 + box * 64) >> 5;
        f_lo = tile + (int64_t)min(w0, w_last) * p.M;
        f_hi = tile + (int64_t)min(w0 + 1, w_last) * p.M;
      } else {
        f_lo = tile + min(i0 + r, m_last);
        f_hi = f_lo;
      }
    };
    seek_item();
    auto fetch = [&](uint32_t* lo, uint32_t* hi) {
      if (WGRAD) {
        const int m = min(f_ls * BK + row_in_box, m_last);
        *lo = f_lo[m];
        *hi = f_hi[m];
      } else {
        *lo = f_lo[(int64_t)min(2 * f_ls, w_last) * p.M];
        *hi = f_hi[(int64_t)min(2 * f_ls + 1, w_last) * p.M];
      }
      f_ls += B_XFORM_GROUPS;
      if (f_ls >= p.lsteps) {
        do {
          f_ls -= p.lsteps;
          f_w += n_pairs;
        } while (f_ls >= p.lsteps);
        seek_item();
      }
    };
    constexpr int kScanLimit = 6;
    uint8_t* const row_base = stage_base + box * B_BOX_BYTES + row_in_box * 128;
    const int sw = r & 7;
    auto process = [&](int it, uint32_t lo, uint32_t hi) -> bool {
      const int s = it % P_STAGES;
      const uint32_t ph = ((uint32_t)it / P_STAGES) & 1u;
      // the MMA waits on `ready` alone, so every warp waits for its CTA's copy before it vouches
      if (!mbar_wait(&bars->full[s], ph, abort_flag)) {
        raise_error(kErrTransform, abort_flag);
        return false;
      }
      uint64_t zeros = ~((uint64_t)lo | ((uint64_t)hi << 32));
      if (zeros != 0ull) {
        const uint32_t row_addr = smem_u32(row_base + s * P_STAGE_BYTES);
        if (__popcll(zeros) <= kScanLimit) {
          while (zeros != 0ull) {
            const int pos = __ffsll((long long)zeros) - 1;
            zeros &= zeros - 1ull;
            const uint32_t addr = row_addr + (uint32_t)((((pos >> 3) ^ sw) << 4) + ((pos & 7) << 1));
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)0) : "memory");
          }
        } else {
          rewrite_row_masked(row_addr, sw, ~zeros);
        }
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars->ready[s]), 0));
      return true;
    };
    constexpr int kRing = 4, kAhead = 3;
    uint32_t lo[kRing], hi[kRing];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) fetch(&lo[u], &hi[u]);
    bool ok = true;
    for (int base = grp; base < total && ok; base += kRing * B_XFORM_GROUPS) {
#pragma unroll
      for (int u = 0; u < kRing; ++u) {
        const int it = base + u * B_XFORM_GROUPS;
        if (it < total && ok) {
          fetch(&lo[(u + kAhead) % kRing], &hi[(u + kAhead) % kRing]);
          ok = process(it, lo[u], hi[u]);
        }
      }
    }
  }

  // nothing of this CTA's shared or tensor memory may go while the peer can still signal or
  // read it: both CTAs meet before the pair's tensor memory is released
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    else
      cudaGetLastError();
  }
  return fn;
}

// bf16 tensor map with 128-byte swizzle.  dims/strides innermost first; strides in bytes for
// dims 1.. (the innermost stride is the element size).
int make_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
             const uint32_t* box) {
  PFN_cuTensorMapEncodeTiled_v12000 fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return AL_ERR_CUDA;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bdim[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr,
                  bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return AL_ERR_CUDA;
  }
  return AL_OK;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

constexpr int F_SMEM = F_STAGES * F_STAGE_BYTES + (int)sizeof(Barriers) + 1024;
constexpr int B_SMEM = B_STAGES * B_STAGE_BYTES + (int)sizeof(Barriers) + 1024;
constexpr int P_SMEM = P_STAGES * P_STAGE_BYTES + (int)sizeof(Barriers) + 1024;
constexpr int FP_SMEM = FP_STAGES * F_STAGE_BYTES + FP_SUM_BYTES + (int)sizeof(Barriers) + 1024;

template <class Kernel>
int ensure_smem(Kernel k, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(%d bytes): %s", bytes, cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  return AL_OK;
}

bool uniform_tiles(const TileTable& tt, int* width) {
  int w = tt.hi(0);
  for (int t = 1; t < tt.T; ++t)
    if (tt.hi(t) - tt.lo(t) != w) return false;
  *width = w;
  return true;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// bf16, all analog tiles equally wide, every row pitch and tile offset a multiple of 16 bytes
static bool tc_shape_ok(const AlDesc& d, const TileTable& tt) {
  int w = 0;
  if (d.dtype != AL_BF16) return false;
  if (!uniform_tiles(tt, &w)) return false;
  if (w % 8 != 0 || d.K % 8 != 0 || d.N % 8 != 0) return false;
  return true;
}
bool tc_forward_supported(const AlDesc& d, const TileTable& tt) { return tc_shape_ok(d, tt); }
bool tc_backward_supported(const AlDesc& d, const TileTable& tt) { return tc_shape_ok(d, tt); }

using FwdKernel = void (*)(const CUtensorMap, const CUtensorMap, const FwdTcParams);
template <bool PAIR>
static FwdKernel pick_fwd_kernel(int mode, int round_dt) {
  switch (mode) {
    case 0: return fwd_tc_kernel<kBF16, 0, PAIR>;
    case 1: return fwd_tc_kernel<kBF16, 1, PAIR>;
    case 2: return fwd_tc_kernel<kBF16, 2, PAIR>;
    case 3: return fwd_tc_kernel<kBF16, 3, PAIR>;
    case 4: return fwd_tc_kernel<kBF16, 4, PAIR>;
    case 5: return fwd_tc_kernel<kBF16, 5, PAIR>;
    case 6: return fwd_tc_kernel<kBF16, 6, PAIR>;
    case 7: return fwd_tc_kernel<kBF16, 7, PAIR>;
    default:
      // CTA pairs exist for bf16 rounding only
      if (PAIR) return fwd_tc_kernel<kBF16, -1, PAIR>;
      return round_dt == AL_BF16 ? fwd_tc_kernel<kBF16, -1, false> : fwd_tc_kernel<kF32, -1, false>;
  }
}
// launch configuration of a kernel that runs as clusters of two CTAs
struct PairLaunch {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr;
  PairLaunch(int grid, int threads, int smem, cudaStream_t s) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
};
// how many CTA pairs of the forward kernel the device runs at once (0: it cannot)
static int max_fwd_pairs(FwdKernel kernel) {
  static FwdKernel seen[24];
  static int count[24];
  static int n_seen = 0;
  for (int i = 0; i < n_seen; ++i)
    if (seen[i] == kernel) return count[i];
  int clusters = 0;
  PairLaunch pl(2 * sm_count(), kFwdThreads, FP_SMEM, nullptr);
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &pl.cfg) != cudaSuccess) {
    cudaGetLastError();
    clusters = 0;
  }
  if (n_seen < 24) {
    seen[n_seen] = kernel;
    count[n_seen++] = clusters;
  }
  return clusters;
}

int launch_fwd_tc(int round_dt, const void* xq, const void* w_mod, int K, const TileTable& tt,
                  const FwdEpilogueParams& ep, int pairing, void* out, cudaStream_t s) {
  ProfScope prof(AL_K_FWD_GEMM, s);
  int w = 0;
  if (!uniform_tiles(tt, &w) || !aligned16(xq) || !aligned16(w_mod) || !aligned16(out)) {
    set_error("fwd_tc: operands must be 16-byte aligned with equally wide tiles");
    return AL_ERR_UNSUPPORTED;
  }
  FwdTcParams p;
  p.tile_w = w;
  p.ksteps = (w + BK - 1) / BK;
  p.num_mb = (ep.M + BM - 1) / BM;
  p.num_nb = (ep.N + F_BN - 1) / F_BN;
  p.ep = ep;
  p.noise = make_noise_keys(ep.seed, ep.offset, 1u);
  p.out = out;
  {
    // |o| <= tile_w * ir * wmax * (1 + noise) and step = 2 * out_bound * ir * wmax / states
    double states = ep.out_res > 1.0f ? ep.out_res : (ep.out_res > 0.0f ? 1.0 / ep.out_res : 1.0);
    double max_code = 8.0 * (double)w * states / (2.0 * (ep.out_bound > 0.0f ? ep.out_bound : 1.0));
    p.small_adc_codes = max_code < 274877906944.0 ? 1 : 0;  // 2^38
  }
  const bool per_channel = ep.w_amax != nullptr && (ep.noise_pc || ep.bound_pc);
  const bool fixed = round_dt == AL_BF16 && !per_channel && ep.out_noise == nullptr && !ep.no_rounding &&
                     p.small_adc_codes;
  const int mode = fixed ? ((ep.has_noise ? 1 : 0) | (ep.has_adc ? 2 : 0) | (ep.has_bound ? 4 : 0)) : -1;
  // CTA pairs (256 x 256 blocks, packed bf16 output stage only) when there is a block per pair
  // of SMs; single CTAs (128 x 128) otherwise.
  // The runtime calls below also bind the device's primary context to the calling thread
  // (autograd runs backward on its own threads); the driver entry point that encodes the
  // tensor maps needs a current context.
  const bool pair_ok = pairing >= 0 && round_dt == AL_BF16 && !per_channel;
  const int pair_tiles = ((ep.M + 2 * BM - 1) / (2 * BM)) * ((ep.N + 2 * F_BN - 1) / (2 * F_BN));
  FwdKernel kernel = nullptr;
  int rc = AL_OK, pairs = 0;
  if (pair_ok) {
    kernel = pick_fwd_kernel<true>(mode, round_dt);
    rc = ensure_smem(kernel, FP_SMEM);
    if (rc) return rc;
    pairs = max_fwd_pairs(kernel);
  }
  const bool pair = pairs > 0 && (pair_tiles >= pairs || pairing > 0);
  if (!pair) {
    kernel = pick_fwd_kernel<false>(mode, round_dt);
    rc = ensure_smem(kernel, F_SMEM);
    if (rc) return rc;
  } else {
    p.num_mb = (ep.M + 2 * BM - 1) / (2 * BM);
    p.num_nb = (ep.N + 2 * F_BN - 1) / (2 * F_BN);
  }
  CUtensorMap map_a, map_b;
  {
    uint64_t dims[3] = {(uint64_t)w, (uint64_t)tt.T, (uint64_t)ep.M};
    uint64_t strides[2] = {(uint64_t)w * 2, (uint64_t)K * 2};
    uint32_t box[3] = {BK, 1, BM};
    rc = make_map(&map_a, xq, 3, dims, strides, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)w, (uint64_t)tt.T, (uint64_t)ep.N};
    uint64_t strides[2] = {(uint64_t)w * 2, (uint64_t)K * 2};
    uint32_t box[3] = {BK, 1, F_BN};
    rc = make_map(&map_b, w_mod, 3, dims, strides, box);
    if (rc) return rc;
  }
  if (pair) {
    PairLaunch pl(2 * (pair_tiles < pairs ? pair_tiles : pairs), kFwdThreads, FP_SMEM, s);
    cudaError_t e = cudaLaunchKernelEx(&pl.cfg, kernel, map_a, map_b, p);
    if (e != cudaSuccess) {
      set_error("fwd_tc (pairs): %s", cudaGetErrorString(e));
      return AL_ERR_CUDA;
    }
    return check_launch("fwd_tc_pair");
  }
  int tiles = p.num_mb * p.num_nb;
  int grid = tiles < sm_count() ? tiles : sm_count();
  kernel<<<grid, kFwdThreads, F_SMEM, s>>>(map_a, map_b, p);
  return check_launch("fwd_tc");
}

// How many 2-CTA clusters of the pair kernel the device runs at once (0: cannot run them).
static int max_pairs(bool wgrad) {
  static int cached[2] = {-1, -1};
  int& n = cached[wgrad ? 1 : 0];
  if (n >= 0) return n;
  n = 0;
  if ((wgrad ? ensure_smem(bwd_tc_pair_kernel<true>, P_SMEM) : ensure_smem(bwd_tc_pair_kernel<false>, P_SMEM)) != AL_OK)
    return n;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sm_count());
  cfg.blockDim = dim3(kBwdThreads);
  cfg.dynamicSmemBytes = P_SMEM;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  cudaError_t e = wgrad ? cudaOccupancyMaxActiveClusters(&clusters, bwd_tc_pair_kernel<true>, &cfg)
                        : cudaOccupancyMaxActiveClusters(&clusters, bwd_tc_pair_kernel<false>, &cfg);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return n;
  }
  n = clusters;
  return n;
}
static int launch_bwd_tc(bool wgrad, const void* g, const void* b_op, const uint32_t* keep_mask,
                         int mask_words, int M, int K, int N, const TileTable& tt, int pairing, void* c_out,
                         cudaStream_t s) {
  int w = 0;
  if (!uniform_tiles(tt, &w) || !aligned16(g) || !aligned16(b_op) || !aligned16(c_out)) {
    set_error("bwd_tc: operands must be 16-byte aligned with equally wide tiles");
    return AL_ERR_UNSUPPORTED;
  }
  BwdTcParams p;
  p.I = wgrad ? N : M;
  p.L = wgrad ? M : N;
  p.K = K;
  p.M = M;
  p.T = tt.T;
  p.tile_w = w;
  p.num_ib = (p.I + BM - 1) / BM;
  p.num_jb = (w + B_BN - 1) / B_BN;
  p.lsteps = (p.L + BK - 1) / BK;
  p.keep_mask = keep_mask;
  p.mask_words = mask_words;
  p.c_out = c_out;
  int rc = wgrad ? ensure_smem(bwd_tc_kernel<true>, B_SMEM) : ensure_smem(bwd_tc_kernel<false>, B_SMEM);
  if (rc) return rc;
  CUtensorMap map_a, map_b;
  {
    // g [M,N]: dims innermost first {N, M}
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)N * 2};
    uint32_t box_k[2] = {BK, BM};   // dgrad: 64 n (reduction) x 128 m
    uint32_t box_mn[2] = {64, BK};  // wgrad: 64 n (MMA-M) x 64 m (reduction)
    rc = make_map(&map_a, g, 2, dims, strides, wgrad ? box_mn : box_k);
    if (rc) return rc;
  }
  {
    // B operand [L, K] row-major (w_mod [N,K] for dgrad, xq [M,K] for wgrad): {K, L}
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)p.L};
    uint64_t strides[1] = {(uint64_t)K * 2};
    uint32_t box[2] = {64, BK};
    rc = make_map(&map_b, b_op, 2, dims, strides, box);
    if (rc) return rc;
  }
  // CTA pairs (256-row blocks) when they fill the machine; single CTAs for smaller problems
  const int pair_work = ((p.I + 2 * BM - 1) / (2 * BM)) * p.T * p.num_jb;
  const int pairs = max_pairs(wgrad);
  if (pairs > 0 && pairing >= 0 && (pair_work >= pairs || pairing > 0)) {
    p.num_ib = (p.I + 2 * BM - 1) / (2 * BM);
    rc = wgrad ? ensure_smem(bwd_tc_pair_kernel<true>, P_SMEM) : ensure_smem(bwd_tc_pair_kernel<false>, P_SMEM);
    if (rc) return rc;
    const int grid = 2 * (pair_work < pairs ? pair_work : pairs);
    if (wgrad)
      bwd_tc_pair_kernel<true><<<grid, kBwdThreads, P_SMEM, s>>>(map_a, map_b, p);
    else
      bwd_tc_pair_kernel<false><<<grid, kBwdThreads, P_SMEM, s>>>(map_a, map_b, p);
    return check_launch(wgrad ? "wgrad_tc_pair" : "dgrad_tc_pair");
  }
  int work = p.num_ib * p.T * p.num_jb;
  int grid = work < sm_count() ? work : sm_count();
  if (wgrad)
    bwd_tc_kernel<true><<<grid, kBwdThreads, B_SMEM, s>>>(map_a, map_b, p);
  else
    bwd_tc_kernel<false><<<grid, kBwdThreads, B_SMEM, s>>>(map_a, map_b, p);
  return check_launch(wgrad ? "wgrad_tc" : "dgrad_tc");
}

int launch_dgrad_tc(const void* g, const void* w_mod, const uint32_t* keep_mask, int mask_words,
                    int M, int K, int N, const TileTable& tt, int pairing, void* grad_x, cudaStream_t s) {
  ProfScope prof(AL_K_DGRAD_GEMM, s);
  return launch_bwd_tc(false, g, w_mod, keep_mask, mask_words, M, K, N, tt, pairing, grad_x, s);
}

int launch_wgrad_tc(const void* g, const void* xq, const uint32_t* keep_mask, int mask_words,
                    int M, int K, int N, const TileTable& tt, int pairing, void* grad_w, cudaStream_t s) {
  ProfScope prof(AL_K_WGRAD_GEMM, s);
  return launch_bwd_tc(true, g, xq, keep_mask, mask_words, M, K, N, tt, pairing, grad_w, s);
}

int tc_read_device_error(cudaStream_t s, uint32_t* code) {
  cudaError_t e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    set_error("al_read_device_error: %s", cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  uint32_t zero = 0;
  e = cudaMemcpyFromSymbol(code, g_tc_error_word, sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_tc_error_word, &zero, sizeof(uint32_t));
  if (e != cudaSuccess) {
    set_error("al_read_device_error: %s", cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  if (*code != 0) {
    set_error("a device-side wait of the tcgen05 kernels gave up (role mask 0x%x)", *code);
    return AL_ERR_DEVICE_TIMEOUT;
  }
  return AL_OK;
}

}  // namespace al
