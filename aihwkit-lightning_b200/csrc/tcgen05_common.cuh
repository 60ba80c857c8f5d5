// Shared by the tcgen05 GEMM translation units (forward, backward): tile constants, PTX wrappers
// for TMA, mbarriers, tensor memory and tcgen05.mma (single CTAs and CTA pairs), shared-memory
// and instruction descriptors, the barrier block of a CTA, and the host helpers that encode
// tensor maps and size launches.  Everything has internal linkage: each translation unit gets
// its own copy, including its own device error word.
//
// Every wait on an mbarrier is bounded (wall-clock limit); a wait that gives up raises the
// device error word, makes the CTA drain its copies in flight, free its TMEM and return.
// No TMA load uses multicast (tcgen05.commit multicasts its mbarrier arrival to a CTA pair).
#pragma once

#include <cuda.h>
#include <cudaTypedefs.h>

#include "analog_math.cuh"
#include "device_fast.cuh"
#include "internal.h"

namespace al {

namespace {

__device__ uint32_t g_tc_error_word = 0;
// Wall-clock limit of every device-side wait, in nanoseconds.  A variable (not a constant) so that
// a test can make the waits run out (al_set_device_wait_limit_ns): a wait that gives up raises
// the error word and the CTA leaves in an orderly way.  Read on the slow path of a wait only.
__device__ unsigned long long g_tc_wait_limit_ns = 2000000000ull;
// Test aid: non-zero makes the forward kernel's MMA issuer withhold the "accumulator full" signal,
// so that the output-stage warps' wait for it runs out (nothing traps or spins without bound: the
// wait gives up after the limit above, the other roles see the abort flag and the kernel returns).
__device__ uint32_t g_tc_withhold_acc_signal = 0;

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle span
constexpr int kThreads = 384;          // 12 warps
constexpr uint64_t kDefaultWaitLimitNs = 2000000000ull;
// A waiting thread is parked by the barrier unit for up to this long per attempt and wakes when
// the barrier's state changes: a thread that polls in a tight loop takes issue slots from the
// warps of its scheduler that have work to do, and the producer and the MMA issuer wait nearly
// all the time.  (Measured: sleeping a fixed time between polls instead is slower -- the wake-up
// then lags the event -- and plain polling slower still.)
constexpr uint32_t kSuspendHintNs = 20000u;

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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t wait_limit_ns() { return *(volatile unsigned long long*)&g_tc_wait_limit_ns; }
// Bounded wait.  Returns false when the wait gave up (time limit, or another role aborted).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 3u) == 3u) {
      if (*abort_flag) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > wait_limit_ns()) return false;
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
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
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

// all analog tiles equally wide, every row pitch and tile offset of the bf16 operands a multiple of 16 bytes
bool tc_tiling_ok(const AlDesc& d, const TileTable& tt) {
  int w = 0;
  if (!uniform_tiles(tt, &w)) return false;
  if (w % 8 != 0 || d.K % 8 != 0 || d.N % 8 != 0) return false;
  return true;
}
bool tc_shape_ok(const AlDesc& d, const TileTable& tt) { return d.dtype == AL_BF16 && tc_tiling_ok(d, tt); }

// Sets this translation unit's limit of the device-side waits.
cudaError_t set_wait_limit(unsigned long long ns) {
  return cudaMemcpyToSymbol(g_tc_wait_limit_ns, &ns, sizeof(ns));
}

cudaError_t set_withhold_acc_signal(uint32_t on) {
  return cudaMemcpyToSymbol(g_tc_withhold_acc_signal, &on, sizeof(on));
}

// Takes (reads and clears) this translation unit's device error word.  The stream must be idle.
cudaError_t take_error_word(uint32_t* code) {
  uint32_t zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(code, g_tc_error_word, sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_tc_error_word, &zero, sizeof(uint32_t));
  return e;
}

}  // namespace

}  // namespace al
