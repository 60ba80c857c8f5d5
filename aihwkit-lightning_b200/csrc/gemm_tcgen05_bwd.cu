// Backward GEMMs of the analog linear path on the Blackwell tensor cores (sm_100a):
//   C[i, lo_t + j] = sum_l (g * keep_t)(i,l) * B(l, lo_t + j)
// dgrad (C = grad_x, A = g, B = w_mod) and wgrad (C = grad_w, A = g^T, B = xq) in one template.
// TMA brings the operands into shared memory (the ones that are contiguous along the output
// dimension as MN-major tiles), groups of four warps apply the ADC clamp mask of the analog tile
// to the staged gradient tile, tcgen05.mma accumulates in tensor memory, four warps drain it.
// Large problems run on CTA pairs (256 x 256 blocks, cta_group::2, six stages), small ones on
// single CTAs (128 x 256 blocks, four stages).
#include "tcgen05_common.cuh"

namespace al {

namespace {

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
  // fp32 layers: the operands arrive as bf16 planes (third dimension of the tensor maps) and an
  // output block accumulates `products` plane products, product q = A plane pa[q] x B plane pb[q];
  // bf16 layers: one product of plane 0.  A has a_planes_per_tile planes per analog tile when the
  // caller prepared it per tile (clamp mask / DAC step folded in), 0 when all tiles share it.
  int32_t products;
  uint8_t pa[8], pb[8];
  int32_t a_planes_per_tile;
  int32_t f32_out;          // C is fp32 (else bf16)
  const float* c_scale_ir;  // [T] input ranges: C[:, tile t] is multiplied by the DAC step of tile t (null: no scaling)
  float inp_res;
  // Reduction split over CTAs (single-CTA kernel, no mask): an output block is computed `splits` times,
  // copy sp over the l-steps [sp * split_lsteps, (sp + 1) * split_lsteps), and stored as fp32 to
  // partial[sp][I][K]; a second kernel adds the copies in the order of sp.  1: no split.
  int32_t splits, split_lsteps;
  float* partial;
};

// r += the 32 columns of the cross-term accumulator at taddr (fp32, round to nearest)
__device__ __forceinline__ void add_cross_terms(uint32_t taddr, uint32_t r[32]) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t x[16];
    tmem_ld16(taddr + (uint32_t)(half * 16), x);
    tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 16; ++j)
      r[half * 16 + j] = __float_as_uint(__fadd_rn(__uint_as_float(r[half * 16 + j]), __uint_as_float(x[j])));
  }
}

// 32 accumulator columns of one row -> C (bf16 or fp32), columns jc .. jc + 31 clipped at j_end
__device__ __forceinline__ void store_c_row(void* c_out, bool f32_out, int ld, int64_t row, int jc, int j_end,
                                            const uint32_t r[32], float scale) {
  if (f32_out) {
    float* dst = reinterpret_cast<float*>(c_out) + row * ld + jc;
#pragma unroll
    for (int v = 0; v < 8; ++v)
      if (jc + v * 4 < j_end)
        *reinterpret_cast<float4*>(dst + v * 4) =
            make_float4(__uint_as_float(r[v * 4]) * scale, __uint_as_float(r[v * 4 + 1]) * scale,
                        __uint_as_float(r[v * 4 + 2]) * scale, __uint_as_float(r[v * 4 + 3]) * scale);
  } else {
    uint16_t* dst = reinterpret_cast<uint16_t*>(c_out) + row * ld + jc;
#pragma unroll
    for (int v = 0; v < 4; ++v)
      if (jc + v * 8 < j_end)
        *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(
            pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1])),
            pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3])),
            pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5])),
            pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7])));
  }
}

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
  const bool split_acc = p.products > 1;
  const int per_split = p.num_ib * p.T * p.num_jb;
  const int num_work = per_split * p.splits;  // item w: copy w / per_split of output block w % per_split

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
        const int sp = w / per_split, blk = w - sp * per_split;
        const int ib = blk / (p.T * p.num_jb);
        const int rem = blk % (p.T * p.num_jb);
        const int t = rem / p.num_jb, jb = rem % p.num_jb;
        const int j0 = t * p.tile_w + jb * B_BN;
        const int ls0 = sp * p.split_lsteps, ls1 = min(ls0 + p.split_lsteps, p.lsteps);
        for (int q = 0; q < p.products && ok; ++q) {
          const int plane_a = p.pa[q] + t * p.a_planes_per_tile, plane_b = p.pb[q];
          for (int ls = ls0; ls < ls1; ++ls, ++it) {
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
              tma_load_3d(sa, &map_a, &bars->full[s], ib * BM, l0, plane_a);
              tma_load_3d(sa + B_BOX_BYTES, &map_a, &bars->full[s], ib * BM + 64, l0, plane_a);
            } else {
              // A = g: K-major [128 rows of m] x [64 n]
              tma_load_3d(sa, &map_a, &bars->full[s], l0, ib * BM, plane_a);
            }
#pragma unroll
            for (int c = 0; c < B_BN / 64; ++c)
              tma_load_3d(sb + c * B_BOX_BYTES, &map_b, &bars->full[s], j0 + c * 64, l0, plane_b);
          }
        }
      }
      const uint32_t n_back = it < (uint32_t)B_STAGES ? it : (uint32_t)B_STAGES;
      for (uint32_t j = it - n_back; j < it; ++j) {
        const int s = j % B_STAGES;
        const uint32_t ph = (j / B_STAGES) & 1u;
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try(&bars->full[s], ph)) {
          if (globaltimer_ns() - t0 > wait_limit_ns()) {
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
        // plane products: the leading product accumulates in buffer 0 and the (much smaller) cross terms
        // in buffer 1 -- the tensor core truncates when it adds into an accumulator, and the truncation is
        // relative to the accumulator's size -- so an item holds both buffers and there is no overlap
        const int b = split_acc ? 0 : (int)(acc_it & 1u);
        const uint32_t aph = split_acc ? (acc_it & 1u) : ((acc_it >> 1) & 1u);
        if (!mbar_wait(&bars->acc_empty[b], aph ^ 1u, abort_flag)) {
          raise_error(kErrMma, abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        const int sp = w / per_split;
        const int nls = min((sp + 1) * p.split_lsteps, p.lsteps) - sp * p.split_lsteps;  // this copy's l-steps
        const int steps = nls * p.products;  // every plane product runs over the whole range
        for (int ls = 0; ls < steps; ++ls, ++it) {
          const bool cross = split_acc && ls >= nls;
          const uint32_t d_tmem = tmem_base + (uint32_t)((cross ? 1 : b) * B_BN);
          const bool first = ls == 0 || (split_acc && ls == nls);
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
            umma_bf16(d_tmem, da + a_step * k4, db + b_step * k4, idesc, (first && k4 == 0) ? 0u : 1u);
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[b]);
      }
      umma_commit(&bars->mma_done);
      uint64_t t0 = globaltimer_ns();
      while (!mbar_try(&bars->mma_done, 0)) {
        if (globaltimer_ns() - t0 > wait_limit_ns()) {
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
      const int sp = w / per_split, blk = w - sp * per_split;
      const int ib = blk / (p.T * p.num_jb);
      const int rem = blk % (p.T * p.num_jb);
      const int t = rem / p.num_jb, jb = rem % p.num_jb;
      const int j0 = t * p.tile_w + jb * B_BN;
      const int j_end = min((t + 1) * p.tile_w, p.K);
      const int i = ib * BM + quad * 32 + lane;
      void* const c_dst = p.splits > 1 ? static_cast<void*>(p.partial + (int64_t)sp * p.I * p.K) : p.c_out;
      const bool c_f32 = p.splits > 1 || p.f32_out != 0;
      const int b = split_acc ? 0 : (int)(acc_it & 1u);
      const uint32_t aph = split_acc ? (acc_it & 1u) : ((acc_it >> 1) & 1u);
      if (!mbar_wait(&bars->acc_full[b], aph, abort_flag)) {
        if (lane == 0) raise_error(kErrEpilogue, abort_flag);
        ok = false;
        break;
      }
      tc_fence_after();
      const float c_scale = p.c_scale_ir != nullptr ? quant_step<kF32>(p.c_scale_ir[t], p.inp_res) : 1.0f;
#pragma unroll 1
      for (int c = 0; c < B_BN / 32; ++c) {
        const int jc = j0 + c * 32;
        if (jc >= j_end) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_base + (uint32_t)(b * B_BN + c * 32), r);
        tmem_wait_ld();
        if (split_acc) add_cross_terms(tmem_base + lane_base + (uint32_t)(B_BN + c * 32), r);
        if (i < p.I) store_c_row(c_dst, c_f32, p.K, i, jc, j_end, r, c_scale);
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
  return mbar_wait(bar, parity, abort_flag);
}

// Work list of the pair kernel.  Pair p takes items p, p + n_pairs, ...  When the blocks do not fill the last round
// (rem = num_work mod n_pairs pairs busy, the others idle for a whole block) and 2 rem <= n_pairs, the last rem blocks
// are cut into two halves of 128 columns each, so that the last round keeps 2 rem pairs busy for a shorter time:
// items [0, n_full) are whole blocks, items [n_full, total) half blocks.  A half block still reads the whole A tile
// per k-step, so it takes about three quarters of a block, not half: the cut is made only where the last round is
// a large share of the launch (at most kSplitTailRounds full rounds before it).  Every role of the kernel walks
// the same list.
constexpr int kSplitTailRounds = 3;
struct PairWork {
  int n_full, total;
};
__host__ __device__ __forceinline__ PairWork pair_work_list(int num_work, int n_pairs, bool allow_halves = true) {
  const int rem = num_work % n_pairs;
  PairWork pw;
  pw.n_full = (allow_halves && rem > 0 && 2 * rem <= n_pairs && num_work / n_pairs <= kSplitTailRounds) ? num_work - rem
                                                                                                        : num_work;
  pw.total = pw.n_full + 2 * (num_work - pw.n_full);
  return pw;
}
// item v -> block index; *half = -1 for a whole block, else which 128-column half of it
__host__ __device__ __forceinline__ int pair_item(const PairWork& pw, int v, int* half) {
  if (v < pw.n_full) {
    *half = -1;
    return v;
  }
  const int h = v - pw.n_full;
  *half = h & 1;
  return pw.n_full + (h >> 1);
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
  const bool split_acc = p.products > 1;  // see bwd_tc_kernel
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int num_work = p.num_ib * p.T * p.num_jb;  // num_ib counts 256-row blocks here
  // half blocks only for plain bf16 operands: with the plane products of an fp32 layer (two accumulators per block)
  // the cut has not been measured, so those launches keep whole blocks
  const PairWork pw = pair_work_list(num_work, n_pairs, p.products == 1);
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
      for (int v = pair; v < pw.total && ok; v += n_pairs) {
        int half;
        const int w = pair_item(pw, v, &half);
        const int ib = w / (p.T * p.num_jb);
        const int rem = w % (p.T * p.num_jb);
        const int t = rem / p.num_jb, jb = rem % p.num_jb;
        const int i0 = ib * (2 * BM) + row_off;
        // this CTA's columns of B: 128 of the block's 256, or 64 of the half block's 128
        const int b_boxes = half >= 0 ? P_BN_CTA / 128 : P_BN_CTA / 64;
        const int j0 = t * p.tile_w + jb * P_BN + (half > 0 ? P_BN / 2 : 0) + (int)rank * b_boxes * 64;
        const uint32_t stage_bytes = (uint32_t)(P_A_BYTES + b_boxes * B_BOX_BYTES);
        for (int q = 0; q < p.products && ok; ++q) {
          const int plane_a = p.pa[q] + t * p.a_planes_per_tile, plane_b = p.pb[q];
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
              mbar_expect_tx(&bars->full[s], stage_bytes);
              bar = smem_u32(&bars->full[s]);
            } else {
              if (leader) mbar_expect_tx(&bars->full[s], 2 * stage_bytes);
              bar = mapa_u32(smem_u32(&bars->full[s]), 0);
            }
            if (WGRAD) {
              tma_load_3d_pair(sa, &map_a, bar, i0, l0, plane_a);
              tma_load_3d_pair(sa + B_BOX_BYTES, &map_a, bar, i0 + 64, l0, plane_a);
            } else {
              tma_load_3d_pair(sa, &map_a, bar, l0, i0, plane_a);
            }
            for (int c = 0; c < b_boxes; ++c)
              tma_load_3d_pair(sb + c * B_BOX_BYTES, &map_b, bar, j0 + c * 64, l0, plane_b);
          }
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
            if (globaltimer_ns() - t0 > wait_limit_ns()) {
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
      constexpr uint32_t idesc_block = make_idesc(2 * BM, P_BN, WGRAD ? 1 : 0, 1);
      constexpr uint32_t idesc_half = make_idesc(2 * BM, P_BN / 2, WGRAD ? 1 : 0, 1);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int v = pair; v < pw.total && ok; v += n_pairs, ++acc_it) {
        const uint32_t idesc = v < pw.n_full ? idesc_block : idesc_half;
        const int b = split_acc ? 0 : (int)(acc_it & 1u);
        const uint32_t aph = split_acc ? (acc_it & 1u) : ((acc_it >> 1) & 1u);
        if (!mbar_wait_cluster(&bars->acc_empty[b], aph ^ 1u, abort_flag)) {
          raise_error(kErrMma, abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        const int steps = p.lsteps * p.products;
        for (int ls = 0; ls < steps; ++ls, ++it) {
          const bool cross = split_acc && ls >= p.lsteps;
          const uint32_t d_tmem = tmem_base + (uint32_t)((cross ? 1 : b) * P_BN);
          const bool first = ls == 0 || (split_acc && ls == p.lsteps);
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
            umma_bf16_pair(d_tmem, da + a_step * k4, db + b_step * k4, idesc, (first && k4 == 0) ? 0u : 1u);
          umma_commit_pair(&bars->empty[s], 3);  // frees the stage in both CTAs
        }
        if (ok) umma_commit_pair(&bars->acc_full[b], 3);
      }
      umma_commit_pair(&bars->mma_done, 1);
      uint64_t t0 = globaltimer_ns();
      while (!mbar_try_cluster(&bars->mma_done, 0)) {
        if (globaltimer_ns() - t0 > wait_limit_ns()) {
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
    for (int v = pair; v < pw.total && ok; v += n_pairs, ++acc_it) {
      int half;
      const int w = pair_item(pw, v, &half);
      const int ib = w / (p.T * p.num_jb);
      const int rem = w % (p.T * p.num_jb);
      const int t = rem / p.num_jb, jb = rem % p.num_jb;
      const int j0 = t * p.tile_w + jb * P_BN + (half > 0 ? P_BN / 2 : 0);
      const int n_chunks = half >= 0 ? P_BN / 64 : P_BN / 32;  // chunks of 32 accumulator columns
      const int j_end = min((t + 1) * p.tile_w, p.K);
      const int i = ib * (2 * BM) + row_off + quad * 32 + lane;
      void* const c_dst = p.c_out;
      const bool c_f32 = p.f32_out != 0;
      const int b = split_acc ? 0 : (int)(acc_it & 1u);
      const uint32_t aph = split_acc ? (acc_it & 1u) : ((acc_it >> 1) & 1u);
      if (!mbar_wait_cluster(&bars->acc_full[b], aph, abort_flag)) {
        if (lane == 0) raise_error(kErrEpilogue, abort_flag);
        ok = false;
        break;
      }
      tc_fence_after();
      const float c_scale = p.c_scale_ir != nullptr ? quant_step<kF32>(p.c_scale_ir[t], p.inp_res) : 1.0f;
#pragma unroll 1
      for (int c = 0; c < n_chunks; ++c) {
        const int jc = j0 + c * 32;
        if (jc >= j_end) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_base + (uint32_t)(b * P_BN + c * 32), r);
        tmem_wait_ld();
        if (split_acc) add_cross_terms(tmem_base + lane_base + (uint32_t)(P_BN + c * 32), r);
        if (i < p.I) store_c_row(c_dst, c_f32, p.K, i, jc, j_end, r, c_scale);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bars->acc_empty[b]), 0));
    }
  } else if (warp >= 8 && masked && pair < pw.total) {
    // ---- mask transform (both CTAs, own A tile): see bwd_tc_kernel -------------------------
    const int grp = (warp - 8) >> 2;
    const int r = threadIdx.x - (8 + 4 * grp) * 32;  // 0..127
    const int row_in_box = WGRAD ? (r & 63) : r;
    const int box = WGRAD ? (r >> 6) : 0;
    const int total = ((pw.total - pair + n_pairs - 1) / n_pairs) * p.lsteps;
    const int m_last = p.M - 1, w_last = p.mask_words - 1;
    int f_w = pair + (grp / p.lsteps) * n_pairs, f_ls = grp % p.lsteps;  // f_w: item of the work list
    const uint32_t* f_lo = p.keep_mask;
    const uint32_t* f_hi = p.keep_mask;
    auto seek_item = [&]() {
      if (f_w >= pw.total) return;
      int half;
      const int blk = pair_item(pw, f_w, &half);  // a half block has the A tile of its block
      const int ib = blk / (p.T * p.num_jb);
      const int t = (blk % (p.T * p.num_jb)) / p.num_jb;
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

}  // namespace

bool tc_backward_supported(const AlDesc& d, const TileTable& tt) { return tc_shape_ok(d, tt); }

// The pair kernel's work list on the host (the same two functions the kernel calls), for the tests.
void tc_pair_work_item(int num_work, int n_pairs, int item, int* total, int* block, int* half) {
  const PairWork pw = pair_work_list(num_work, n_pairs);
  *total = pw.total;
  *block = -1;
  *half = -1;
  if (item >= 0 && item < pw.total) *block = pair_item(pw, item, half);
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
// Plane layout of the operands of an fp32 layer (see BwdTcParams); all-zero = bf16 operands.
struct PlaneSpec {
  int products = 1;
  uint8_t pa[8] = {0}, pb[8] = {0};
  int a_planes = 1;           // planes in the A tensor (all tiles)
  int b_planes = 1;
  int a_planes_per_tile = 0;
  int f32_out = 0;
  const float* c_scale_ir = nullptr;
  float inp_res = 0.0f;
  // weight gradient whose output has few blocks: the reduction over the batch rows is split over `splits`
  // CTAs per block (fp32 copies in `partial`, added by a second kernel); see BwdTcParams
  int splits = 1;
  float* partial = nullptr;
};

static int launch_bwd_tc(bool wgrad, const void* g, const void* b_op, const uint32_t* keep_mask,
                         int mask_words, int M, int K, int N, const TileTable& tt, int pairing, void* c_out,
                         cudaStream_t s, const PlaneSpec& spec = PlaneSpec()) {
  int w = 0;
  if (!uniform_tiles(tt, &w) || !aligned16(g) || !aligned16(b_op) || !aligned16(c_out)) {
    set_error("bwd_tc: operands must be 16-byte aligned with equally wide tiles");
    return AL_ERR_UNSUPPORTED;
  }
  if (spec.products > 1 && keep_mask != nullptr) {
    set_error("bwd_tc: plane products take their clamp mask folded into the A planes");
    return AL_ERR_BAD_ARGUMENT;
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
  p.products = spec.products;
  for (int q = 0; q < 8; ++q) {
    p.pa[q] = spec.pa[q];
    p.pb[q] = spec.pb[q];
  }
  p.a_planes_per_tile = spec.a_planes_per_tile;
  p.f32_out = spec.f32_out;
  p.c_scale_ir = spec.c_scale_ir;
  p.inp_res = spec.inp_res;
  p.splits = 1;
  p.split_lsteps = p.lsteps;
  p.partial = nullptr;
  if (spec.splits > 1) {
    if (!wgrad || keep_mask != nullptr || spec.partial == nullptr) {
      set_error("bwd_tc: a split reduction is for the weight gradient without a clamp mask and needs a partial-sum buffer");
      return AL_ERR_BAD_ARGUMENT;
    }
    p.split_lsteps = (p.lsteps + spec.splits - 1) / spec.splits;
    p.splits = (p.lsteps + p.split_lsteps - 1) / p.split_lsteps;  // no empty copy
    p.partial = spec.partial;
  }
  int rc = wgrad ? ensure_smem(bwd_tc_kernel<true>, B_SMEM) : ensure_smem(bwd_tc_kernel<false>, B_SMEM);
  if (rc) return rc;
  CUtensorMap map_a, map_b;
  {
    // g [planes][M,N]: dims innermost first {N, M, planes}
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)spec.a_planes};
    uint64_t strides[2] = {(uint64_t)N * 2, (uint64_t)M * N * 2};
    uint32_t box_k[3] = {BK, BM, 1};   // dgrad: 64 n (reduction) x 128 m
    uint32_t box_mn[3] = {64, BK, 1};  // wgrad: 64 n (MMA-M) x 64 m (reduction)
    rc = make_map(&map_a, g, 3, dims, strides, wgrad ? box_mn : box_k);
    if (rc) return rc;
  }
  {
    // B operand [planes][L, K] row-major (w_mod [N,K] for dgrad, xq [M,K] for wgrad): {K, L, planes}
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)p.L, (uint64_t)spec.b_planes};
    uint64_t strides[2] = {(uint64_t)K * 2, (uint64_t)p.L * K * 2};
    uint32_t box[3] = {64, BK, 1};
    rc = make_map(&map_b, b_op, 3, dims, strides, box);
    if (rc) return rc;
  }
  // CTA pairs (256-row blocks) when they fill the machine; single CTAs for smaller problems
  const int pair_work = ((p.I + 2 * BM - 1) / (2 * BM)) * p.T * p.num_jb;
  int pairs = max_pairs(wgrad);
  const int keep_free = comm_reserved_sms();
  if (pairs > 1 && keep_free > 0) pairs = pairs - (keep_free + 1) / 2 > 1 ? pairs - (keep_free + 1) / 2 : 1;
  if (p.splits == 1 && pairs > 0 && pairing >= 0 && (pair_work >= pairs || pairing > 0)) {
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
  int work = p.num_ib * p.T * p.num_jb * p.splits;
  const int sms = sm_count() - keep_free > 1 ? sm_count() - keep_free : 1;
  int grid = work < sms ? work : sms;
  if (wgrad)
    bwd_tc_kernel<true><<<grid, kBwdThreads, B_SMEM, s>>>(map_a, map_b, p);
  else
    bwd_tc_kernel<false><<<grid, kBwdThreads, B_SMEM, s>>>(map_a, map_b, p);
  rc = check_launch(wgrad ? "wgrad_tc" : "dgrad_tc");
  if (rc || p.splits == 1) return rc;
  return launch_sum_partials(spec.f32_out ? AL_F32 : AL_BF16, p.partial, p.splits, (int64_t)p.I * K, c_out, s);
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

// fp32 layers.  g_planes: [sets][kPlanes][M][N] bf16 planes of the (masked) upstream gradient, sets = T
// when they were prepared per analog tile and 1 otherwise; w_planes [kPlanes][N][K]; codes16 [M,K] bf16 codes.
int launch_dgrad_tc_f32(const void* g_planes, int sets, const void* w_planes, int M, int K, int N, const TileTable& tt,
                        int pairing, void* grad_x, cudaStream_t s) {
  ProfScope prof(AL_K_DGRAD_GEMM, s);
  PlaneSpec spec;
  // Both operands are fp32 here.  The products of the two leading planes of each -- g0 w0, g0 w1, g1 w0 --
  // leave a relative error of about 3e-6 (what the third planes and g1 w1 would add is below 2^-17 of the
  // result), inside the 1e-5 bar of fp32 layers at half the work of the six products down to 2^-16.
  spec.products = 3;
  const uint8_t pa[3] = {0, 0, 1}, pb[3] = {0, 1, 0};
  for (int q = 0; q < 3; ++q) {
    spec.pa[q] = pa[q];
    spec.pb[q] = pb[q];
  }
  static_assert(kPlanes >= 2, "the three products below read two planes of each operand");
  spec.a_planes = kPlanes * sets;
  spec.b_planes = kPlanes;
  spec.a_planes_per_tile = sets > 1 ? kPlanes : 0;
  spec.f32_out = 1;
  TileTable one;
  one.T = 1;
  one.ends[0] = K;
  return launch_bwd_tc(false, g_planes, w_planes, nullptr, 0, M, K, N, sets > 1 ? tt : one, pairing, grad_x, s, spec);
}

// scale_ir: [T] static input ranges whose DAC step multiplies the tile's columns of grad_w (null when
// the step is already folded into per-tile planes)
int launch_wgrad_tc_f32(const void* g_planes, int sets, const void* codes16, int M, int K, int N, const TileTable& tt,
                        const float* scale_ir, float inp_res, int pairing, void* grad_w, cudaStream_t s, int splits,
                        float* partial) {
  ProfScope prof(AL_K_WGRAD_GEMM, s);
  PlaneSpec spec;
  spec.products = kPlanes;  // the codes are exact in one plane
  for (int q = 0; q < kPlanes; ++q) {
    spec.pa[q] = (uint8_t)q;
    spec.pb[q] = 0;
  }
  spec.a_planes = kPlanes * sets;
  spec.b_planes = 1;
  spec.a_planes_per_tile = sets > 1 ? kPlanes : 0;
  spec.f32_out = 1;
  spec.c_scale_ir = scale_ir;
  spec.inp_res = inp_res;
  spec.splits = splits;
  spec.partial = partial;
  return launch_bwd_tc(true, g_planes, codes16, nullptr, 0, M, K, N, tt, pairing, grad_w, s, spec);
}

int tc_set_wait_limit(unsigned long long ns) {
  cudaError_t e = set_wait_limit(ns);
  if (e == cudaSuccess) e = tc_fwd_set_wait_limit(ns);
  if (e != cudaSuccess) {
    set_error("al_set_device_wait_limit_ns: %s", cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  return AL_OK;
}

int tc_read_device_error(cudaStream_t s, uint32_t* code) {
  cudaError_t e = cudaStreamSynchronize(s);
  uint32_t fwd_code = 0;
  *code = 0;
  if (e == cudaSuccess) e = take_error_word(code);
  if (e == cudaSuccess) e = tc_fwd_take_error_word(&fwd_code);
  if (e != cudaSuccess) {
    set_error("al_read_device_error: %s", cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  *code |= fwd_code;
  if (*code != 0) {
    set_error("a device-side wait of the tcgen05 kernels gave up (role mask 0x%x)", *code);
    return AL_ERR_DEVICE_TIMEOUT;
  }
  return AL_OK;
}

}  // namespace al
