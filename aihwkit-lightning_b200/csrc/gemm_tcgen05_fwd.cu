// Forward GEMM of the analog linear path on the Blackwell tensor cores (sm_100a):
//   out[m,n] = sum_t stage_t( xq[m, tile t] . w_mod[n, tile t] ) + bias[n]
// Operands are brought into shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle),
// multiplied by tcgen05.mma with fp32 accumulators in tensor memory (TMEM) and drained by
// tcgen05.ld.  One persistent, warp-specialised kernel: the K loop is cut at the analog-tile
// boundaries; each analog tile accumulates into one of two TMEM accumulators, and while the
// tensor core works on tile t+1 sixteen epilogue warps run tile t's output stage (rounding,
// output noise, ADC quantisation, clamp, clamp-mask bits) and add it to a running sum.  Large
// problems run on CTA pairs (256 x 256 blocks, cta_group::2), small ones on single CTAs
// (128 x 128 blocks).
#include "tcgen05_common.cuh"

namespace al {

namespace {

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
struct FwdTcParams {
  int32_t small_adc_codes;  // |ADC code| provably below 2^38: unguarded add-based rint is exact
  int32_t tile_w;      // width of every analog tile (all equal on this path)
  int32_t ksteps;      // ceil(tile_w / 64)
  int32_t num_mb, num_nb;
  int32_t planes_b;    // bf16 planes of the weights (kPlanes for an fp32 layer, else 1): accumulated per analog tile
  float inp_res;       // fp32 layers: the A operand holds integer DAC codes, the accumulator is scaled by the DAC step
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
//
// IO: element type of the layer's tensors (input ranges, bias, replayed noise, per-channel scales,
// outputs).  IO = fp32: the A operand holds the DAC codes as bf16 integers and the weights come as
// bf16 planes (fourth dimension of their tensor map) that are accumulated one after the other;
// the output stage multiplies the accumulator by the DAC step of its (row, tile) first.
template <int RD, int MODE, bool PAIR, int IO = kBF16>
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
          const int steps = p.ksteps * p.planes_b;
          for (int st = 0; st < steps; ++st, ++it) {
            const int ks = st % p.ksteps, plane = st / p.ksteps;
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
              if (IO == kF32) tma_load_4d(sa + F_A_BYTES, &map_b, &bars->full[s], ks * BK, t, nb * F_BN, plane);
              else tma_load_3d(sa + F_A_BYTES, &map_b, &bars->full[s], ks * BK, t, nb * F_BN);
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
            if (globaltimer_ns() - t0 > wait_limit_ns()) {
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
      const bool withhold = *(volatile uint32_t*)&g_tc_withhold_acc_signal != 0u;  // test aid, see its declaration
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
          const int steps = p.ksteps * p.planes_b;
          for (int ks = 0; ks < steps; ++ks, ++it) {
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
          if (ok && !withhold) {
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
        if (globaltimer_ns() - t0 > wait_limit_ns()) {
          raise_error(kErrDrain, abort_flag);
          break;
        }
      }
    }
  } else if (warp >= 4) {
    // ---- epilogue: per-tile output stage and running sum ----------------------------------
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
    const NoiseCounter noise_ctr = noise_counter(p.noise);
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
          if (ep.ir_mode == AL_IR_DYNAMIC) ir = Elem<IO>::load(ep.ir_rows, (int64_t)t * M + m);
          else if (ep.ir_mode == AL_IR_STATIC) ir = Elem<IO>::load(ep.ir_rows, t);
        }
        const float t_max = ep.w_tile_max ? ep.w_tile_max[t] : 0.0f;
        // fp32 layers: accumulator = sum of code * weight; the DAC step turns it into the tile's product
        const float dac_step = IO == kF32 ? quant_step<kF32>(ir, p.inp_res) : 1.0f;
        float sc = rnd<RD>(fmul(t_max, rnd<RD>(fmul(ep.noise_coef, ir))));
        bool noise_now = has_noise;
        if (kMergedNoise) {
          noise_var = t == 0 ? sc * sc : fmaf(sc, sc, noise_var);
          noise_now = t == T - 1;
        } else {
          noise_var = sc * sc;
        }
        // fixed modes: the scale of the noise goes under the generator's square root
        const float noise_neg_c = kNegTwoLn2 * noise_var;
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
        // fixed modes: ADC in packed bf16 arithmetic (stepc and its reciprocal are bf16 values or round to them)
        const __nv_bfloat162 y2 = __float2bfloat162_rn(rstep), nstepc2b = __float2bfloat162_rn(-stepc);
        // this thread's row of the shared-memory running sum (PAIR): chunk c of 8 columns sits at
        // 16 * (c ^ (row & 7)), so the eight rows a quarter-warp reads hit distinct banks
        const int srow = quad * 32 + lane;
        const uint32_t sum_row = smem_u32(sum_base) + (uint32_t)srow * (uint32_t)(kBN * 2);
        // word (t, first column of this warp / 32, row m) of the clamp mask; the next word of the row is M further
        uint32_t* const mask_p = ep.keep_mask != nullptr
                                     ? ep.keep_mask + ((int64_t)t * ep.mask_words + (n_first >> 5)) * M + (row_ok ? m : 0)
                                     : nullptr;
        // the compile-time output stages unroll the walk over this warp's columns: every offset below
        // becomes an immediate
        constexpr int kUnrollH = kFixed ? kCols / 16 : 1;
#pragma unroll kUnrollH
        for (int h = 0; h < kCols / 16; ++h) {
          const int cc = col0 + h * 16;
          const int nh = n_first + h * 16;
          const int n0 = n_first + (h >> 1) * 32;  // the 32 columns whose mask word this half belongs to
          // layers with few output channels: column groups beyond the last channel hold nothing (uniform
          // across the warp; a group is skipped as a whole, so that its mask word keeps its one writer)
          if (!kFixed && n0 >= N) break;
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
          if (IO == kF32) {
#pragma unroll
            for (int j = 0; j < 16; ++j) accr[j] = __float_as_uint(fmul(__uint_as_float(accr[j]), dac_step));
          }
          if constexpr (kFixed) {
            // ---- output stage fixed at compile time: everything in packed bf16 arithmetic --------
            if (t == 0) {
#pragma unroll
              for (int pr = 0; pr < 8; ++pr) sumr[pr] = 0u;  // +0.0 in both halves
            }
            uint32_t kept = 0;  // bit 2*pr (low half) and bit 16 + 2*pr + 1 (high half): element kept
#pragma unroll
            for (int g8 = 0; g8 < 2; ++g8) {
              uint32_t bits[4];
              if (noise_now) {
                const int nq = nh + g8 * 8;
                philox7_keyed(p.noise, noise_ctr, row_group8 + (uint32_t)((nq < N ? nq : 0) >> 3), bits);
              }
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const int pr = g8 * 4 + q4;  // element 2*pr in the low half, 2*pr+1 in the high half
                __nv_bfloat162 o2 = __floats2bfloat162_rn(__uint_as_float(accr[2 * pr]), __uint_as_float(accr[2 * pr + 1]));
                if (noise_now) o2 = box_muller16_fma(bits[q4], noise_neg_c, o2);
                if (has_adc) o2 = adc_bf16x2(o2, y2, nstepc2b, step2);
                if (has_bound) {
                  // kept <=> the clamp leaves the value unchanged (false for NaN, like the reference's
                  // -bound <= o <= bound)
                  const __nv_bfloat162 c2 = __hmin2_nan(__hmax2_nan(o2, nbound2), bound2);
                  kept |= __heq2_mask(c2, o2) & ((1u << (2 * pr)) | (1u << (17 + 2 * pr)));
                  o2 = c2;
                }
                sumr[pr] = as_u32(__hadd2_rn(as_bf162(sumr[pr]), o2));
              }
            }
            if (!has_bound) kept = 0xffffffffu;
            keep_bits |= ((kept | (kept >> 16)) & 0xffffu) << ((h & 1) * 16);
          } else {
          float z[16];
          if (noise_now) {
#pragma unroll
            for (int g8 = 0; g8 < 2; ++g8) {
              const int nq = nh + g8 * 8;
              if (replay) {
                const uint64_t idx = ((uint64_t)t * M + (row_ok ? m : 0)) * N + (nq < N ? nq : 0);
                if (IO == kF32) {
                  const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ep.out_noise) + idx);
                  const float4 lo4 = src[0], hi4 = src[1];
                  z[g8 * 8 + 0] = lo4.x; z[g8 * 8 + 1] = lo4.y; z[g8 * 8 + 2] = lo4.z; z[g8 * 8 + 3] = lo4.w;
                  z[g8 * 8 + 4] = hi4.x; z[g8 * 8 + 5] = hi4.y; z[g8 * 8 + 6] = hi4.z; z[g8 * 8 + 7] = hi4.w;
                } else {
                  const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(ep.out_noise) + idx);
                  const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    z[g8 * 8 + 2 * q] = __uint_as_float(rw[q] << 16);
                    z[g8 * 8 + 2 * q + 1] = __uint_as_float(rw[q] & 0xffff0000u);
                  }
                }
              } else {
                normal8_keyed(p.noise, noise_ctr, row_group8 + (uint32_t)((nq < N ? nq : 0) >> 3), &z[g8 * 8]);
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
              const float cmax = n < N ? Elem<IO>::load(ep.w_amax, (int64_t)t * N + n) : 0.0f;
              bool keep;
              const float o = tile_epilogue<RD>(__uint_as_float(accr[j]), ir, ep.noise_pc ? cmax : t_max,
                                                ep.bound_pc ? cmax : t_max, has_noise ? rnd<RD>(z[j]) : 0.0f,
                                                cfg, &keep);
              sumr[j] = __float_as_uint(t == 0 ? fadd(0.0f, o) : rnd<RD>(fadd(__uint_as_float(sumr[j]), o)));
              keep_bits |= (keep ? 1u : 0u) << ((h & 1) * 16 + j);
            }
          }
          }  // !kFixed
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
          } else if (row_ok && IO == kF32) {
            // final (fp32 layer): bias, store 16 floats of this row
            float* dst = reinterpret_cast<float*>(p.out) + (int64_t)m * N + nh;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (nh + v * 4 < N) {
                float f[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  f[e] = __uint_as_float(sumr[v * 4 + e]);
                  if (ep.bias) f[e] = fadd(f[e], Elem<kF32>::load(ep.bias, nh + v * 4 + e));
                }
                *reinterpret_cast<float4*>(dst + v * 4) = make_float4(f[0], f[1], f[2], f[3]);
              }
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
          if ((h & 1) && mask_p != nullptr && row_ok && (n0 >> 5) < ep.mask_words)
            mask_p[(int64_t)(h >> 1) * M] = keep_bits;  // lanes = consecutive rows
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

}  // namespace

bool tc_forward_supported(const AlDesc& d, const TileTable& tt) { return tc_shape_ok(d, tt); }

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

// how many CTA pairs of the forward kernel the device runs at once (0: it cannot)
static int max_fwd_pairs(FwdKernel kernel, int smem) {
  static FwdKernel seen[24];
  static int count[24];
  static int n_seen = 0;
  for (int i = 0; i < n_seen; ++i)
    if (seen[i] == kernel) return count[i];
  int clusters = 0;
  PairLaunch pl(2 * sm_count(), kFwdThreads, smem, nullptr);
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
  p.noise = make_noise_keys(ep.seed, ep.offset, 1u, ep.offset_base);
  p.out = out;
  p.planes_b = 1;
  p.inp_res = 0.0f;
  {
    // |o| <= tile_w * ir * wmax * (1 + noise) and step = 2 * out_bound * ir * wmax / states
    double states = ep.out_res > 1.0f ? ep.out_res : (ep.out_res > 0.0f ? 1.0 / ep.out_res : 1.0);
    double max_code = 8.0 * (double)w * states / (2.0 * (ep.out_bound > 0.0f ? ep.out_bound : 1.0));
    p.small_adc_codes = max_code < 274877906944.0 ? 1 : 0;  // 2^38
  }
  const bool per_channel = ep.w_amax != nullptr && (ep.noise_pc || ep.bound_pc);
  // the compile-time output stages quantise in packed bf16 arithmetic, which needs every ADC code
  // beyond +-127 to end on the clamp (up to 254 states: the 8-bit converter and below)
  const bool fixed = round_dt == AL_BF16 && !per_channel && ep.out_noise == nullptr && !ep.no_rounding &&
                     p.small_adc_codes && (!ep.has_adc || adc_codes_fit_a_byte(ep.out_res, ep.has_bound != 0));
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
  const int pair_smem = FP_SMEM;
  if (pair_ok) {
    kernel = pick_fwd_kernel<true>(mode, round_dt);
    rc = ensure_smem(kernel, pair_smem);
    if (rc) return rc;
    pairs = max_fwd_pairs(kernel, pair_smem);
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
    PairLaunch pl(2 * (pair_tiles < pairs ? pair_tiles : pairs), kFwdThreads, pair_smem, s);
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

// fp32 with the DAC on and integer codes of at most 9 bits (exact in bf16), tiles as for bf16
bool tc_f32_supported(const AlDesc& d, const TileTable& tt) {
  if (d.dtype != AL_F32 || !tc_tiling_ok(d, tt)) return false;
  if (d.ir_mode == AL_IR_OFF || !(d.inp_res > 0) || d.no_rounding) return false;
  const double states = d.inp_res > 1.0 ? d.inp_res : 1.0 / d.inp_res;
  return states <= 510.0;
}

// Forward of an fp32 layer on the tensor cores: A = DAC codes as bf16 [M,K], B = the bf16 planes of the
// modified weights [kPlanes][N][K]; single CTAs (128 x 128 blocks, fp32 running sum in tensor memory), every
// output-stage switch read at run time.
int launch_fwd_tc_f32(const void* codes16, const void* w_planes, int K, const TileTable& tt,
                      const FwdEpilogueParams& ep, float inp_res, void* out, cudaStream_t s) {
  ProfScope prof(AL_K_FWD_GEMM, s);
  int w = 0;
  if (!uniform_tiles(tt, &w) || !aligned16(codes16) || !aligned16(w_planes) || !aligned16(out)) {
    set_error("fwd_tc_f32: operands must be 16-byte aligned with equally wide tiles");
    return AL_ERR_UNSUPPORTED;
  }
  FwdTcParams p;
  p.tile_w = w;
  p.ksteps = (w + BK - 1) / BK;
  p.num_mb = (ep.M + BM - 1) / BM;
  p.num_nb = (ep.N + F_BN - 1) / F_BN;
  p.ep = ep;
  p.noise = make_noise_keys(ep.seed, ep.offset, 1u, ep.offset_base);
  p.out = out;
  p.planes_b = kPlanes;
  p.inp_res = inp_res;
  p.small_adc_codes = 0;  // fp32 accumulators: guarded rint
  auto kernel = fwd_tc_kernel<kF32, -1, false, kF32>;
  int rc = ensure_smem(kernel, F_SMEM);
  if (rc) return rc;
  CUtensorMap map_a, map_b;
  {
    uint64_t dims[3] = {(uint64_t)w, (uint64_t)tt.T, (uint64_t)ep.M};
    uint64_t strides[2] = {(uint64_t)w * 2, (uint64_t)K * 2};
    uint32_t box[3] = {BK, 1, BM};
    rc = make_map(&map_a, codes16, 3, dims, strides, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)w, (uint64_t)tt.T, (uint64_t)ep.N, (uint64_t)kPlanes};
    uint64_t strides[3] = {(uint64_t)w * 2, (uint64_t)K * 2, (uint64_t)ep.N * K * 2};
    uint32_t box[4] = {BK, 1, F_BN, 1};
    rc = make_map(&map_b, w_planes, 4, dims, strides, box);
    if (rc) return rc;
  }
  const int tiles = p.num_mb * p.num_nb;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kernel<<<grid, kFwdThreads, F_SMEM, s>>>(map_a, map_b, p);
  return check_launch("fwd_tc_f32");
}

cudaError_t tc_fwd_take_error_word(uint32_t* code) { return take_error_word(code); }
cudaError_t tc_fwd_set_wait_limit(unsigned long long ns) { return set_wait_limit(ns); }
cudaError_t tc_fwd_set_withhold_acc_signal(uint32_t on) { return set_withhold_acc_signal(on); }

}  // namespace al
