// CUDA-core GEMMs of the analog linear path.  They serve the fp32 layers (whose 1e-5 parity
// bound rules out single-pass tensor-core arithmetic) and every shape the TMA-fed tcgen05
// kernels cannot take (tile boundaries that are not 16-byte aligned).  One output block of 4096
// elements per CTA -- 64x64, or 128x32 / 256x16 (and their transposes) for the layers with few
// output channels that convolutions produce, so that no lane multiplies padding -- 4x4 outputs
// per thread, fp32 accumulation; the forward kernel runs the per-tile output stage (noise, ADC,
// clamp, cross-tile sum) in registers at the end of every analog tile, the backward kernels
// apply the ADC clamp mask of the tile to the gradient operand.  The weight gradient reduces
// over the rows of the batch: when the output has too few blocks to fill the GPU that reduction
// is split over CTAs, each writing a partial sum that a second kernel adds up in a fixed order.
#include "analog_math.cuh"
#include "internal.h"

namespace al {

namespace {

constexpr int BK = 16;
constexpr int kBlockElems = 4096;  // outputs per CTA: 256 threads x (4 x 4)
constexpr int kPad = 4;             // row padding of the staged blocks: rows stay 16-byte aligned
constexpr int kThreads = 256;

// A [ROWS x 16] operand block travels global -> registers (block_fetch) -> shared memory as
// floats, sm[l][i] (block_commit): the fetch of block k+1 is issued before the multiply-adds of
// block k, so that its latency hides behind them.
// L_CONTIG: the reduction index l is the contiguous one in memory, else the block-row index i.
template <int ROWS>
struct BlockRegs {
  static constexpr int kIters = (ROWS * BK + kThreads - 1) / kThreads;            // one element per turn
  static constexpr int kVecIters = (ROWS * BK / 4 + kThreads - 1) / kThreads;    // four elements per turn
  static constexpr int kRegs = kIters > 4 * kVecIters ? kIters : 4 * kVecIters;
  float v[kRegs];
};

// four consecutive elements starting at element idx (idx a multiple of 4, base 16-byte aligned)
template <int DT>
__device__ __forceinline__ void load4(const void* __restrict__ p, int64_t idx, float out[4]) {
  if (DT == kF32) {
    const float4 f = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx);
    out[0] = f.x; out[1] = f.y; out[2] = f.z; out[3] = f.w;
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + idx);
    out[0] = __uint_as_float(u.x << 16); out[1] = __uint_as_float(u.x & 0xffff0000u);
    out[2] = __uint_as_float(u.y << 16); out[3] = __uint_as_float(u.y & 0xffff0000u);
  }
}
template <int DT>
__device__ __forceinline__ void store4(void* __restrict__ p, int64_t idx, const float v[4]) {
  if (DT == kF32) {
    *reinterpret_cast<float4*>(static_cast<float*>(p) + idx) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
    *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p) + idx) =
        make_uint2((uint32_t)f32_to_bf16_bits(v[0]) | ((uint32_t)f32_to_bf16_bits(v[1]) << 16),
                   (uint32_t)f32_to_bf16_bits(v[2]) | ((uint32_t)f32_to_bf16_bits(v[3]) << 16));
  }
}

// VEC: the operand's contiguous dimension can be read four elements at a time (the launcher checked
// the alignment of its base, row stride and tile starts); edges fall back to single elements.
template <int DT, bool L_CONTIG, int ROWS, bool VEC>
__device__ __forceinline__ void block_fetch(const void* __restrict__ p, int64_t stride_i, int64_t stride_l, int i0,
                                            int i_end, int l0, int l_end, int tid, BlockRegs<ROWS>& regs) {
  if (VEC) {
    constexpr int kUnits = ROWS * BK / 4;
#pragma unroll
    for (int r = 0; r < BlockRegs<ROWS>::kVecIters; ++r) {
      const int u = tid + r * kThreads;
      const int i = L_CONTIG ? u / (BK / 4) : (u % (ROWS / 4)) * 4;
      const int l = L_CONTIG ? (u % (BK / 4)) * 4 : u / (ROWS / 4);
      float* v = &regs.v[4 * r];
      v[0] = v[1] = v[2] = v[3] = 0.0f;
      if (kUnits % kThreads != 0 && u >= kUnits) continue;
      if (L_CONTIG) {
        if (i0 + i >= i_end) continue;
        const int64_t base = (int64_t)(i0 + i) * stride_i + (l0 + l);
        if (l0 + l + 3 < l_end) {
          load4<DT>(p, base, v);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (l0 + l + j < l_end) v[j] = Elem<DT>::load(p, base + j);
        }
      } else {
        if (l0 + l >= l_end) continue;
        const int64_t base = (int64_t)(l0 + l) * stride_l + (i0 + i);
        if (i0 + i + 3 < i_end) {
          load4<DT>(p, base, v);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (i0 + i + j < i_end) v[j] = Elem<DT>::load(p, base + j);
        }
      }
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < BlockRegs<ROWS>::kIters; ++r) {
    const int e = tid + r * kThreads;
    const int i = L_CONTIG ? e / BK : e % ROWS;
    const int l = L_CONTIG ? e % BK : e / ROWS;
    float v = 0.0f;
    if ((ROWS * BK % kThreads == 0 || e < ROWS * BK) && i0 + i < i_end && l0 + l < l_end)
      v = Elem<DT>::load(p, (int64_t)(i0 + i) * stride_i + (int64_t)(l0 + l) * stride_l);
    regs.v[r] = v;
  }
}

template <bool L_CONTIG, int ROWS, bool VEC>
__device__ __forceinline__ void block_commit(const BlockRegs<ROWS>& regs, float (*sm)[ROWS + kPad], int tid) {
  if (VEC) {
    constexpr int kUnits = ROWS * BK / 4;
#pragma unroll
    for (int r = 0; r < BlockRegs<ROWS>::kVecIters; ++r) {
      const int u = tid + r * kThreads;
      if (kUnits % kThreads != 0 && u >= kUnits) continue;
      const int i = L_CONTIG ? u / (BK / 4) : (u % (ROWS / 4)) * 4;
      const int l = L_CONTIG ? (u % (BK / 4)) * 4 : u / (ROWS / 4);
      const float* v = &regs.v[4 * r];
      if (L_CONTIG) {
#pragma unroll
        for (int j = 0; j < 4; ++j) sm[l + j][i] = v[j];
      } else {
        *reinterpret_cast<float4*>(&sm[l][i]) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < BlockRegs<ROWS>::kIters; ++r) {
    const int e = tid + r * kThreads;
    const int i = L_CONTIG ? e / BK : e % ROWS;
    const int l = L_CONTIG ? e % BK : e / ROWS;
    if (ROWS * BK % kThreads == 0 || e < ROWS * BK) sm[l][i] = regs.v[r];
  }
}

// thread (ty, tx) owns rows ty*4 .. +3 and columns tx*4 .. +3: one 16-byte shared-memory load
// per operand and reduction step feeds 16 multiply-adds
template <int TBM, int TBN>
__device__ __forceinline__ void mac_block(const float (*As)[TBM + kPad], const float (*Bs)[TBN + kPad],
                                          int ty, int tx, float acc[4][4]) {
#pragma unroll
  for (int l = 0; l < BK; ++l) {
    const float4 av = *reinterpret_cast<const float4*>(&As[l][ty * 4]);
    const float4 bv = *reinterpret_cast<const float4*>(&Bs[l][tx * 4]);
    const float a[4] = {av.x, av.y, av.z, av.w}, b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// out[m, n] = sum_t stage_t( xq[m, tile t] . w_mod[n, tile t] ) + bias[n]
// BN in {16, 32, 64}: a block narrower than 64 is only launched when it covers all of N, so that
// every 32-bit word of the keep mask has one writer.
template <int DT, int RD, int BN, bool VEC>
__global__ void __launch_bounds__(kThreads)
fwd_simt_kernel(const void* __restrict__ xq, const void* __restrict__ w_mod, int K, TileTable tt,
                FwdEpilogueParams ep, void* __restrict__ out, int vec_out) {
  constexpr int BM = kBlockElems / BN, TX = BN / 4;
  __shared__ __align__(16) float As[BK][BM + kPad];
  __shared__ __align__(16) float Bs[BK][BN + kPad];
  const int tid = threadIdx.x, tx = tid % TX, ty = tid / TX, lane = tid & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;  // row blocks on x: no 65535 limit
  const int M = ep.M, N = ep.N;

  TileEpilogueCfg cfg;
  cfg.has_noise = ep.has_noise;
  cfg.has_bound = ep.has_bound;
  cfg.has_adc = ep.has_adc;
  cfg.no_rounding = ep.no_rounding;
  cfg.noise_coef = ep.noise_coef;
  cfg.out_bound = ep.out_bound;
  cfg.out_res = ep.out_res;

  const uint64_t noise_offset = ep.offset + (ep.offset_base != nullptr ? *ep.offset_base : 0ull);
  float sum[4][4] = {};
  for (int t = 0; t < tt.T; ++t) {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    const int lo = tt.lo(t), hi = tt.hi(t);
    BlockRegs<BM> ra;
    BlockRegs<BN> rb;
    block_fetch<DT, true, BM, VEC>(xq, K, 1, m0, M, lo, hi, tid, ra);
    block_fetch<DT, true, BN, VEC>(w_mod, K, 1, n0, N, lo, hi, tid, rb);
    for (int k0 = lo; k0 < hi; k0 += BK) {
      block_commit<true, BM, VEC>(ra, As, tid);
      block_commit<true, BN, VEC>(rb, Bs, tid);
      __syncthreads();
      if (k0 + BK < hi) {
        block_fetch<DT, true, BM, VEC>(xq, K, 1, m0, M, k0 + BK, hi, tid, ra);
        block_fetch<DT, true, BN, VEC>(w_mod, K, 1, n0, N, k0 + BK, hi, tid, rb);
      }
      mac_block<BM, BN>(As, Bs, ty, tx, acc);
      __syncthreads();
    }
    // per-tile output stage
    float t_max = ep.w_tile_max ? rnd<DT>(ep.w_tile_max[t]) : 0.0f;
    float s_col_noise[4], s_col_bound[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      float cmax = (n < N && ep.w_amax && (ep.noise_pc || ep.bound_pc))
                       ? Elem<DT>::load(ep.w_amax, (int64_t)t * N + n)
                       : 0.0f;
      s_col_noise[j] = ep.noise_pc ? cmax : t_max;
      s_col_bound[j] = ep.bound_pc ? cmax : t_max;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int m = m0 + ty * 4 + i;
      float ir = 0.0f;
      if (m < M) {
        if (ep.ir_mode == AL_IR_DYNAMIC) ir = Elem<DT>::load(ep.ir_rows, (int64_t)t * M + m);
        else if (ep.ir_mode == AL_IR_STATIC) ir = Elem<DT>::load(ep.ir_rows, t);
      }
      uint32_t nibble = 0u;
      // the thread's four columns are one group of four of the noise stream when N is a multiple
      // of 4: one generator call instead of four, same values
      const bool quad = ep.has_noise && ep.out_noise == nullptr && (N & 3) == 0 && m < M && n0 + tx * 4 < N;
      float z4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      if (quad) normal4(ep.seed, noise_offset, 1u, (((uint64_t)t * M + m) * N + n0 + tx * 4) >> 2, z4);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int n = n0 + tx * 4 + j;
        bool keep = false;
        if (m < M && n < N) {
          float xi = 0.0f;
          if (quad) {
            xi = rnd<RD>(z4[j]);
          } else if (ep.has_noise) {
            uint64_t idx = ((uint64_t)t * M + m) * N + n;
            xi = ep.out_noise ? Elem<DT>::load(ep.out_noise, (int64_t)idx)
                              : rnd<RD>(normal1(ep.seed, noise_offset, 1u, idx));
          }
          float o = tile_epilogue<RD>(acc[i][j], ir, s_col_noise[j], s_col_bound[j], xi, cfg, &keep);
          sum[i][j] = t == 0 ? fadd(0.0f, o) : rnd<RD>(fadd(sum[i][j], o));
        }
        nibble |= (keep ? 1u : 0u) << j;
        // keeps the sixteen output stages of a thread from being interleaved (registers: 80 instead of 210+)
        __syncwarp();
      }
      if (ep.keep_mask != nullptr) {
        // the kGroup lanes of this row that share a 32-bit mask word OR their nibbles together
        constexpr int kGroup = TX < 8 ? TX : 8;
        const uint32_t gmask = ((1u << kGroup) - 1u) << (lane & ~(kGroup - 1));
        const uint32_t word = __reduce_or_sync(gmask, nibble << (4 * (tx & 7)));
        const int wi = n0 / 32 + (tx >> 3);
        if ((tx & (kGroup - 1)) == 0 && m < M && wi < ep.mask_words)
          ep.keep_mask[((int64_t)t * ep.mask_words + wi) * M + m] = word;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + ty * 4 + i;
    if (m >= M) continue;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      v[j] = sum[i][j];
      if (ep.bias && n < N) v[j] = fadd(rnd<RD>(v[j]), Elem<DT>::load(ep.bias, n));
    }
    if (vec_out && n0 + tx * 4 + 3 < N) {
      store4<DT>(out, (int64_t)m * N + n0 + tx * 4, v);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + tx * 4 + j < N) Elem<DT>::store(out, (int64_t)m * N + n0 + tx * 4 + j, v[j]);
    }
  }
}

// Backward GEMMs.  C[i, lo_t + j] = sum_l A(i,l) * keep_t(i,l) * B(lo_t + j, l), where
//   dgrad: i = m, l = n, A = g [M,N] (l contiguous), B = w_mod (j contiguous), C = grad_x
//   wgrad: i = n, l = m, A = g^T     (i contiguous), B = xq    (j contiguous), C = grad_w
// blockIdx.z = t * splits + s: split s reduces l over [s * chunk, (s + 1) * chunk) and, when
// splits > 1, stores its fp32 partial block to partial[s][i][column] instead of C.
template <int DT, bool WGRAD, int TBM, int TBN, bool VEC>
__global__ void __launch_bounds__(kThreads)
bwd_simt_kernel(const void* __restrict__ g, const void* __restrict__ b_op,
                const uint32_t* __restrict__ keep_mask, int mask_words, int M, int K, int N,
                TileTable tt, int splits, int chunk, float* __restrict__ partial, void* __restrict__ c_out) {
  static_assert(TBM * TBN == kBlockElems, "4x4 outputs per thread");
  constexpr int TX = TBN / 4;
  __shared__ __align__(16) float As[BK][TBM + kPad];
  __shared__ __align__(16) float Bs[BK][TBN + kPad];
  const int tid = threadIdx.x, tx = tid % TX, ty = tid / TX;
  const int t = blockIdx.z / splits, split = blockIdx.z - t * splits;
  const int lo = tt.lo(t), hi = tt.hi(t);
  // the row blocks of C sit on gridDim.x (up to 2^31 - 1 of them), the column blocks on y
  const int j0 = lo + blockIdx.y * TBN;
  if (j0 >= hi) return;
  const int i0 = blockIdx.x * TBM;
  const int I = WGRAD ? N : M;  // rows of C
  const int L = WGRAD ? M : N;  // reduction length
  const int l_begin = split * chunk;
  const int l_end = l_begin + chunk < L ? l_begin + chunk : L;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // threads whose 4x4 outputs all lie outside C (a 256-wide block on a 144-wide tile leaves whole
  // warps without work) skip the multiply-adds; they still help staging the operands
  const bool owns_output = i0 + ty * 4 < I && j0 + tx * 4 < hi;
  BlockRegs<TBM> ra;
  BlockRegs<TBN> rb;
  auto fetch = [&](int l0) {
    if (WGRAD) block_fetch<DT, false, TBM, VEC>(g, 1, N, i0, I, l0, l_end, tid, ra);
    else block_fetch<DT, true, TBM, VEC>(g, N, 1, i0, I, l0, l_end, tid, ra);
    block_fetch<DT, false, TBN, VEC>(b_op, 1, K, j0, hi, l0, l_end, tid, rb);
  };
  if (l_begin < l_end) fetch(l_begin);
  for (int l0 = l_begin; l0 < l_end; l0 += BK) {
    block_commit<!WGRAD, TBM, VEC>(ra, As, tid);
    block_commit<false, TBN, VEC>(rb, Bs, tid);
    __syncthreads();
    if (l0 + BK < l_end) fetch(l0 + BK);
    if (keep_mask != nullptr) {
      // zero the gradient entries the ADC clamp of this tile blocked
      for (int e = tid; e < TBM * BK; e += kThreads) {
        int i = e % TBM, l = e / TBM;
        int gi = i0 + i, gl = l0 + l;
        if (gi < I && gl < l_end) {
          int m = WGRAD ? gl : gi, n = WGRAD ? gi : gl;
          uint32_t word = keep_mask[((int64_t)t * mask_words + (n >> 5)) * M + m];
          if (((word >> (n & 31)) & 1u) == 0u) As[l][i] = 0.0f;
        }
      }
      __syncthreads();
    }
    if (owns_output) mac_block<TBM, TBN>(As, Bs, ty, tx, acc);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gi = i0 + ty * 4 + i;
    if (gi >= I) continue;
    const int gj0 = j0 + tx * 4;
    if (VEC && gj0 + 3 < hi) {
      if (splits > 1) store4<kF32>(partial, ((int64_t)split * I + gi) * K + gj0, acc[i]);
      else store4<DT>(c_out, (int64_t)gi * K + gj0, acc[i]);
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gj = gj0 + j;
      if (gj < hi) {
        if (splits > 1) partial[((int64_t)split * I + gi) * K + gj] = acc[i][j];
        else Elem<DT>::store(c_out, (int64_t)gi * K + gj, acc[i][j]);
      }
    }
  }
}

// c[e] = sum_s partial[s][e] in a fixed order: a block of 32 x 8 threads takes 32 consecutive elements;
// thread (i, g) adds the copies s = g, g + 8, ... of element i in that order, then the eight group sums
// are added in the order of g.  (One thread per element walking all copies took 12 us for 296 copies of
// a 16 x 144 gradient: a chain of 296 dependent loads on nine blocks.)
constexpr int kSumGroups = 8;
template <int DT>
__global__ void __launch_bounds__(32 * kSumGroups)
sum_partials_kernel(const float* __restrict__ partial, int splits, int64_t count, void* __restrict__ c_out) {
  __shared__ float part[kSumGroups][32];
  const int i = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int64_t e = (int64_t)blockIdx.x * 32 + i;
  float v = 0.0f;
  if (e < count)
    for (int s = g; s < splits; s += kSumGroups) v = fadd(v, partial[(int64_t)s * count + e]);
  part[g][i] = v;
  __syncthreads();
  if (g == 0 && e < count) {
    float sum = part[0][i];
#pragma unroll
    for (int k = 1; k < kSumGroups; ++k) sum = fadd(sum, part[k][i]);
    Elem<DT>::store(c_out, e, sum);
  }
}

// Can rows of a [.., K] matrix be read four elements at a time from every tile start?
inline bool vec4_rows(const void* p, int dtype, int K, const TileTable& tt) {
  const uintptr_t align = dtype == AL_F32 ? 16 : 8;
  if (p == nullptr || reinterpret_cast<uintptr_t>(p) % align != 0 || K % 4 != 0) return false;
  for (int t = 0; t < tt.T; ++t)
    if (tt.lo(t) % 4 != 0) return false;
  return true;
}
inline bool vec4_plain(const void* p, int dtype, int cols) {
  const uintptr_t align = dtype == AL_F32 ? 16 : 8;
  return p != nullptr && reinterpret_cast<uintptr_t>(p) % align == 0 && cols % 4 == 0;
}

inline int max_tile_width(const TileTable& tt) {
  int w = 0;
  for (int t = 0; t < tt.T; ++t) w = tt.hi(t) - tt.lo(t) > w ? tt.hi(t) - tt.lo(t) : w;
  return w;
}

template <int BN>
void fwd_simt_launch(int dtype, int round_dt, const void* xq, const void* w_mod, int K, const TileTable& tt,
                     const FwdEpilogueParams& ep, void* out, cudaStream_t s) {
  constexpr int BM = kBlockElems / BN;
  dim3 grid((ep.M + BM - 1) / BM, (ep.N + BN - 1) / BN);
  const int vec_k = vec4_rows(xq, dtype, K, tt) && vec4_rows(w_mod, dtype, K, tt);
  const int vec_out = vec4_plain(out, dtype, ep.N);
#define AL_FWD_SIMT(DT_, RD_)                                                                                   \
  do {                                                                                                           \
    if (vec_k) fwd_simt_kernel<DT_, RD_, BN, true><<<grid, kThreads, 0, s>>>(xq, w_mod, K, tt, ep, out, vec_out); \
    else fwd_simt_kernel<DT_, RD_, BN, false><<<grid, kThreads, 0, s>>>(xq, w_mod, K, tt, ep, out, vec_out);      \
  } while (0)
  if (dtype == AL_F32) AL_FWD_SIMT(kF32, kF32);
  else if (round_dt == AL_BF16) AL_FWD_SIMT(kBF16, kBF16);
  else AL_FWD_SIMT(kBF16, kF32);
#undef AL_FWD_SIMT
}

template <int TBM, int TBN>
void wgrad_simt_launch(int dtype, const void* g, const void* xq, const uint32_t* keep_mask, int mask_words, int M,
                       int K, int N, const TileTable& tt, int splits, int chunk, float* partial, void* grad_w,
                       cudaStream_t s) {
  dim3 grid((N + TBM - 1) / TBM, (max_tile_width(tt) + TBN - 1) / TBN, tt.T * splits);
  // vec_k: rows of xq and of grad_w (or its fp32 partials) from every tile start; vec_n: rows of g
  const int vec_k = vec4_rows(xq, dtype, K, tt) && vec4_rows(grad_w, dtype, K, tt) &&
                    (splits == 1 || vec4_rows(partial, AL_F32, K, tt));
  const int vec_n = vec4_plain(g, dtype, N);
#define AL_WGRAD_SIMT(DT_, VEC_)                                                                              \
  bwd_simt_kernel<DT_, true, TBM, TBN, VEC_><<<grid, kThreads, 0, s>>>(g, xq, keep_mask, mask_words, M, K, N, tt, \
                                                                       splits, chunk, partial, grad_w)
  const bool vec = vec_k && vec_n;
  if (dtype == AL_F32) {
    if (vec) AL_WGRAD_SIMT(kF32, true);
    else AL_WGRAD_SIMT(kF32, false);
  } else {
    if (vec) AL_WGRAD_SIMT(kBF16, true);
    else AL_WGRAD_SIMT(kBF16, false);
  }
#undef AL_WGRAD_SIMT
}

// Number of CTAs the reduction over the batch rows is split over: enough to put two waves of
// blocks on a 148-SM part, at least 512 rows each.  A function of the LAYER's sizes alone (T is
// the layer's tile count, whatever tile table the GEMM itself runs with), so that the sizing of
// the partial-sum buffer and the launch cannot disagree.
int wgrad_splits(int M, int K, int N, int T) {
  const int tbm = N <= 16 ? 16 : N <= 32 ? 32 : 64;
  const int tbn = kBlockElems / tbm;
  const int width = (K + T - 1) / T;
  const int64_t blocks = (int64_t)((width + tbn - 1) / tbn) * ((N + tbm - 1) / tbm) * T;
  int64_t want = (296 + blocks - 1) / blocks;
  const int64_t most = (M + 511) / 512;
  if (want > most) want = most;
  return want < 1 ? 1 : (int)want;
}

}  // namespace

int launch_sum_partials(int dtype, const float* partial, int splits, int64_t count, void* c_out, cudaStream_t s) {
  const unsigned blocks = (unsigned)((count + 31) / 32);
  if (dtype == AL_F32) sum_partials_kernel<kF32><<<blocks, 32 * kSumGroups, 0, s>>>(partial, splits, count, c_out);
  else sum_partials_kernel<kBF16><<<blocks, 32 * kSumGroups, 0, s>>>(partial, splits, count, c_out);
  return check_launch("sum_partials");
}

void wgrad_simt_plan(int M, int K, int N, int layer_T, int* splits, int* chunk_rows) {
  const int s = wgrad_splits(M, K, N, layer_T);
  const int per = (M + s - 1) / s;
  const int chunk = (per + BK - 1) / BK * BK;
  // rounding the chunk up to whole k-steps can leave trailing splits without rows: drop them
  *splits = (M + chunk - 1) / chunk;
  *chunk_rows = chunk;
}

int64_t wgrad_simt_partial_floats(int M, int K, int N, int layer_T) {
  int splits, chunk;
  wgrad_simt_plan(M, K, N, layer_T, &splits, &chunk);
  return splits > 1 ? (int64_t)splits * N * K : 0;
}

int launch_fwd_simt(int dtype, int round_dt, const void* xq, const void* w_mod, int K,
                    const TileTable& tt, const FwdEpilogueParams& ep, void* out, cudaStream_t s) {
  ProfScope prof(AL_K_FWD_GEMM, s);
  if (ep.N <= 16) fwd_simt_launch<16>(dtype, round_dt, xq, w_mod, K, tt, ep, out, s);
  else if (ep.N <= 32) fwd_simt_launch<32>(dtype, round_dt, xq, w_mod, K, tt, ep, out, s);
  else fwd_simt_launch<64>(dtype, round_dt, xq, w_mod, K, tt, ep, out, s);
  return check_launch("fwd_simt");
}

int launch_dgrad_simt(int dtype, const void* g, const void* w_mod, const uint32_t* keep_mask,
                      int mask_words, int M, int K, int N, const TileTable& tt, void* grad_x,
                      cudaStream_t s) {
  ProfScope prof(AL_K_DGRAD_GEMM, s);
  dim3 grid((M + 63) / 64, (max_tile_width(tt) + 63) / 64, tt.T);
  const int vec_k = vec4_rows(w_mod, dtype, K, tt) && vec4_rows(grad_x, dtype, K, tt);
  const int vec_n = vec4_plain(g, dtype, N);
#define AL_DGRAD_SIMT(DT_, VEC_)                                                                                \
  bwd_simt_kernel<DT_, false, 64, 64, VEC_><<<grid, kThreads, 0, s>>>(g, w_mod, keep_mask, mask_words, M, K, N, tt, 1, \
                                                                      N, nullptr, grad_x)
  const bool vec = vec_k && vec_n;
  if (dtype == AL_F32) {
    if (vec) AL_DGRAD_SIMT(kF32, true);
    else AL_DGRAD_SIMT(kF32, false);
  } else {
    if (vec) AL_DGRAD_SIMT(kBF16, true);
    else AL_DGRAD_SIMT(kBF16, false);
  }
#undef AL_DGRAD_SIMT
  return check_launch("dgrad_simt");
}

int launch_wgrad_simt(int dtype, const void* g, const void* xq, const uint32_t* keep_mask,
                      int mask_words, int M, int K, int N, const TileTable& tt, int layer_T, float* partial,
                      int64_t partial_capacity, void* grad_w, cudaStream_t s) {
  // the split count comes from the layer's tile count -- the argument the caller sized `partial`
  // with -- never from `tt`, which is the one-tile table when there is no clamp mask
  int splits, chunk;
  wgrad_simt_plan(M, K, N, layer_T, &splits, &chunk);
  ProfScope prof(AL_K_WGRAD_GEMM, s, splits > 1 ? 2 : 1);
  if (splits > 1 && (partial == nullptr || (int64_t)splits * N * K > partial_capacity)) {
    set_error("wgrad_simt: the partial-sum buffer holds %lld floats, %d splits x %d x %d need %lld",
              (long long)(partial ? partial_capacity : 0), splits, N, K, (long long)splits * N * K);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (N <= 16) wgrad_simt_launch<16, 256>(dtype, g, xq, keep_mask, mask_words, M, K, N, tt, splits, chunk, partial, grad_w, s);
  else if (N <= 32) wgrad_simt_launch<32, 128>(dtype, g, xq, keep_mask, mask_words, M, K, N, tt, splits, chunk, partial, grad_w, s);
  else wgrad_simt_launch<64, 64>(dtype, g, xq, keep_mask, mask_words, M, K, N, tt, splits, chunk, partial, grad_w, s);
  int rc = check_launch("wgrad_simt");
  if (rc || splits == 1) return rc;
  return launch_sum_partials(dtype, partial, splits, (int64_t)N * K, grad_w, s);
}

}  // namespace al
