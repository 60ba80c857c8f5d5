// CUDA-core GEMMs of the analog linear path.  They serve the fp32 layers (whose 1e-5 parity
// bound rules out single-pass tensor-core arithmetic) and every shape the TMA-fed tcgen05
// kernels cannot take (tile boundaries that are not 16-byte aligned).  One 64x64 output block
// per CTA, 4x4 outputs per thread, fp32 accumulation; the forward kernel runs the per-tile
// output stage (noise, ADC, clamp, cross-tile sum) in registers at the end of every analog
// tile, the backward kernels apply the ADC clamp mask of the tile to the gradient operand.
#include "analog_math.cuh"
#include "internal.h"

namespace al {

namespace {

constexpr int BM = 64, BN = 64, BK = 16;
constexpr int kThreads = 256;

// Stages a [64 x 16] operand block into shared memory as floats, sm[l][i].
// L_CONTIG: the reduction index l is the contiguous one in memory, else the block-row index i.
template <int DT, bool L_CONTIG>
__device__ __forceinline__ void stage_block(const void* __restrict__ p, int64_t stride_i,
                                            int64_t stride_l, int i0, int i_end, int l0, int l_end,
                                            float (*sm)[BM + 1], int tid) {
#pragma unroll
  for (int r = 0; r < (BM * BK) / kThreads; ++r) {
    int i, l;
    if (L_CONTIG) {
      l = tid % BK;
      i = tid / BK + r * (kThreads / BK);
    } else {
      i = tid % BM;
      l = tid / BM + r * (kThreads / BM);
    }
    float v = 0.0f;
    if (i0 + i < i_end && l0 + l < l_end)
      v = Elem<DT>::load(p, (int64_t)(i0 + i) * stride_i + (int64_t)(l0 + l) * stride_l);
    sm[l][i] = v;
  }
}

__device__ __forceinline__ void mac_block(const float (*As)[BM + 1], const float (*Bs)[BN + 1],
                                          int ty, int tx, float acc[4][4]) {
#pragma unroll
  for (int l = 0; l < BK; ++l) {
    float a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = As[l][ty * 4 + i];
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = Bs[l][tx + 16 * j];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// out[m, n] = sum_t stage_t( xq[m, tile t] . w_mod[n, tile t] ) + bias[n]
template <int DT, int RD>
__global__ void __launch_bounds__(kThreads)
fwd_simt_kernel(const void* __restrict__ xq, const void* __restrict__ w_mod, int K, TileTable tt,
                FwdEpilogueParams ep, void* __restrict__ out) {
  __shared__ float As[BK][BM + 1];
  __shared__ float Bs[BK][BN + 1];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16, lane = tid & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int M = ep.M, N = ep.N;

  TileEpilogueCfg cfg;
  cfg.has_noise = ep.has_noise;
  cfg.has_bound = ep.has_bound;
  cfg.has_adc = ep.has_adc;
  cfg.no_rounding = ep.no_rounding;
  cfg.noise_coef = ep.noise_coef;
  cfg.out_bound = ep.out_bound;
  cfg.out_res = ep.out_res;

  float sum[4][4] = {};
  for (int t = 0; t < tt.T; ++t) {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    const int lo = tt.lo(t), hi = tt.hi(t);
    for (int k0 = lo; k0 < hi; k0 += BK) {
      stage_block<DT, true>(xq, K, 1, m0, M, k0, hi, As, tid);
      stage_block<DT, true>(w_mod, K, 1, n0, N, k0, hi, Bs, tid);
      __syncthreads();
      mac_block(As, Bs, ty, tx, acc);
      __syncthreads();
    }
    // per-tile output stage
    float t_max = ep.w_tile_max ? rnd<DT>(ep.w_tile_max[t]) : 0.0f;
    float s_col_noise[4], s_col_bound[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx + 16 * j;
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
      uint32_t bal[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int n = n0 + tx + 16 * j;
        bool keep = false;
        if (m < M && n < N) {
          float xi = 0.0f;
          if (ep.has_noise) {
            uint64_t idx = ((uint64_t)t * M + m) * N + n;
            xi = ep.out_noise ? Elem<DT>::load(ep.out_noise, (int64_t)idx)
                              : rnd<RD>(normal1(ep.seed, ep.offset, 1u, idx));
          }
          float o = tile_epilogue<RD>(acc[i][j], ir, s_col_noise[j], s_col_bound[j], xi, cfg, &keep);
          sum[i][j] = t == 0 ? fadd(0.0f, o) : rnd<RD>(fadd(sum[i][j], o));
        }
        bal[j] = __ballot_sync(0xffffffffu, keep);
      }
      if (ep.keep_mask != nullptr && (lane == 0 || lane == 16) && m < M) {
        int sh = lane == 0 ? 0 : 16;
        uint32_t w0 = ((bal[0] >> sh) & 0xffffu) | (((bal[1] >> sh) & 0xffffu) << 16);
        uint32_t w1 = ((bal[2] >> sh) & 0xffffu) | (((bal[3] >> sh) & 0xffffu) << 16);
        int64_t base = ((int64_t)t * ep.mask_words + n0 / 32) * M + m;
        if (n0 / 32 < ep.mask_words) ep.keep_mask[base] = w0;
        if (n0 / 32 + 1 < ep.mask_words) ep.keep_mask[base + M] = w1;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + ty * 4 + i;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx + 16 * j;
      if (m < M && n < N) {
        float v = sum[i][j];
        if (ep.bias) v = fadd(rnd<RD>(v), Elem<DT>::load(ep.bias, n));
        Elem<DT>::store(out, (int64_t)m * N + n, v);
      }
    }
  }
}

// Backward GEMMs.  C[i, lo_t + j] = sum_l A(i,l) * keep_t(i,l) * B(lo_t + j, l), where
//   dgrad: i = m, l = n, A = g [M,N] (l contiguous), B = w_mod (j contiguous), C = grad_x
//   wgrad: i = n, l = m, A = g^T     (i contiguous), B = xq    (j contiguous), C = grad_w
template <int DT, bool WGRAD>
__global__ void __launch_bounds__(kThreads)
bwd_simt_kernel(const void* __restrict__ g, const void* __restrict__ b_op,
                const uint32_t* __restrict__ keep_mask, int mask_words, int M, int K, int N,
                TileTable tt, void* __restrict__ c_out) {
  __shared__ float As[BK][BM + 1];
  __shared__ float Bs[BK][BN + 1];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int t = blockIdx.z;
  const int lo = tt.lo(t), hi = tt.hi(t);
  const int j0 = lo + blockIdx.x * BN;
  if (j0 >= hi) return;
  const int i0 = blockIdx.y * BM;
  const int I = WGRAD ? N : M;  // rows of C
  const int L = WGRAD ? M : N;  // reduction length
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int l0 = 0; l0 < L; l0 += BK) {
    if (WGRAD) stage_block<DT, false>(g, 1, N, i0, I, l0, L, As, tid);
    else stage_block<DT, true>(g, N, 1, i0, I, l0, L, As, tid);
    stage_block<DT, false>(b_op, 1, K, j0, hi, l0, L, Bs, tid);
    __syncthreads();
    if (keep_mask != nullptr) {
      // zero the gradient entries the ADC clamp of this tile blocked
      for (int e = tid; e < BM * BK; e += kThreads) {
        int i = e % BM, l = e / BM;
        int gi = i0 + i, gl = l0 + l;
        if (gi < I && gl < L) {
          int m = WGRAD ? gl : gi, n = WGRAD ? gi : gl;
          uint32_t word = keep_mask[((int64_t)t * mask_words + (n >> 5)) * M + m];
          if (((word >> (n & 31)) & 1u) == 0u) As[l][i] = 0.0f;
        }
      }
      __syncthreads();
    }
    mac_block(As, Bs, ty, tx, acc);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gi = i0 + ty * 4 + i;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gj = j0 + tx + 16 * j;
      if (gi < I && gj < hi) Elem<DT>::store(c_out, (int64_t)gi * K + gj, acc[i][j]);
    }
  }
}

inline int max_tile_width(const TileTable& tt) {
  int w = 0;
  for (int t = 0; t < tt.T; ++t) w = tt.hi(t) - tt.lo(t) > w ? tt.hi(t) - tt.lo(t) : w;
  return w;
}

}  // namespace

int launch_fwd_simt(int dtype, int round_dt, const void* xq, const void* w_mod, int K,
                    const TileTable& tt, const FwdEpilogueParams& ep, void* out, cudaStream_t s) {
  ProfScope prof(AL_K_FWD_GEMM, s);
  dim3 grid((ep.N + BN - 1) / BN, (ep.M + BM - 1) / BM);
  if (dtype == AL_F32)
    fwd_simt_kernel<kF32, kF32><<<grid, kThreads, 0, s>>>(xq, w_mod, K, tt, ep, out);
  else if (round_dt == AL_BF16)
    fwd_simt_kernel<kBF16, kBF16><<<grid, kThreads, 0, s>>>(xq, w_mod, K, tt, ep, out);
  else
    fwd_simt_kernel<kBF16, kF32><<<grid, kThreads, 0, s>>>(xq, w_mod, K, tt, ep, out);
  return check_launch("fwd_simt");
}

int launch_dgrad_simt(int dtype, const void* g, const void* w_mod, const uint32_t* keep_mask,
                      int mask_words, int M, int K, int N, const TileTable& tt, void* grad_x,
                      cudaStream_t s) {
  ProfScope prof(AL_K_DGRAD_GEMM, s);
  dim3 grid((max_tile_width(tt) + BN - 1) / BN, (M + BM - 1) / BM, tt.T);
  if (dtype == AL_F32)
    bwd_simt_kernel<kF32, false><<<grid, kThreads, 0, s>>>(g, w_mod, keep_mask, mask_words, M, K, N, tt, grad_x);
  else
    bwd_simt_kernel<kBF16, false><<<grid, kThreads, 0, s>>>(g, w_mod, keep_mask, mask_words, M, K, N, tt, grad_x);
  return check_launch("dgrad_simt");
}

int launch_wgrad_simt(int dtype, const void* g, const void* xq, const uint32_t* keep_mask,
                      int mask_words, int M, int K, int N, const TileTable& tt, void* grad_w,
                      cudaStream_t s) {
  ProfScope prof(AL_K_WGRAD_GEMM, s);
  dim3 grid((max_tile_width(tt) + BN - 1) / BN, (N + BM - 1) / BM, tt.T);
  if (dtype == AL_F32)
    bwd_simt_kernel<kF32, true><<<grid, kThreads, 0, s>>>(g, xq, keep_mask, mask_words, M, K, N, tt, grad_w);
  else
    bwd_simt_kernel<kBF16, true><<<grid, kThreads, 0, s>>>(g, xq, keep_mask, mask_words, M, K, N, tt, grad_w);
  return check_launch("wgrad_simt");
}

}  // namespace al
