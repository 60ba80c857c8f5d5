// Forward path for a handful of rows (M <= 16, e.g. single-token decoding): the layer is bound by
// streaming the weights from HBM once, so one kernel reads every (8 output channels x analog
// tile) block of W exactly once and takes from it both what the model needs of the weights --
// the per-channel abs-max and the tile maximum -- and the 16 x 8 block of tile dot products
// (mma.sync m16n8k16, bf16 in, fp32 accumulate; the tensor throughput is irrelevant here, the
// instruction only saves the CUDA cores the 16 x 8 x k multiply-adds).  The per-tile output stage
// needs the tile maximum over ALL channels, which is known only when the whole tile has been
// streamed, so it runs in a second, tiny kernel over the [T, 16, N] fp32 partial results.
//
// The DAC runs inside the same kernel: every CTA stages the 16 x tile_w slice of the raw inputs it
// multiplies with, takes the per-row range of the slice (dynamic input range) and quantises it in
// shared memory with the arithmetic of the stand-alone DAC pass, so a call of this path has no
// input pre-pass and no quantised copy of the inputs in HBM.
//
// Preconditions (checked by the caller): bf16, equally wide tiles with 16-byte aligned starts,
// no weight modifier active in this call (the GEMM reads `w` itself) and no output noise.
#include <cuda_bf16.h>

#include "analog_math.cuh"
#include "device_fast.cuh"
#include "internal.h"

namespace al {

namespace {

constexpr int kRows = 16;       // rows of one MMA; rows >= M are zero
constexpr int kWarps = 8;       // warps per CTA, each owns 8 output channels
constexpr int kChanPerWarp = 8;

__device__ __forceinline__ void mma_16x8x16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// pitch of a staged input row in bf16 elements: a multiple of 64 plus 32, so that consecutive rows
// are 64 bytes apart modulo 128 and the 16-byte reads of a quarter-warp (two rows x four
// k-chunks) fall on distinct banks
__host__ __device__ inline int x_pitch(int tile_w) { return ((tile_w + 63) / 64) * 64 + 32; }

// What the in-kernel DAC needs (dac.on == 0: the inputs arrive quantised).
struct SmallmDac {
  int on;
  int ir_mode;               // AL_IR_DYNAMIC or AL_IR_STATIC
  const uint16_t* ir_static;  // [T] ranges of a static input range
  float inp_res;
  int no_rounding;
  int small_codes;    // |code| stays far below 2^22: the add-based rint applies
  uint16_t* ir_rows;  // [T][M]: the dynamic ranges, written by the first column of CTAs
};

// grid: (ceil(N / 64), T).  acc [T][16][N] fp32, w_amax [T][N] bf16, tile_max [T] (float bits,
// zeroed by the caller).
__global__ void __launch_bounds__(kWarps * 32)
smallm_partial_kernel(const uint16_t* __restrict__ xq, int M, int K, const uint16_t* __restrict__ w, int N,
                      int tile_w, float* __restrict__ acc, uint16_t* __restrict__ w_amax,
                      float* __restrict__ tile_max, const SmallmDac dac) {
  extern __shared__ __align__(16) uint16_t x_s[];  // [16][pitch]
  const int t = blockIdx.y;
  const int lo = t * tile_w;
  const int pitch = x_pitch(tile_w);
  const int vec_per_row = pitch / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tg = lane & 3;
  const int n0 = (blockIdx.x * kWarps + warp) * kChanPerWarp;
  const bool active = n0 < N;
  const int n = active ? n0 + g : 0;  // the channel whose weights this thread streams (N is a multiple of 8)
  const uint16_t* wrow = w + (int64_t)n * K + lo;
  const int chunks = (tile_w + 31) / 32;  // 32 k per step: thread tg covers k = 32 kc + 8 tg .. + 7
  constexpr int kUnroll = 8;              // 8 x 16 bytes in flight per thread
  // the first batch of weight loads goes out before the inputs are staged, so that the two
  // latencies overlap
  uint4 wv[kUnroll];
  auto load_batch = [&](int kc0) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = (kc0 + u) * 32 + 8 * tg;
      wv[u] = (active && kc0 + u < chunks && k < tile_w) ? __ldg(reinterpret_cast<const uint4*>(wrow + k))
                                                         : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  load_batch(0);
  // stage the tile's slice of the inputs; rows >= M and the padding are zero
  for (int idx = threadIdx.x; idx < kRows * vec_per_row; idx += blockDim.x) {
    const int m = idx / vec_per_row, v = idx - m * vec_per_row;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (m < M && v * 8 < tile_w) val = *reinterpret_cast<const uint4*>(xq + (int64_t)m * K + lo + v * 8);
    *reinterpret_cast<uint4*>(x_s + m * pitch + v * 8) = val;
  }
  __syncthreads();
  if (dac.on) {
    // DAC of the staged slice by all threads, one 16-byte vector at a time: range of every (row,
    // tile) segment first, then the element-wise chain of the stand-alone pass (dac_prepare /
    // dac_apply; its packed bf16 form when rounding is on and the codes are small)
    __shared__ unsigned int row_bits[kRows];
    __shared__ QuantSeg row_q[kRows];
    const int vecs = tile_w / 8, total = M * vecs;
    if (dac.ir_mode == AL_IR_DYNAMIC) {
      if (threadIdx.x < kRows) row_bits[threadIdx.x] = 0u;
      __syncthreads();
      for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int m = idx / vecs, v = idx - m * vecs;
        const uint4 raw = *reinterpret_cast<const uint4*>(x_s + m * pitch + v * 8);
        __nv_bfloat162 a2 = __hmax2(__habs2(as_bf162(raw.x)), __habs2(as_bf162(raw.y)));
        a2 = __hmax2(a2, __hmax2(__habs2(as_bf162(raw.z)), __habs2(as_bf162(raw.w))));
        // non-negative floats order like their bit patterns
        atomicMax(&row_bits[m], __float_as_uint(fmaxf(__low2float(a2), __high2float(a2))));
      }
      __syncthreads();
    }
    if (threadIdx.x < M) {
      float ir;
      bool clampit = false;
      if (dac.ir_mode == AL_IR_DYNAMIC) {
        ir = __uint_as_float(row_bits[threadIdx.x]);
        if (blockIdx.x == 0) dac.ir_rows[(int64_t)t * M + threadIdx.x] = f32_to_bf16_bits(ir);
      } else {
        ir = bf16_bits_to_f32(dac.ir_static[t]);
        clampit = true;
      }
      row_q[threadIdx.x] = dac_prepare<kBF16>(ir, dac.inp_res, clampit, dac.no_rounding != 0);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
      const int m = idx / vecs, v = idx - m * vecs;
      const QuantSeg q = row_q[m];
      uint4* slot = reinterpret_cast<uint4*>(x_s + m * pitch + v * 8);
      const uint4 raw = *slot;
      uint32_t wd[4] = {raw.x, raw.y, raw.z, raw.w};
      if (q.quantise && !q.no_rounding && dac.small_codes) {
        const __nv_bfloat162 b2 = __float2bfloat162_rn(q.bound), nb2 = __float2bfloat162_rn(-q.bound);
        const __nv_bfloat162 step2 = __float2bfloat162_rn(q.step);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 x2 = as_bf162(wd[i]);
          if (q.clampit) x2 = __hmin2_nan(__hmax2_nan(x2, nb2), b2);
          const __nv_bfloat162 q2 = __floats2bfloat162_rn(fdiv_rcp(__low2float(x2), q.stepc, q.rstep),
                                                          fdiv_rcp(__high2float(x2), q.stepc, q.rstep));
          const float c_lo = rint_small(__low2float(q2)), c_hi = rint_small(__high2float(q2));
          const uint32_t c2 = (__float_as_uint(c_lo) >> 16) | (__float_as_uint(c_hi) & 0xffff0000u);
          wd[i] = as_u32(__hmul2_rn(as_bf162(c2), step2));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float code;
          const uint32_t lo16 = f32_to_bf16_bits(dac_apply<kBF16>(q, bf16_bits_to_f32((uint16_t)(wd[i] & 0xffffu)), &code));
          const uint32_t hi16 = f32_to_bf16_bits(dac_apply<kBF16>(q, bf16_bits_to_f32((uint16_t)(wd[i] >> 16)), &code));
          wd[i] = lo16 | (hi16 << 16);
        }
      }
      *slot = make_uint4(wd[0], wd[1], wd[2], wd[3]);
    }
    __syncthreads();
  }
  if (!active) return;

  const uint16_t* xa = x_s + g * pitch;
  const uint16_t* xb = x_s + (g + 8) * pitch;
  float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  __nv_bfloat162 m2 = __float2bfloat162_rn(0.0f);
  for (int kc0 = 0; kc0 < chunks; kc0 += kUnroll) {
    if (kc0 > 0) load_batch(kc0);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (kc0 + u < chunks) {
        const int k = (kc0 + u) * 32 + 8 * tg;
        const uint4 a = *reinterpret_cast<const uint4*>(xa + k);
        const uint4 b = *reinterpret_cast<const uint4*>(xb + k);
        // The MMA's k index is a label: this thread supplies the same eight physical k to A and B.
        mma_16x8x16(c, a.x, b.x, a.y, b.y, wv[u].x, wv[u].y);
        mma_16x8x16(c, a.z, b.z, a.w, b.w, wv[u].z, wv[u].w);
        m2 = __hmax2(m2, __habs2(as_bf162(wv[u].x)));
        m2 = __hmax2(m2, __habs2(as_bf162(wv[u].y)));
        m2 = __hmax2(m2, __habs2(as_bf162(wv[u].z)));
        m2 = __hmax2(m2, __habs2(as_bf162(wv[u].w)));
      }
    }
  }
  // c0, c1: row g, channels n0 + 2 tg, + 1; c2, c3: row g + 8
  float* arow = acc + ((int64_t)t * kRows + g) * N + n0 + 2 * tg;
  *reinterpret_cast<float2*>(arow) = make_float2(c[0], c[1]);
  *reinterpret_cast<float2*>(arow + (int64_t)8 * N) = make_float2(c[2], c[3]);
  // abs-max of channel n: over this thread's values, then over the four threads of the channel
  float amax = fmaxf(__low2float(m2), __high2float(m2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (tg == 0) w_amax[(int64_t)t * N + n] = f32_to_bf16_bits(amax);
  float wmax = amax;
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
  if (lane == 0) {
    unsigned int* slot = reinterpret_cast<unsigned int*>(tile_max) + t;
    const unsigned int bits = __float_as_uint(wmax);
    if (bits > *reinterpret_cast<volatile unsigned int*>(slot)) atomicMax(slot, bits);
  }
}

// out[m, n] = sum_t stage_t(acc[t, m, n]) + bias[n]; one thread per output
template <int RD>
__global__ void __launch_bounds__(256)
smallm_epilogue_kernel(const float* __restrict__ acc, FwdEpilogueParams ep, void* __restrict__ out) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int m = blockIdx.y;
  if (n >= ep.N) return;
  TileEpilogueCfg cfg;
  cfg.has_noise = 0; cfg.has_bound = ep.has_bound; cfg.has_adc = ep.has_adc;
  cfg.no_rounding = ep.no_rounding; cfg.noise_coef = ep.noise_coef; cfg.out_bound = ep.out_bound;
  cfg.out_res = ep.out_res;
  float sum = 0.0f;
  for (int t = 0; t < ep.T; ++t) {
    float ir = 0.0f;
    if (ep.ir_mode == AL_IR_DYNAMIC) ir = Elem<kBF16>::load(ep.ir_rows, (int64_t)t * ep.M + m);
    else if (ep.ir_mode == AL_IR_STATIC) ir = Elem<kBF16>::load(ep.ir_rows, t);
    const float t_max = rnd<kBF16>(ep.w_tile_max[t]);
    const float s_bound = ep.bound_pc ? Elem<kBF16>::load(ep.w_amax, (int64_t)t * ep.N + n) : t_max;
    bool keep;
    const float o = tile_epilogue<RD>(acc[((int64_t)t * kRows + m) * ep.N + n], ir, t_max, s_bound, 0.0f, cfg, &keep);
    sum = t == 0 ? fadd(0.0f, o) : rnd<RD>(fadd(sum, o));
  }
  if (ep.bias) sum = fadd(rnd<RD>(sum), Elem<kBF16>::load(ep.bias, n));
  Elem<kBF16>::store(out, (int64_t)m * ep.N + n, sum);
}

}  // namespace

int64_t smallm_scratch_floats(int N, int T) { return (int64_t)T * kRows * N; }

bool smallm_forward_supported(int M, int K, int N, const TileTable& tt) {
  if (M < 1 || M > kRows || K % 8 != 0 || N % 8 != 0) return false;
  const int w = tt.hi(0);
  for (int t = 1; t < tt.T; ++t)
    if (tt.hi(t) - tt.lo(t) != w) return false;
  return w % 8 == 0 && (size_t)kRows * x_pitch(w) * 2 <= 200 * 1024;
}

int launch_fwd_smallm(int round_dt, const void* xq, const void* w, int K, const TileTable& tt,
                      const FwdEpilogueParams& ep, void* w_amax, float* tile_max, float* scratch, void* out,
                      cudaStream_t s, int dac_in_kernel, const void* ir_static, float inp_res, int no_rounding) {
  ProfScope prof(AL_K_FWD_GEMM, s, 2);
  const int tile_w = tt.hi(0);
  const int smem = kRows * x_pitch(tile_w) * 2;
  cudaError_t e = cudaFuncSetAttribute(smallm_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess) e = cudaMemsetAsync(tile_max, 0, sizeof(float) * tt.T, s);
  if (e != cudaSuccess) {
    set_error("fwd_smallm: %s", cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  dim3 grid((ep.N + kWarps * kChanPerWarp - 1) / (kWarps * kChanPerWarp), tt.T);
  SmallmDac dac;
  dac.on = dac_in_kernel;
  dac.ir_mode = ep.ir_mode;
  dac.ir_static = reinterpret_cast<const uint16_t*>(ir_static);
  dac.inp_res = inp_res;
  dac.no_rounding = no_rounding;
  {
    const float states = inp_res > 0.0f ? (inp_res > 1.0f ? inp_res : 1.0f / inp_res) : 0.0f;
    dac.small_codes = states < 4.0e6f;
  }
  dac.ir_rows = reinterpret_cast<uint16_t*>(const_cast<void*>(ep.ir_rows));
  smallm_partial_kernel<<<grid, kWarps * 32, smem, s>>>(
      reinterpret_cast<const uint16_t*>(xq), ep.M, K, reinterpret_cast<const uint16_t*>(w), ep.N, tile_w, scratch,
      reinterpret_cast<uint16_t*>(w_amax), tile_max, dac);
  int rc = check_launch("smallm_partial");
  if (rc) return rc;
  FwdEpilogueParams e2 = ep;
  e2.w_amax = w_amax;
  e2.w_tile_max = tile_max;
  dim3 grid2((ep.N + 255) / 256, ep.M);
  if (round_dt == AL_BF16) smallm_epilogue_kernel<kBF16><<<grid2, 256, 0, s>>>(scratch, e2, out);
  else smallm_epilogue_kernel<kF32><<<grid2, 256, 0, s>>>(scratch, e2, out);
  return check_launch("smallm_epilogue");
}

}  // namespace al
