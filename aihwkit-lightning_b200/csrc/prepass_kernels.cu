// Operand pre-passes of the analog GEMM: the DAC (input range + input quantisation) that
// turns x into the GEMM's A operand, and the weight modifier (discretisation + additive
// Gaussian noise) that turns w into the B operand.  Both stream their operand once: one warp
// per (row, tile) segment, 128-bit loads/stores on the aligned body.
#include "analog_math.cuh"
#include "internal.h"

namespace al {

namespace {

constexpr int kWarpsPerBlock = 8;

template <int DT>
struct Pack;  // 16-byte vectors of DT elements
template <>
struct Pack<kF32> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const void* p, float v[4]) {
    float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  static __device__ __forceinline__ void store(void* p, const float v[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Pack<kBF16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const void* p, float v[8]) {
    uint4 q = *reinterpret_cast<const uint4*>(p);
    uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(void* p, const float v[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = (uint32_t)f32_to_bf16_bits(v[2 * i]) | ((uint32_t)f32_to_bf16_bits(v[2 * i + 1]) << 16);
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// Geometry of one segment as seen by a warp: scalar head, vector body, scalar tail.  All
// arrays that are walked together (input, output, optional extras) share the element offset,
// so they share the alignment as long as their base pointers are 16-byte aligned.
struct SegPlan {
  int head, nvec, done;
};
template <int DT>
__device__ __forceinline__ SegPlan plan_segment(int64_t start, int len) {
  constexpr int VN = Pack<DT>::N;
  int mis = (int)(start % VN);
  SegPlan p;
  p.head = mis == 0 ? 0 : VN - mis;
  if (p.head > len) p.head = len;
  p.nvec = (len - p.head) / VN;
  p.done = p.head + p.nvec * VN;
  return p;
}

template <int DT>
__device__ __forceinline__ float warp_abs_max(const void* a, int64_t start, int len, int lane,
                                              bool aligned_base) {
  constexpr int VN = Pack<DT>::N;
  constexpr int ES = 16 / VN;
  float m = 0.0f;
  if (aligned_base) {
    SegPlan p = plan_segment<DT>(start, len);
    if (lane < p.head) m = fabsf(Elem<DT>::load(a, start + lane));
    const char* body = reinterpret_cast<const char*>(a) + (start + p.head) * ES;
    for (int v = lane; v < p.nvec; v += 32) {
      float x[VN];
      Pack<DT>::load(body + (int64_t)v * 16, x);
#pragma unroll
      for (int i = 0; i < VN; ++i) m = fmaxf(m, fabsf(x[i]));
    }
    for (int i = p.done + lane; i < len; i += 32) m = fmaxf(m, fabsf(Elem<DT>::load(a, start + i)));
  } else {
    for (int i = lane; i < len; i += 32) m = fmaxf(m, fabsf(Elem<DT>::load(a, start + i)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  return m;
}

// xq[m, tile] = DAC(x[m, tile]); ir_rows[t, m] = abs-max of the segment (dynamic mode).
template <int DT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
dac_kernel(const void* __restrict__ x, int M, int K, TileTable tt, int ir_mode,
           const void* __restrict__ ir_static, float inp_res, int no_rounding,
           void* __restrict__ xq, void* __restrict__ ir_rows, void* __restrict__ codes,
           int aligned_base) {
  constexpr int VN = Pack<DT>::N;
  constexpr int ES = 16 / VN;
  int64_t seg = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (seg >= (int64_t)M * tt.T) return;
  int m = (int)(seg / tt.T), t = (int)(seg % tt.T);
  int lo = tt.lo(t), len = tt.hi(t) - lo;
  int64_t start = (int64_t)m * K + lo;
  float ir = 0.0f;
  bool clampit = false;
  if (ir_mode == AL_IR_DYNAMIC) {
    ir = warp_abs_max<DT>(x, start, len, lane, aligned_base != 0);
    if (lane == 0) Elem<DT>::store(ir_rows, (int64_t)t * M + m, ir);
  } else if (ir_mode == AL_IR_STATIC) {
    ir = Elem<DT>::load(ir_static, t);
    clampit = true;
  }
  const bool nr = no_rounding != 0;
  if (aligned_base && codes == nullptr) {
    SegPlan p = plan_segment<DT>(start, len);
    if (lane < p.head)
      Elem<DT>::store(xq, start + lane, dac<DT>(Elem<DT>::load(x, start + lane), ir, inp_res, clampit, nr, nullptr));
    const char* src = reinterpret_cast<const char*>(x) + (start + p.head) * ES;
    char* dst = reinterpret_cast<char*>(xq) + (start + p.head) * ES;
    for (int v = lane; v < p.nvec; v += 32) {
      float a[VN];
      Pack<DT>::load(src + (int64_t)v * 16, a);
#pragma unroll
      for (int i = 0; i < VN; ++i) a[i] = dac<DT>(a[i], ir, inp_res, clampit, nr, nullptr);
      Pack<DT>::store(dst + (int64_t)v * 16, a);
    }
    for (int i = p.done + lane; i < len; i += 32)
      Elem<DT>::store(xq, start + i, dac<DT>(Elem<DT>::load(x, start + i), ir, inp_res, clampit, nr, nullptr));
  } else {
    for (int i = lane; i < len; i += 32) {
      float c;
      float q = dac<DT>(Elem<DT>::load(x, start + i), ir, inp_res, clampit, nr, &c);
      Elem<DT>::store(xq, start + i, q);
      if (codes) Elem<DT>::store(codes, start + i, c);
    }
  }
}

// w_mod[n, tile] = noise(discretise(w[n, tile]))
template <int DT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
weight_modify_kernel(const void* __restrict__ w, int N, int K, TileTable tt,
                     const void* __restrict__ w_amax, const float* __restrict__ tile_max,
                     const int32_t* __restrict__ flags, int quant_type, float n_states,
                     float max_state, int noise_type, float std_dev,
                     const void* __restrict__ w_noise, uint64_t seed, uint64_t offset,
                     int no_rounding, void* __restrict__ w_mod) {
  int64_t seg = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (seg >= (int64_t)N * tt.T) return;
  int n = (int)(seg / tt.T), t = (int)(seg % tt.T);
  int lo = tt.lo(t), len = tt.hi(t) - lo;
  int64_t start = (int64_t)n * K + lo;
  float row_max = Elem<DT>::load(w_amax, (int64_t)t * N + n);
  float t_max = rnd<DT>(tile_max[t]);
  float q_scale = quant_type == AL_QUANT_DISCRETIZE ? t_max : row_max;
  float n_scale = noise_type == AL_NOISE_ADD_NORMAL ? t_max : row_max;
  bool gt1 = flags[t] != 0;
  const bool nr = no_rounding != 0;
  for (int i = lane; i < len; i += 32) {
    float v = Elem<DT>::load(w, start + i);
    if (quant_type != AL_QUANT_NONE) v = discretize<DT>(v, q_scale, n_states, max_state, gt1, nr);
    if (noise_type != AL_NOISE_NONE) {
      float xi = w_noise ? Elem<DT>::load(w_noise, start + i)
                         : rnd<DT>(normal1(seed, offset, 0u, (uint64_t)(start + i)));
      v = add_weight_noise<DT>(v, std_dev, n_scale, xi);
    }
    Elem<DT>::store(w_mod, start + i, v);
  }
}

inline unsigned seg_blocks(int64_t segs) { return (unsigned)((segs + kWarpsPerBlock - 1) / kWarpsPerBlock); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int launch_dac(int dtype, const void* x, int M, int K, const TileTable& tt, int ir_mode,
               const void* ir_static, float inp_res, int no_rounding, void* xq, void* ir_rows,
               void* codes, cudaStream_t s) {
  ProfScope prof(AL_K_DAC, s);
  int64_t segs = (int64_t)M * tt.T;
  int aligned = aligned16(x) && aligned16(xq);
  if (dtype == AL_F32)
    dac_kernel<kF32><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(x, M, K, tt, ir_mode, ir_static, inp_res, no_rounding, xq, ir_rows, codes, aligned);
  else
    dac_kernel<kBF16><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(x, M, K, tt, ir_mode, ir_static, inp_res, no_rounding, xq, ir_rows, codes, aligned);
  return check_launch("dac");
}

int launch_weight_modify(int dtype, const void* w, int N, int K, const TileTable& tt,
                         const void* w_amax, const float* tile_max, const int32_t* flags,
                         int quant_type, float n_states, float max_state, int noise_type,
                         float std_dev, const void* w_noise, uint64_t seed, uint64_t offset,
                         int no_rounding, void* w_mod, cudaStream_t s) {
  ProfScope prof(AL_K_WEIGHT_MODIFY, s);
  int64_t segs = (int64_t)N * tt.T;
  if (dtype == AL_F32)
    weight_modify_kernel<kF32><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(w, N, K, tt, w_amax, tile_max, flags, quant_type, n_states, max_state, noise_type, std_dev, w_noise, seed, offset, no_rounding, w_mod);
  else
    weight_modify_kernel<kBF16><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(w, N, K, tt, w_amax, tile_max, flags, quant_type, n_states, max_state, noise_type, std_dev, w_noise, seed, offset, no_rounding, w_mod);
  return check_launch("weight_modify");
}

}  // namespace al
