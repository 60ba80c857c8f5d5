// Operand pre-passes of the analog GEMM: the DAC (input range + input quantisation) that
// turns x into the GEMM's A operand, and the weight modifier (discretisation + additive
// Gaussian noise) that turns w into the B operand.  Both stream their operand once: one warp
// per (row, tile) segment, 128-bit loads/stores on the aligned body, per-segment constants
// (quantisation step, its reciprocal, noise amplitude) computed once per warp.
#include "analog_math.cuh"
#include "device_fast.cuh"
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
  // values are already exactly representable in bf16: packing is a pure bit move
  static __device__ __forceinline__ void store(void* p, const float v[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = (__float_as_uint(v[2 * i]) >> 16) | (__float_as_uint(v[2 * i + 1]) & 0xffff0000u);
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// Geometry of one segment as seen by a warp: scalar head, vector body, scalar tail.  All
// arrays that are walked together (input, output, noise) share the element offset, so they
// share the alignment as long as their base pointers are 16-byte aligned.
struct SegPlan {
  int head, nvec, done;
};
template <int DT>
__device__ __forceinline__ SegPlan plan_segment(int64_t start, int len, bool aligned_base) {
  constexpr int VN = Pack<DT>::N;
  SegPlan p;
  if (!aligned_base) {  // everything through the scalar path
    p.head = len;
    p.nvec = 0;
    p.done = len;
    return p;
  }
  int mis = (int)(start % VN);
  p.head = mis == 0 ? 0 : VN - mis;
  if (p.head > len) p.head = len;
  p.nvec = (len - p.head) / VN;
  p.done = p.head + p.nvec * VN;
  return p;
}

template <int DT>
__device__ __forceinline__ float warp_abs_max(const void* a, int64_t start, int len, int lane,
                                              const SegPlan& p) {
  constexpr int VN = Pack<DT>::N;
  constexpr int ES = 16 / VN;
  float m = 0.0f;
  for (int i = lane; i < p.head; i += 32) m = fmaxf(m, fabsf(Elem<DT>::load(a, start + i)));
  const char* body = reinterpret_cast<const char*>(a) + (start + p.head) * ES;
  if (DT == kBF16) {
    // packed: |x| and max on two bf16 at a time
    __nv_bfloat162 m2 = __float2bfloat162_rn(0.0f);
    for (int v = lane; v < p.nvec; v += 32) {
      const uint4 q = *reinterpret_cast<const uint4*>(body + (int64_t)v * 16);
      m2 = __hmax2(m2, __habs2(as_bf162(q.x)));
      m2 = __hmax2(m2, __habs2(as_bf162(q.y)));
      m2 = __hmax2(m2, __habs2(as_bf162(q.z)));
      m2 = __hmax2(m2, __habs2(as_bf162(q.w)));
    }
    m = fmaxf(m, fmaxf(__low2float(m2), __high2float(m2)));
  } else {
    for (int v = lane; v < p.nvec; v += 32) {
      float x[VN];
      Pack<DT>::load(body + (int64_t)v * 16, x);
#pragma unroll
      for (int i = 0; i < VN; ++i) m = fmaxf(m, fabsf(x[i]));
    }
  }
  for (int i = p.done + lane; i < len; i += 32) m = fmaxf(m, fabsf(Elem<DT>::load(a, start + i)));
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
           uint16_t* __restrict__ codes16, int aligned_base, int small_codes) {
  constexpr int VN = Pack<DT>::N;
  constexpr int ES = 16 / VN;
  const unsigned seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);  // rows * T < 2^31 (checked by the host)
  int lane = threadIdx.x & 31;
  if (seg >= (unsigned)M * (unsigned)tt.T) return;
  const int m = (int)(seg / (unsigned)tt.T), t = (int)(seg - (unsigned)m * (unsigned)tt.T);
  int lo = tt.lo(t), len = tt.hi(t) - lo;
  int64_t start = (int64_t)m * K + lo;
  const SegPlan p = plan_segment<DT>(start, len, aligned_base != 0 && codes == nullptr);
  float ir = 0.0f;
  bool clampit = false;
  if (ir_mode == AL_IR_DYNAMIC) {
    ir = warp_abs_max<DT>(x, start, len, lane, p);
    if (lane == 0) Elem<DT>::store(ir_rows, (int64_t)t * M + m, ir);
  } else if (ir_mode == AL_IR_STATIC) {
    ir = Elem<DT>::load(ir_static, t);
    clampit = true;
  }
  const QuantSeg q = dac_prepare<DT>(ir, inp_res, clampit, no_rounding != 0);
  for (int i = lane; i < p.head; i += 32) {
    float c;
    Elem<DT>::store(xq, start + i, dac_apply<DT>(q, Elem<DT>::load(x, start + i), &c));
    if (codes) Elem<DT>::store(codes, start + i, c);
    if (codes16) codes16[start + i] = f32_to_bf16_bits(c);  // small integers: exact
  }
  const char* src = reinterpret_cast<const char*>(x) + (start + p.head) * ES;
  char* dst = reinterpret_cast<char*>(xq) + (start + p.head) * ES;
  if (DT == kBF16 && q.quantise && !q.no_rounding && small_codes) {
    // The common case in bf16x2 arithmetic: a correctly rounded bf16 multiply equals "fp32
    // multiply, round to bf16" for bf16 operands (the fp32 product is exact), the same holds
    // for the clamp; the quotient goes through fp32 (reciprocal-based exact division), one
    // packed conversion and an add-based rint (codes are far below 2^22 here).
    const __nv_bfloat162 b2 = __float2bfloat162_rn(q.bound), nb2 = __float2bfloat162_rn(-q.bound);
    const __nv_bfloat162 step2 = __float2bfloat162_rn(q.step);
    const float stepc = q.stepc, rstep = q.rstep;
    const bool clamp_first = q.clampit != 0;
    for (int v = lane; v < p.nvec; v += 32) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + (int64_t)v * 16);
      uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 x2 = as_bf162(w[i]);
        if (clamp_first) x2 = __hmin2_nan(__hmax2_nan(x2, nb2), b2);
        const __nv_bfloat162 q2 = __floats2bfloat162_rn(fdiv_rcp(__low2float(x2), stepc, rstep),
                                                        fdiv_rcp(__high2float(x2), stepc, rstep));
        const float c_lo = rint_small(__low2float(q2)), c_hi = rint_small(__high2float(q2));
        // an integer of at most 8 significant bits is a bf16 value: packing is a bit move
        const uint32_t c2 = (__float_as_uint(c_lo) >> 16) | (__float_as_uint(c_hi) & 0xffff0000u);
        w[i] = as_u32(__hmul2_rn(as_bf162(c2), step2));
      }
      *reinterpret_cast<uint4*>(dst + (int64_t)v * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    for (int v = lane; v < p.nvec; v += 32) {
      float a[VN], c[VN];
      Pack<DT>::load(src + (int64_t)v * 16, a);
#pragma unroll
      for (int i = 0; i < VN; ++i) a[i] = dac_apply<DT>(q, a[i], &c[i]);
      Pack<DT>::store(dst + (int64_t)v * 16, a);
      if (codes16 != nullptr) {
#pragma unroll
        for (int i = 0; i < VN; ++i) codes16[start + p.head + (int64_t)v * VN + i] = f32_to_bf16_bits(c[i]);
      }
    }
  }
  for (int i = p.done + lane; i < len; i += 32) {
    float c;
    Elem<DT>::store(xq, start + i, dac_apply<DT>(q, Elem<DT>::load(x, start + i), &c));
    if (codes16) codes16[start + i] = f32_to_bf16_bits(c);
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
                     int no_rounding, void* __restrict__ w_mod, int aligned_base,
                     const uint64_t* __restrict__ offset_base) {
  constexpr int VN = Pack<DT>::N;
  constexpr int ES = 16 / VN;
  if (offset_base != nullptr) offset += *offset_base;  // the caller's call counter on the device
  const unsigned seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);  // rows * T < 2^31 (checked by the host)
  int lane = threadIdx.x & 31;
  if (seg >= (unsigned)N * (unsigned)tt.T) return;
  const int n = (int)(seg / (unsigned)tt.T), t = (int)(seg - (unsigned)n * (unsigned)tt.T);
  int lo = tt.lo(t), len = tt.hi(t) - lo;
  int64_t start = (int64_t)n * K + lo;
  float row_max = Elem<DT>::load(w_amax, (int64_t)t * N + n);
  float t_max = rnd<DT>(tile_max[t]);
  const float n_scale = noise_type == AL_NOISE_ADD_NORMAL ? t_max : row_max;
  const WeightSeg ws =
      quant_type == kQuantLearnClamp
          ? weight_prepare_learn_clamp<DT>(row_max, flags[t] != 0, noise_type, std_dev, n_scale)
          : weight_prepare<DT>(quant_type, quant_type == AL_QUANT_DISCRETIZE ? t_max : row_max, n_states,
                               max_state, flags[t] != 0, noise_type, std_dev, n_scale, no_rounding != 0);
  const SegPlan p = plan_segment<DT>(start, len, aligned_base != 0);
  auto one = [&](int i) {
    float xi = 0.0f;
    if (ws.noise)
      xi = w_noise ? Elem<DT>::load(w_noise, start + i)
                   : rnd<DT>(normal1(seed, offset, 0u, (uint64_t)(start + i)));
    Elem<DT>::store(w_mod, start + i, weight_apply<DT>(ws, Elem<DT>::load(w, start + i), xi));
  };
  for (int i = lane; i < p.head; i += 32) one(i);
  const char* src = reinterpret_cast<const char*>(w) + (start + p.head) * ES;
  const char* nsrc = reinterpret_cast<const char*>(w_noise) + (start + p.head) * ES;
  char* dst = reinterpret_cast<char*>(w_mod) + (start + p.head) * ES;
  for (int v = lane; v < p.nvec; v += 32) {
    float a[VN], xi[VN];
    Pack<DT>::load(src + (int64_t)v * 16, a);
    if (ws.noise) {
      if (w_noise) {
        Pack<DT>::load(nsrc + (int64_t)v * 16, xi);
      } else {
        // the vector starts at a multiple of VN elements, i.e. on a group-of-four boundary
        const uint64_t g0 = (uint64_t)(start + p.head + (int64_t)v * VN) >> 2;
#pragma unroll
        for (int g = 0; g < VN / 4; ++g) {
          normal4(seed, offset, 0u, g0 + g, &xi[4 * g]);
#pragma unroll
          for (int e = 0; e < 4; ++e) xi[4 * g + e] = rnd_int<DT>(xi[4 * g + e]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < VN; ++i) xi[i] = 0.0f;
    }
#pragma unroll
    for (int i = 0; i < VN; ++i) a[i] = weight_apply<DT>(ws, a[i], xi[i]);
    Pack<DT>::store(dst + (int64_t)v * 16, a);
  }
  for (int i = p.done + lane; i < len; i += 32) one(i);
}

// Weight pre-pass in one sweep, for modifiers whose scale is the segment's own abs-max (or
// that do nothing): per (channel, tile) segment the warp computes the abs-max, stores it,
// folds it into the tile's abs-max with an integer atomicMax (exact and order independent for
// non-negative floats) and, if weight noise is on, writes w + (std_dev * abs-max) * xi.
template <int DT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
weight_fused_kernel(const void* __restrict__ w, int N, int K, TileTable tt, void* __restrict__ w_amax,
                    float* __restrict__ tile_max, int noise_type, float std_dev,
                    const void* __restrict__ w_noise, uint64_t seed, uint64_t offset,
                    void* __restrict__ w_mod, int aligned_base, const uint64_t* __restrict__ offset_base) {
  constexpr int VN = Pack<DT>::N;
  constexpr int ES = 16 / VN;
  if (offset_base != nullptr) offset += *offset_base;  // the caller's call counter on the device
  const unsigned seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);  // rows * T < 2^31 (checked by the host)
  int lane = threadIdx.x & 31;
  if (seg >= (unsigned)N * (unsigned)tt.T) return;
  const int n = (int)(seg / (unsigned)tt.T), t = (int)(seg - (unsigned)n * (unsigned)tt.T);
  int lo = tt.lo(t), len = tt.hi(t) - lo;
  int64_t start = (int64_t)n * K + lo;
  const SegPlan p = plan_segment<DT>(start, len, aligned_base != 0);
  const float row_max = warp_abs_max<DT>(w, start, len, lane, p);
  if (lane == 0) {
    Elem<DT>::store(w_amax, (int64_t)t * N + n, row_max);
    // the running maximum only grows: a plain read first keeps all but a few warps off the
    // atomic unit (tens of thousands of atomics on T addresses would serialise)
    unsigned int* slot = reinterpret_cast<unsigned int*>(tile_max) + t;
    const unsigned int bits = __float_as_uint(row_max);
    if (bits > *reinterpret_cast<volatile unsigned int*>(slot)) atomicMax(slot, bits);
  }
  if (noise_type == AL_NOISE_NONE) return;
  const WeightSeg ws = weight_prepare<DT>(AL_QUANT_NONE, row_max, 1.0f, 1.0f, false, noise_type, std_dev,
                                          row_max, false);
  auto one = [&](int i) {
    float xi = w_noise ? Elem<DT>::load(w_noise, start + i)
                       : rnd<DT>(normal1(seed, offset, 0u, (uint64_t)(start + i)));
    Elem<DT>::store(w_mod, start + i, weight_apply<DT>(ws, Elem<DT>::load(w, start + i), xi));
  };
  for (int i = lane; i < p.head; i += 32) one(i);
  const char* src = reinterpret_cast<const char*>(w) + (start + p.head) * ES;
  const char* nsrc = reinterpret_cast<const char*>(w_noise) + (start + p.head) * ES;
  char* dst = reinterpret_cast<char*>(w_mod) + (start + p.head) * ES;
  for (int v = lane; v < p.nvec; v += 32) {
    float xi[8];
    if (w_noise) {
      float tmp[VN];
      Pack<DT>::load(nsrc + (int64_t)v * 16, tmp);
#pragma unroll
      for (int i = 0; i < VN; ++i) xi[i] = tmp[i];
    } else {
      // VN == 8: one group of eight; VN == 4: the half of the group this vector covers
      const uint64_t e0 = (uint64_t)(start + p.head + (int64_t)v * VN);
      float z[8];
      normal8_fast(seed, offset, 0u, e0 >> 3, z);
#pragma unroll
      for (int i = 0; i < VN; ++i) xi[i] = z[(VN == 8 ? 0 : (int)(e0 & 4)) + i];
    }
    if (DT == kBF16) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + (int64_t)v * 16);
      uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
      const __nv_bfloat162 amp2 = __float2bfloat162_rn(ws.amp);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 z2 = __floats2bfloat162_rn(xi[2 * i], xi[2 * i + 1]);
        wv[i] = as_u32(__hadd2_rn(as_bf162(wv[i]), __hmul2_rn(amp2, z2)));
      }
      *reinterpret_cast<uint4*>(dst + (int64_t)v * 16) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
    } else {
      float a[VN];
      Pack<DT>::load(src + (int64_t)v * 16, a);
#pragma unroll
      for (int i = 0; i < VN; ++i) a[i] = weight_apply<DT>(ws, a[i], xi[i]);
      Pack<DT>::store(dst + (int64_t)v * 16, a);
    }
  }
  for (int i = p.done + lane; i < len; i += 32) one(i);
}

inline unsigned seg_blocks(int64_t segs) { return (unsigned)((segs + kWarpsPerBlock - 1) / kWarpsPerBlock); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }


// ---- batched bf16 fast path of the DAC ------------------------------------------------------------------
// A warp that handles one 1 KiB segment has 1 KiB of loads in flight and then a chain of
// dependent steps (reduce, constants, arithmetic, store): the DAC kernel above is bound by that
// latency, not by HBM.  When every analog tile is 256 * Q elements wide (Q = 1, 2, 4, 8)
// and 16-byte aligned, a warp takes 8 / Q consecutive tiles of one row instead: all eight 16-byte
// vectors of a lane are loaded up front (4 KiB in flight per warp), the per-tile abs-max comes
// from the registers, and the same registers are transformed and stored.
constexpr int kBatchVecs = 8;

__device__ __forceinline__ float vecs_abs_max(const uint4* v, int count) {
  __nv_bfloat162 m2 = __float2bfloat162_rn(0.0f);
  for (int j = 0; j < count; ++j) {
    m2 = __hmax2(m2, __habs2(as_bf162(v[j].x)));
    m2 = __hmax2(m2, __habs2(as_bf162(v[j].y)));
    m2 = __hmax2(m2, __habs2(as_bf162(v[j].z)));
    m2 = __hmax2(m2, __habs2(as_bf162(v[j].w)));
  }
  float m = fmaxf(__low2float(m2), __high2float(m2));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  return m;
}

template <int Q>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
dac_batched_kernel(const uint16_t* __restrict__ x, int M, int K, int T, int ir_mode,
                   const uint16_t* __restrict__ ir_static, float inp_res, uint16_t* __restrict__ xq,
                   uint16_t* __restrict__ ir_rows, uint32_t* __restrict__ zero_words, int zero_count) {
  // side job of the first block: clear the words the weight pre-pass that follows accumulates into
  // (saves that pass a memset between the two kernels)
  if (blockIdx.x == 0 && (int)threadIdx.x < zero_count) zero_words[threadIdx.x] = 0u;
  constexpr int kTiles = kBatchVecs / Q;  // tiles per warp
  constexpr int kTileW = 256 * Q;
  const int batches = (T + kTiles - 1) / kTiles;
  const unsigned wid = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (unsigned)M * (unsigned)batches) return;
  const int m = (int)(wid / (unsigned)batches), t0 = (int)(wid - (unsigned)m * (unsigned)batches) * kTiles;
  const int64_t row = (int64_t)m * K;
  uint4 v[kBatchVecs];
#pragma unroll
  for (int j = 0; j < kBatchVecs; ++j) {
    const int t = t0 + j / Q;
    v[j] = t < T ? __ldg(reinterpret_cast<const uint4*>(x + row + (int64_t)t * kTileW + ((j % Q) * 32 + lane) * 8))
                 : make_uint4(0u, 0u, 0u, 0u);
  }
  const uint64_t magic2 = f32x2_pack(12582912.0f, 12582912.0f), nmagic2 = f32x2_pack(-12582912.0f, -12582912.0f);
#pragma unroll
  for (int i = 0; i < kTiles; ++i) {
    const int t = t0 + i;
    if (t >= T) break;
    float ir;
    bool clampit = false;
    if (ir_mode == AL_IR_DYNAMIC) {
      ir = vecs_abs_max(&v[i * Q], Q);
      if (lane == 0) ir_rows[(int64_t)t * M + m] = f32_to_bf16_bits(ir);
    } else {
      ir = Elem<kBF16>::load(ir_static, t);
      clampit = true;
    }
    const QuantSeg q = dac_prepare<kBF16>(ir, inp_res, clampit, false);
    const __nv_bfloat162 b2 = __float2bfloat162_rn(q.bound), nb2 = __float2bfloat162_rn(-q.bound);
    const __nv_bfloat162 step2 = __float2bfloat162_rn(q.step);
    const uint64_t nstepc2 = f32x2_pack(-q.stepc, -q.stepc), rstep2 = f32x2_pack(q.rstep, q.rstep);
#pragma unroll
    for (int jj = 0; jj < Q; ++jj) {
      uint32_t w[4] = {v[i * Q + jj].x, v[i * Q + jj].y, v[i * Q + jj].z, v[i * Q + jj].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 x2 = as_bf162(w[e]);
        if (clampit) x2 = __hmin2_nan(__hmax2_nan(x2, nb2), b2);
        float q_lo, q_hi, c_lo, c_hi;
        f32x2_unpack(f32x2_div_rcp(f32x2_pack(__low2float(x2), __high2float(x2)), nstepc2, rstep2), &q_lo, &q_hi);
        const __nv_bfloat162 q2 = __floats2bfloat162_rn(q_lo, q_hi);
        f32x2_unpack(f32x2_add(f32x2_add(f32x2_pack(__low2float(q2), __high2float(q2)), magic2), nmagic2), &c_lo, &c_hi);
        // an integer of at most 8 significant bits is a bf16 value: packing is a bit move
        const uint32_t c2 = __byte_perm(__float_as_uint(c_lo), __float_as_uint(c_hi), 0x7632);
        w[e] = as_u32(__hmul2_rn(as_bf162(c2), step2));
      }
      *reinterpret_cast<uint4*>(xq + row + (int64_t)t * kTileW + (jj * 32 + lane) * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// Persistent form of weight_fused_kernel for bf16 tiles of 256 * Q elements: a resident grid of
// warps walks the (channel, tile) segments with the vectors of its next segment already in flight
// while it reduces, perturbs and stores the current one, so a warp always has a load outstanding
// and the grid needs no block turnover.  Tile maxima: one atomic per warp at the very end.
template <int Q>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
weight_fused_stream_kernel(const uint16_t* __restrict__ w, int N, int K, int T, uint16_t* __restrict__ w_amax,
                           float* __restrict__ tile_max, int noise_type, float std_dev, const NoiseKeys nk,
                           uint16_t* __restrict__ w_mod) {
  constexpr int kTileW = 256 * Q;
  const int lane = threadIdx.x & 31;
  const unsigned n_warps = gridDim.x * kWarpsPerBlock;
  const unsigned segs = (unsigned)N * (unsigned)T;
  const NoiseCounter ctr = noise_counter(nk);
  unsigned seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  // the grid is sized so that n_warps is a multiple of T: a warp always meets the same tile
  const int t = (int)(seg % (unsigned)T);
  float run_max = 0.0f;
  uint4 cur[Q], nxt[Q];
  auto load = [&](unsigned sg, uint4* dst) {
    const int64_t base = (int64_t)(sg / (unsigned)T) * K + (int64_t)t * kTileW;
#pragma unroll
    for (int j = 0; j < Q; ++j)
      dst[j] = sg < segs ? __ldg(reinterpret_cast<const uint4*>(w + base + (j * 32 + lane) * 8)) : make_uint4(0u, 0u, 0u, 0u);
  };
  load(seg, cur);
  for (; seg < segs; seg += n_warps) {
    load(seg + n_warps, nxt);
    const int n = (int)(seg / (unsigned)T);
    const float row_max = vecs_abs_max(cur, Q);
    run_max = fmaxf(run_max, row_max);
    if (lane == 0) w_amax[(int64_t)t * N + n] = f32_to_bf16_bits(row_max);
    if (noise_type != AL_NOISE_NONE) {
      const __nv_bfloat162 amp2 = __float2bfloat162_rn(rnd<kBF16>(fmul(std_dev, row_max)));
#pragma unroll
      for (int j = 0; j < Q; ++j) {
        const int64_t e0 = (int64_t)n * K + (int64_t)t * kTileW + (j * 32 + lane) * 8;
        float z[8];
        normal8_keyed(nk, ctr, (uint64_t)e0 >> 3, z);
        uint32_t wv[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __nv_bfloat162 z2 = __floats2bfloat162_rn(z[2 * e], z[2 * e + 1]);
          wv[e] = as_u32(__hadd2_rn(as_bf162(wv[e]), __hmul2_rn(amp2, z2)));
        }
        *reinterpret_cast<uint4*>(w_mod + e0) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < Q; ++j) cur[j] = nxt[j];
  }
  if (lane == 0) {
    unsigned int* slot = reinterpret_cast<unsigned int*>(tile_max) + t;
    const unsigned int bits = __float_as_uint(run_max);
    if (bits > *reinterpret_cast<volatile unsigned int*>(slot)) atomicMax(slot, bits);
  }
}

// A resident grid (what the occupancy query says fits, times the SM count) whose warp count is a
// multiple of T.  Returns -1 when there is none, else the launch status.
template <int Q>
int launch_weight_stream(const void* w, int N, int K, int T, void* w_amax, float* tile_max, int noise_type,
                         float std_dev, const NoiseKeys& nk, void* w_mod, cudaStream_t s) {
  static int resident = 0;  // blocks of this instantiation the device holds at once
  if (resident == 0) {
    int sms = 0, dev = 0, per_sm = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, weight_fused_stream_kernel<Q>, kWarpsPerBlock * 32, 0) !=
            cudaSuccess || per_sm <= 0)
      per_sm = 2;
    resident = sms * per_sm;
  }
  const int64_t segs = (int64_t)N * T;
  int64_t blocks = resident;
  if (blocks * kWarpsPerBlock > segs) blocks = segs / kWarpsPerBlock;
  while (blocks > 0 && (blocks * kWarpsPerBlock) % T != 0) --blocks;
  if (blocks <= 0) return -1;
  weight_fused_stream_kernel<Q><<<(unsigned)blocks, kWarpsPerBlock * 32, 0, s>>>(
      reinterpret_cast<const uint16_t*>(w), N, K, T, reinterpret_cast<uint16_t*>(w_amax), tile_max, noise_type, std_dev,
      nk, reinterpret_cast<uint16_t*>(w_mod));
  return check_launch("weight_fused_stream");
}

// Q for a tiling the batched kernels take (0: use the general kernels)
int batched_q(const TileTable& tt, int K) {
  const int w = tt.hi(0);
  if (w != 256 && w != 512 && w != 1024 && w != 2048) return 0;
  for (int t = 1; t < tt.T; ++t)
    if (tt.hi(t) - tt.lo(t) != w) return 0;
  if ((int64_t)tt.T * w != K) return 0;
  return w / 256;
}

}  // namespace

int launch_dac(int dtype, const void* x, int M, int K, const TileTable& tt, int ir_mode,
               const void* ir_static, float inp_res, int no_rounding, void* xq, void* ir_rows,
               void* codes, cudaStream_t s, void* codes16, void* zero_words, int zero_count, bool* zeroed) {
  ProfScope prof(AL_K_DAC, s);
  if (zeroed) *zeroed = false;
  int64_t segs = (int64_t)M * tt.T;
  int aligned = aligned16(x) && aligned16(xq);
  // |code| <= max(inp_res, 1/inp_res)/2 + 1: the guard-free rint needs that below 2^22
  float states = inp_res > 0.0f ? (inp_res > 1.0f ? inp_res : 1.0f / inp_res) : 0.0f;
  int small_codes = states < 4.0e6f;
  const int q = batched_q(tt, K);
  if (dtype == AL_BF16 && q > 0 && aligned && codes == nullptr && inp_res > 0.0f && !no_rounding && small_codes &&
      (ir_mode == AL_IR_DYNAMIC || ir_mode == AL_IR_STATIC) && aligned16(ir_rows)) {
    const int64_t warps = (int64_t)M * ((tt.T + kBatchVecs / q - 1) / (kBatchVecs / q));
    const unsigned blocks = seg_blocks(warps);
    const uint16_t* xs = reinterpret_cast<const uint16_t*>(x);
    const uint16_t* irs = reinterpret_cast<const uint16_t*>(ir_static);
    uint16_t* xqs = reinterpret_cast<uint16_t*>(xq);
    uint16_t* irr = reinterpret_cast<uint16_t*>(ir_rows);
    uint32_t* zw = reinterpret_cast<uint32_t*>(zero_words);
    if (zw == nullptr || zero_count > kWarpsPerBlock * 32) zero_count = 0;
    if (zeroed) *zeroed = zero_count > 0;
    switch (q) {
      case 1: dac_batched_kernel<1><<<blocks, kWarpsPerBlock * 32, 0, s>>>(xs, M, K, tt.T, ir_mode, irs, inp_res, xqs, irr, zw, zero_count); break;
      case 2: dac_batched_kernel<2><<<blocks, kWarpsPerBlock * 32, 0, s>>>(xs, M, K, tt.T, ir_mode, irs, inp_res, xqs, irr, zw, zero_count); break;
      case 4: dac_batched_kernel<4><<<blocks, kWarpsPerBlock * 32, 0, s>>>(xs, M, K, tt.T, ir_mode, irs, inp_res, xqs, irr, zw, zero_count); break;
      default: dac_batched_kernel<8><<<blocks, kWarpsPerBlock * 32, 0, s>>>(xs, M, K, tt.T, ir_mode, irs, inp_res, xqs, irr, zw, zero_count); break;
    }
    return check_launch("dac_batched");
  }
  if (dtype == AL_F32)
    dac_kernel<kF32><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(x, M, K, tt, ir_mode, ir_static, inp_res, no_rounding, xq, ir_rows, codes, static_cast<uint16_t*>(codes16), aligned, small_codes);
  else
    dac_kernel<kBF16><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(x, M, K, tt, ir_mode, ir_static, inp_res, no_rounding, xq, ir_rows, codes, nullptr, aligned, small_codes);
  return check_launch("dac");
}

int launch_weight_modify(int dtype, const void* w, int N, int K, const TileTable& tt,
                         const void* w_amax, const float* tile_max, const int32_t* flags,
                         int quant_type, float n_states, float max_state, int noise_type,
                         float std_dev, const void* w_noise, uint64_t seed, uint64_t offset,
                         int no_rounding, void* w_mod, cudaStream_t s, const uint64_t* offset_base) {
  ProfScope prof(AL_K_WEIGHT_MODIFY, s);
  int64_t segs = (int64_t)N * tt.T;
  int aligned = aligned16(w) && aligned16(w_mod) && (w_noise == nullptr || aligned16(w_noise));
  if (dtype == AL_F32)
    weight_modify_kernel<kF32><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(w, N, K, tt, w_amax, tile_max, flags, quant_type, n_states, max_state, noise_type, std_dev, w_noise, seed, offset, no_rounding, w_mod, aligned, offset_base);
  else
    weight_modify_kernel<kBF16><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(w, N, K, tt, w_amax, tile_max, flags, quant_type, n_states, max_state, noise_type, std_dev, w_noise, seed, offset, no_rounding, w_mod, aligned, offset_base);
  return check_launch("weight_modify");
}

int launch_weight_fused(int dtype, const void* w, int N, int K, const TileTable& tt, void* w_amax,
                        float* tile_max, int noise_type, float std_dev, const void* w_noise,
                        uint64_t seed, uint64_t offset, void* w_mod, cudaStream_t s, const uint64_t* offset_base,
                        bool tile_max_zeroed) {
  ProfScope prof(AL_K_WEIGHT_MODIFY, s);
  int64_t segs = (int64_t)N * tt.T;
  int aligned = aligned16(w) && (w_mod == nullptr || aligned16(w_mod)) && (w_noise == nullptr || aligned16(w_noise));
  // tile_max[T] floats followed by T int32 flags (zero: the discretiser is off on this path); cleared
  // here unless the DAC kernel before this one already did it
  cudaError_t e = tile_max_zeroed ? cudaSuccess : cudaMemsetAsync(tile_max, 0, 2 * sizeof(float) * tt.T, s);
  if (e != cudaSuccess) {
    set_error("weight_fused: memset: %s", cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  const int q = batched_q(tt, K);
  if (dtype == AL_BF16 && q > 0 && q <= 4 && aligned && w_noise == nullptr && aligned16(w_amax) &&
      (noise_type == AL_NOISE_NONE || w_mod != nullptr)) {
    const NoiseKeys nk = make_noise_keys(seed, offset, 0u, offset_base);
    int rc = -1;
    switch (q) {
      case 1: rc = launch_weight_stream<1>(w, N, K, tt.T, w_amax, tile_max, noise_type, std_dev, nk, w_mod, s); break;
      case 2: rc = launch_weight_stream<2>(w, N, K, tt.T, w_amax, tile_max, noise_type, std_dev, nk, w_mod, s); break;
      default: rc = launch_weight_stream<4>(w, N, K, tt.T, w_amax, tile_max, noise_type, std_dev, nk, w_mod, s); break;
    }
    if (rc >= 0) return rc;  // < 0: no grid with a multiple of T warps, take the general kernel
  }
  if (dtype == AL_F32)
    weight_fused_kernel<kF32><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(w, N, K, tt, w_amax, tile_max, noise_type, std_dev, w_noise, seed, offset, w_mod, aligned, offset_base);
  else
    weight_fused_kernel<kBF16><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(w, N, K, tt, w_amax, tile_max, noise_type, std_dev, w_noise, seed, offset, w_mod, aligned, offset_base);
  return check_launch("weight_fused");
}

}  // namespace al
