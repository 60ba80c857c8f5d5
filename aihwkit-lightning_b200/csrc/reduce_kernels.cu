// Reductions of the analog linear path: per-(row, tile) abs-max, per-tile abs-max over rows,
// per-tile standard deviation over all rows, the predicated input-range update and the
// Gaussian weight clipping.  All are HBM-bound scans: one warp per (row, tile) segment,
// 128-bit loads on the aligned body of the segment, warp-shuffle reductions, and a fixed
// merge order (no floating-point atomics), so results are bitwise repeatable.
#include <mutex>

#include "analog_math.cuh"
#include "internal.h"

namespace al {

namespace {

constexpr int kWarpsPerBlock = 8;

template <int DT>
struct Vec;  // 16-byte vector of DT elements
template <>
struct Vec<kF32> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const void* p, float v[4]) {
    float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
};
template <>
struct Vec<kBF16> {
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
};

// Calls f(value) for every element of the segment [start, start+len) of a DT array, spreading
// the elements over the 32 lanes of the calling warp: scalar head up to the first 16-byte
// boundary, vector body, scalar tail.
template <int DT, class F>
__device__ __forceinline__ void warp_scan_segment(const void* base, int64_t start, int len,
                                                  int lane, F f) {
  constexpr int VN = Vec<DT>::N;
  constexpr int ES = 16 / VN;
  const char* p = reinterpret_cast<const char*>(base) + start * ES;
  int mis = (int)((reinterpret_cast<uintptr_t>(p) & 15) / ES);
  int head = mis == 0 ? 0 : VN - mis;
  if (head > len) head = len;
  if (lane < head) f(Elem<DT>::load(p, lane));
  int nvec = (len - head) / VN;
  const char* body = p + (int64_t)head * ES;
  for (int v = lane; v < nvec; v += 32) {
    float x[VN];
    Vec<DT>::load(body + (int64_t)v * 16, x);
#pragma unroll
    for (int i = 0; i < VN; ++i) f(x[i]);
  }
  int done = head + nvec * VN;
  for (int i = done + lane; i < len; i += 32) f(Elem<DT>::load(p, i));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// out[t, r] = max |a[r, tile t]|
template <int DT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
abs_max_tiles_kernel(const void* __restrict__ a, int rows, int K, TileTable tt,
                     void* __restrict__ out) {
  const unsigned seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);  // rows * T < 2^31 (checked by the host)
  int lane = threadIdx.x & 31;
  if (seg >= (unsigned)rows * (unsigned)tt.T) return;
  const int r = (int)(seg / (unsigned)tt.T), t = (int)(seg - (unsigned)r * (unsigned)tt.T);
  int lo = tt.lo(t), hi = tt.hi(t);
  float m = 0.0f;
  warp_scan_segment<DT>(a, (int64_t)r * K + lo, hi - lo, lane, [&](float v) { m = fmaxf(m, fabsf(v)); });
  m = warp_max(m);
  if (lane == 0) Elem<DT>::store(out, (int64_t)t * rows + r, m);
}

// tile_max[t] = max_r amax[t, r]; flags[t] = the "(res > 1).all()" switch of the weight
// discretiser for that tile.
template <int DT>
__global__ void tile_max_kernel(const void* __restrict__ amax, int rows, int quant_type,
                                float n_states, float* __restrict__ tile_max,
                                int32_t* __restrict__ flags) {
  __shared__ float s_max[256];
  __shared__ int s_all[256];
  int t = blockIdx.x;
  float m = 0.0f;
  int all = 1;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    float v = Elem<DT>::load(amax, (int64_t)t * rows + r);
    m = fmaxf(m, v);
    if (quant_type == AL_QUANT_DISCRETIZE_PER_CHANNEL) all &= discretize_scale_gt1<DT>(v, n_states) ? 1 : 0;
    if (quant_type == kQuantLearnClamp) all &= v > 1.0f ? 1 : 0;
  }
  s_max[threadIdx.x] = m;
  s_all[threadIdx.x] = all;
  __syncthreads();
  for (int o = blockDim.x / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      s_max[threadIdx.x] = fmaxf(s_max[threadIdx.x], s_max[threadIdx.x + o]);
      s_all[threadIdx.x] &= s_all[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    tile_max[t] = s_max[0];
    int f = 0;
    if (quant_type == AL_QUANT_DISCRETIZE) f = discretize_scale_gt1<DT>(s_max[0], n_states) ? 1 : 0;
    if (quant_type == AL_QUANT_DISCRETIZE_PER_CHANNEL || quant_type == kQuantLearnClamp) f = s_all[0];
    flags[t] = f;
  }
}

// Stage 1 of the per-tile std: (mean, M2) of every (row, tile) segment, two passes over the
// segment (the second one is served by L1/L2).
template <int DT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
segment_moments_kernel(const void* __restrict__ a, int rows, int K, TileTable tt,
                       float* __restrict__ partial) {
  const unsigned seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);  // rows * T < 2^31 (checked by the host)
  int lane = threadIdx.x & 31;
  if (seg >= (unsigned)rows * (unsigned)tt.T) return;
  const int r = (int)(seg / (unsigned)tt.T), t = (int)(seg - (unsigned)r * (unsigned)tt.T);
  int lo = tt.lo(t), len = tt.hi(t) - lo;
  float s = 0.0f;
  warp_scan_segment<DT>(a, (int64_t)r * K + lo, len, lane, [&](float v) { s += v; });
  float mean = warp_sum(s) / (float)len;
  float m2 = 0.0f;
  warp_scan_segment<DT>(a, (int64_t)r * K + lo, len, lane, [&](float v) {
    float d = v - mean;
    m2 = fmaf(d, d, m2);
  });
  m2 = warp_sum(m2);
  if (lane == 0) {
    partial[((int64_t)t * rows + r) * 2] = mean;
    partial[((int64_t)t * rows + r) * 2 + 1] = m2;
  }
}

struct Moments {
  double n, mean, m2;
};
__device__ __forceinline__ Moments merge(const Moments& a, const Moments& b) {
  if (b.n == 0.0) return a;
  if (a.n == 0.0) return b;
  Moments o;
  o.n = a.n + b.n;
  double d = b.mean - a.mean;
  o.mean = a.mean + d * (b.n / o.n);
  o.m2 = a.m2 + b.m2 + d * d * (a.n * b.n / o.n);
  return o;
}

// Stage 2: pairwise merge (Chan et al.) of the row partials of one tile in double, fixed order.
template <int DT>
__global__ void merge_moments_kernel(const float* __restrict__ partial, int rows, TileTable tt,
                                     float* __restrict__ out) {
  __shared__ Moments sm[256];
  int t = blockIdx.x;
  double width = (double)(tt.hi(t) - tt.lo(t));
  Moments acc = {0.0, 0.0, 0.0};
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    Moments p = {width, (double)partial[((int64_t)t * rows + r) * 2],
                 (double)partial[((int64_t)t * rows + r) * 2 + 1]};
    acc = merge(acc, p);
  }
  sm[threadIdx.x] = acc;
  __syncthreads();
  for (int o = blockDim.x / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) sm[threadIdx.x] = merge(sm[threadIdx.x], sm[threadIdx.x + o]);
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    double var = sm[0].m2 / (sm[0].n - 1.0);
    out[t] = rnd<DT>((float)sqrt(var));
  }
}

// Running mean of init_std_alpha*std over the first init_from_data training calls, on the
// device (no host read of the counter), then the ranges used by this call are copied out.
template <int DT>
__global__ void ir_update_kernel(void* input_range, void* update_idx, const float* std, int T,
                                 int init_from_data, float init_std_alpha, int do_update,
                                 void* ir_used) {
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    float ir = Elem<DT>::load(input_range, t);
    if (do_update) {
      float idx = Elem<DT>::load(update_idx, t);
      if (idx < (float)init_from_data) {
        float sd = std[t];
        if (sd > 0.0f) {
          float idx1 = rnd<DT>(fadd(idx, 1.0f));
          float v = fdiv(fadd(fmul(ir, idx), fmul(init_std_alpha, sd)), idx1);
          ir = rnd<DT>(v);
          Elem<DT>::store(update_idx, t, idx1);
        }
        ir = fabsf(ir);
        Elem<DT>::store(input_range, t, ir);
      }
    }
    Elem<DT>::store(ir_used, t, ir);
  }
}

// Per-row Gaussian clipping: w[r,:] <- clamp(w[r,:], +-sigma*std(w[r,:])).
template <int DT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
clip_rows_kernel(void* w, int rows, int cols, float sigma) {
  int r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (r >= rows) return;
  float s = 0.0f;
  warp_scan_segment<DT>(w, (int64_t)r * cols, cols, lane, [&](float v) { s += v; });
  float mean = warp_sum(s) / (float)cols;
  float m2 = 0.0f;
  warp_scan_segment<DT>(w, (int64_t)r * cols, cols, lane, [&](float v) {
    float d = v - mean;
    m2 = fmaf(d, d, m2);
  });
  m2 = warp_sum(m2);
  float sd = rnd<DT>(sqrtf(m2 / (float)(cols - 1)));
  float lim = rnd<DT>(fmul(sigma, sd));
  for (int c = lane; c < cols; c += 32) {
    float v = Elem<DT>::load(w, (int64_t)r * cols + c);
    Elem<DT>::store(w, (int64_t)r * cols + c, fminf(fmaxf(v, -lim), lim));
  }
}

template <int DT>
__global__ void clip_all_kernel(void* w, int64_t n, float sigma, const float* std_scalar) {
  float lim = rnd<DT>(fmul(sigma, std_scalar[0]));
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float v = Elem<DT>::load(w, i);
    Elem<DT>::store(w, i, fminf(fmaxf(v, -lim), lim));
  }
}

inline unsigned seg_blocks(int64_t segs) { return (unsigned)((segs + kWarpsPerBlock - 1) / kWarpsPerBlock); }

}  // namespace

#define AL_DISPATCH_DT(dtype, ...)            \
  if ((dtype) == AL_F32) {                    \
    constexpr int DT = kF32;                  \
    __VA_ARGS__;                              \
  } else {                                    \
    constexpr int DT = kBF16;                 \
    __VA_ARGS__;                              \
  }

int launch_abs_max_tiles(int dtype, const void* a, int rows, int K, const TileTable& tt,
                         void* out, cudaStream_t s) {
  ProfScope prof(AL_K_ABS_MAX, s);
  int64_t segs = (int64_t)rows * tt.T;
  AL_DISPATCH_DT(dtype, (abs_max_tiles_kernel<DT><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(a, rows, K, tt, out)));
  return check_launch("abs_max_tiles");
}

int launch_tile_max(int dtype, const void* amax, int rows, const TileTable& tt, int quant_type,
                    float n_states, float* tile_max, int32_t* flags, cudaStream_t s) {
  ProfScope prof(AL_K_TILE_MAX, s);
  AL_DISPATCH_DT(dtype, (tile_max_kernel<DT><<<tt.T, 256, 0, s>>>(amax, rows, quant_type, n_states, tile_max, flags)));
  return check_launch("tile_max");
}

int launch_std_tiles(int dtype, const void* a, int rows, int K, const TileTable& tt, float* out,
                     float* scratch, cudaStream_t s) {
  ProfScope prof(AL_K_STD, s, 2);
  int64_t segs = (int64_t)rows * tt.T;
  AL_DISPATCH_DT(dtype, (segment_moments_kernel<DT><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(a, rows, K, tt, scratch)));
  int rc = check_launch("segment_moments");
  if (rc) return rc;
  AL_DISPATCH_DT(dtype, (merge_moments_kernel<DT><<<tt.T, 256, 0, s>>>(scratch, rows, tt, out)));
  return check_launch("merge_moments");
}

int launch_ir_update(int dtype, void* input_range, void* update_idx, const float* std, int T,
                     int init_from_data, float init_std_alpha, int do_update, void* ir_used,
                     cudaStream_t s) {
  ProfScope prof(AL_K_IR_UPDATE, s);
  AL_DISPATCH_DT(dtype, (ir_update_kernel<DT><<<1, 256, 0, s>>>(input_range, update_idx, std, T, init_from_data, init_std_alpha, do_update, ir_used)));
  return check_launch("ir_update");
}

int launch_clip_weights(int dtype, void* w, int rows, int cols, int clip_type, float sigma,
                        float* scratch, cudaStream_t s) {
  ProfScope prof(AL_K_CLIP, s);
  if (clip_type == AL_CLIP_LAYER_GAUSSIAN_PER_CHANNEL) {
    AL_DISPATCH_DT(dtype, (clip_rows_kernel<DT><<<seg_blocks(rows), kWarpsPerBlock * 32, 0, s>>>(w, rows, cols, sigma)));
    return check_launch("clip_rows");
  }
  TileTable tt;
  tt.T = 1;
  tt.ends[0] = cols;
  // scratch: [0, 2*rows) row partials, then 1 float for the std
  int rc = launch_std_tiles(dtype, w, rows, cols, tt, scratch + 2 * (int64_t)rows, scratch, s);
  if (rc) return rc;
  int64_t n = (int64_t)rows * cols;
  unsigned blocks = (unsigned)((n + 1023) / 1024);
  if (blocks > 148 * 8) blocks = 148 * 8;
  AL_DISPATCH_DT(dtype, (clip_all_kernel<DT><<<blocks, 256, 0, s>>>(w, n, sigma, scratch + 2 * (int64_t)rows)));
  return check_launch("clip_all");
}

}  // namespace al

namespace al {
namespace {

// fast mode, stage 1: (min, max) of every (row, tile) segment; skipped for tiles whose update
// counter already reached init_from_data
template <int DT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
segment_minmax_kernel(const void* __restrict__ a, int rows, int K, TileTable tt,
                      const void* __restrict__ update_idx, int init_from_data,
                      float* __restrict__ partial) {
  const unsigned seg = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (seg >= (unsigned)rows * (unsigned)tt.T) return;
  const int r = (int)(seg / (unsigned)tt.T), t = (int)(seg - (unsigned)r * (unsigned)tt.T);
  if (!(Elem<DT>::load(update_idx, t) < (float)init_from_data)) return;
  int lo = tt.lo(t), len = tt.hi(t) - lo;
  float mn = INFINITY, mx = -INFINITY;
  warp_scan_segment<DT>(a, (int64_t)r * K + lo, len, lane, [&](float v) {
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0) {
    partial[((int64_t)t * rows + r) * 2] = mn;
    partial[((int64_t)t * rows + r) * 2 + 1] = mx;
  }
}

// fast mode, stage 2: one block per tile reduces the row partials and applies the update of
// `apply_input_range_fast` (reference torch_linear.py:386-420), every op rounded to DT
template <int DT>
__global__ void ir_fast_update_kernel(const float* __restrict__ partial, int rows, void* input_range,
                                      void* update_idx, void* x_min, void* x_max, int init_from_data,
                                      float momentum, float one_minus_momentum, int minmax_mode,
                                      int do_update, void* ir_used) {
  __shared__ float s_mn[256], s_mx[256];
  const int t = blockIdx.x;
  float ir = Elem<DT>::load(input_range, t);
  const float idx = Elem<DT>::load(update_idx, t);
  const bool update = do_update && idx < (float)init_from_data;  // uniform over the block
  if (update) {
    float mn = INFINITY, mx = -INFINITY;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
      mn = fminf(mn, partial[((int64_t)t * rows + r) * 2]);
      mx = fmaxf(mx, partial[((int64_t)t * rows + r) * 2 + 1]);
    }
    s_mn[threadIdx.x] = mn;
    s_mx[threadIdx.x] = mx;
    __syncthreads();
    for (int o = blockDim.x / 2; o > 0; o >>= 1) {
      if (threadIdx.x < o) {
        s_mn[threadIdx.x] = fminf(s_mn[threadIdx.x], s_mn[threadIdx.x + o]);
        s_mx[threadIdx.x] = fmaxf(s_mx[threadIdx.x], s_mx[threadIdx.x + o]);
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      const float act_min = s_mn[0], act_max = s_mx[0];
      float xmin = Elem<DT>::load(x_min, t), xmax = Elem<DT>::load(x_max, t);
      if (xmin > -1.1e-5f && xmax < 1.1e-5f) {  // first update: start from the observed range
        xmin = rnd<DT>(fadd(xmin, act_min));
        xmax = rnd<DT>(fadd(xmax, act_max));
      } else if (minmax_mode) {  // act_range_momentum == -1: running extrema
        xmin = fminf(xmin, act_min);
        xmax = fmaxf(xmax, act_max);
      } else {
        xmin = rnd<DT>(fadd(rnd<DT>(fmul(xmin, momentum)), rnd<DT>(fmul(act_min, one_minus_momentum))));
        xmax = rnd<DT>(fadd(rnd<DT>(fmul(xmax, momentum)), rnd<DT>(fmul(act_max, one_minus_momentum))));
      }
      Elem<DT>::store(x_min, t, xmin);
      Elem<DT>::store(x_max, t, xmax);
      Elem<DT>::store(update_idx, t, rnd<DT>(fadd(idx, 1.0f)));
      ir = fmaxf(fabsf(xmin), fabsf(xmax));
      Elem<DT>::store(input_range, t, ir);
    }
  }
  if (threadIdx.x == 0) Elem<DT>::store(ir_used, t, ir);
}

}  // namespace

int launch_ir_fast_update(int dtype, const void* x, int M, int K, const TileTable& tt, void* input_range,
                          void* update_idx, void* x_min, void* x_max, int init_from_data, float momentum,
                          float one_minus_momentum, int minmax_mode, int do_update, float* scratch,
                          void* ir_used, cudaStream_t s) {
  ProfScope prof(AL_K_IR_UPDATE, s, do_update ? 2 : 1);
  if (do_update) {
    int64_t segs = (int64_t)M * tt.T;
    AL_DISPATCH_DT(dtype, (segment_minmax_kernel<DT><<<seg_blocks(segs), kWarpsPerBlock * 32, 0, s>>>(x, M, K, tt, update_idx, init_from_data, scratch)));
    int rc = check_launch("segment_minmax");
    if (rc) return rc;
  }
  AL_DISPATCH_DT(dtype, (ir_fast_update_kernel<DT><<<tt.T, 256, 0, s>>>(scratch, M, input_range, update_idx, x_min, x_max, init_from_data, momentum, one_minus_momentum, minmax_mode, do_update, ir_used)));
  return check_launch("ir_fast_update");
}

}  // namespace al

// ---- per-tile std without a caller-supplied scratch buffer ---------------------------------
//
// al_std_tiles needs 2 floats of scratch per (row, tile) segment for its stage-1 partials and
// asks the caller to bring that buffer.  Some hosts of this library cannot produce one at the
// point where they want the statistic: an inference server that hands each plugin a fixed
// device arena at start-up and forbids later cudaMalloc calls (they synchronise the whole
// device and would stall its other streams), or a calibration hook that runs inside someone
// else's forward pass and owns no allocator at all.  For them the partials live in the array
// below, which is part of the library image: every GPU that loads the library holds these
// 2 MiB until the process exits, whether the entry point is used or not.
//
// All calls on a device share the array and it keeps whatever the previous call left in it.
// Nothing in it has to start at zero: stage 1 overwrites every slot stage 2 reads.  Two calls
// whose kernels overlap on the GPU (different streams, or different host threads on
// different streams) would overwrite each other's partials -- serialise them.
static __device__ __align__(256) float g_std_static_scratch[2 * AL_STD_STATIC_MAX_SEGMENTS];

namespace al {
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
float* g_static_ptr[kMaxDevices] = {};  // device address of the array, per device ordinal
}  // namespace
}  // namespace al

extern "C" int al_std_tiles_static(int32_t dtype, const void* a, int32_t rows, int32_t K,
                                   const int32_t* tile_ends_host, int32_t T, float* out,
                                   void* stream) {
  using namespace al;
  if (dtype != AL_F32 && dtype != AL_BF16) {
    set_error("al_std_tiles_static: unknown dtype %d", dtype);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (!a || !out || !tile_ends_host || rows < 1 || K < 1 || T < 1) {
    set_error("al_std_tiles_static: null pointer or empty matrix");
    return AL_ERR_BAD_ARGUMENT;
  }
  if (T > kMaxTiles || (int64_t)rows * T > (int64_t)AL_STD_STATIC_MAX_SEGMENTS) {
    set_error("al_std_tiles_static: rows*T = %lld exceeds the built-in scratch of %d segments "
              "(use al_std_tiles with your own scratch buffer)",
              (long long)rows * T, (int)AL_STD_STATIC_MAX_SEGMENTS);
    return AL_ERR_TOO_LARGE;
  }
  TileTable tt;
  tt.T = T;
  int prev = 0;
  for (int t = 0; t < T; ++t) {
    if (tile_ends_host[t] <= prev) {
      set_error("al_std_tiles_static: tile ends must be strictly increasing");
      return AL_ERR_BAD_ARGUMENT;
    }
    tt.ends[t] = prev = tile_ends_host[t];
  }
  if (prev != K) {
    set_error("al_std_tiles_static: last tile end %d != K=%d", prev, K);
    return AL_ERR_BAD_ARGUMENT;
  }
  // Set-up, once per device, with that device current: host code cannot use the array's name as
  // a device address, it has to ask the runtime for it.
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("al_std_tiles_static: cannot identify the current device");
    cudaGetLastError();
    return AL_ERR_CUDA;
  }
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_std_static_scratch);
      if (e != cudaSuccess || p == nullptr) {
        set_error("al_std_tiles_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return AL_ERR_CUDA;
      }
      g_static_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_static_ptr[dev];
  }
  return launch_std_tiles(dtype, a, rows, K, tt, out, scratch, (cudaStream_t)stream);
}
