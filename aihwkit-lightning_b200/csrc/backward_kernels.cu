// Element-wise and reduction parts of the backward pass: the bias gradient (column sums of
// the upstream gradient) and, for learned/fixed input ranges, the input-range gradient with
// its decay term followed by the straight-through zeroing of clipped inputs.  Both reduce in
// two stages with a fixed order (no floating-point atomics).
#include "analog_math.cuh"
#include "internal.h"

namespace al {

namespace {

constexpr int kBiasChunks = 256;

// partial[c, n] = sum of g[m, n] over the rows m of chunk c
template <int DT>
__global__ void bias_partial_kernel(const void* __restrict__ g, int M, int N, int rows_per_chunk,
                                    float* __restrict__ partial) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  int c = blockIdx.y;
  if (n >= N) return;
  int m_lo = c * rows_per_chunk, m_hi = min(M, m_lo + rows_per_chunk);
  float s = 0.0f;
  for (int m = m_lo; m < m_hi; ++m) s += Elem<DT>::load(g, (int64_t)m * N + n);
  partial[(int64_t)c * N + n] = s;
}
template <int DT>
__global__ void bias_final_kernel(const float* __restrict__ partial, int chunks, int N,
                                  void* __restrict__ grad_bias) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float s = 0.0f;
  for (int c = 0; c < chunks; ++c) s += partial[(int64_t)c * N + n];
  Elem<DT>::store(grad_bias, n, s);
}

// One warp per (row, tile): partial sums for the range gradient, then zero grad_x where the
// input was clipped and does not sit exactly on the range.
template <int DT>
__global__ void __launch_bounds__(256)
static_ir_partial_kernel(const void* __restrict__ x, const void* __restrict__ ir_used,
                         void* __restrict__ grad_x, int M, int K, TileTable tt,
                         float* __restrict__ partial, int fast_mode) {
  const unsigned seg = blockIdx.x * 8 + (threadIdx.x >> 5);  // rows * T < 2^31 (checked by the host)
  int lane = threadIdx.x & 31;
  if (seg >= (unsigned)M * (unsigned)tt.T) return;
  const int m = (int)(seg / (unsigned)tt.T), t = (int)(seg - (unsigned)m * (unsigned)tt.T);
  int lo = tt.lo(t), len = tt.hi(t) - lo;
  int64_t start = (int64_t)m * K + lo;
  float ir = Elem<DT>::load(ir_used, t);
  float s_up = 0.0f, s_lo = 0.0f, cnt = 0.0f;
  for (int i = lane; i < len; i += 32) {
    float xv = Elem<DT>::load(x, start + i);
    float gv = Elem<DT>::load(grad_x, start + i);
    if (fast_mode) {
      // plain clamp with tensor bounds: the bounds collect the gradient outside [-ir, ir]
      bool up = xv > ir, dn = xv < -ir;
      if (up) s_up += gv;
      if (dn) s_lo += gv;
      if (up || dn) Elem<DT>::store(grad_x, start + i, 0.0f);
      continue;
    }
    bool up = xv >= ir, dn = xv <= -ir;
    if (up) s_up += fminf(gv, 0.0f);
    if (dn) s_lo += fmaxf(gv, 0.0f);
    if (up || dn) {
      cnt += 1.0f;
      if (fabsf(xv) != ir) Elem<DT>::store(grad_x, start + i, 0.0f);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s_up += __shfl_xor_sync(0xffffffffu, s_up, o);
    s_lo += __shfl_xor_sync(0xffffffffu, s_lo, o);
    cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  }
  if (lane == 0) {
    float* p = partial + ((int64_t)t * M + m) * 3;
    p[0] = s_up;
    p[1] = s_lo;
    p[2] = cnt;
  }
}

template <int DT>
__global__ void static_ir_final_kernel(const float* __restrict__ partial,
                                       const void* __restrict__ ir_used, int M, TileTable tt,
                                       float decay, float input_min_percentage,
                                       void* __restrict__ grad_ir, int fast_mode) {
  __shared__ double sm[3][256];
  int t = blockIdx.x;
  double a = 0.0, b = 0.0, c = 0.0;
  for (int m = threadIdx.x; m < M; m += blockDim.x) {
    const float* p = partial + ((int64_t)t * M + m) * 3;
    a += (double)p[0];
    b += (double)p[1];
    c += (double)p[2];
  }
  sm[0][threadIdx.x] = a;
  sm[1][threadIdx.x] = b;
  sm[2][threadIdx.x] = c;
  __syncthreads();
  for (int o = blockDim.x / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      sm[0][threadIdx.x] += sm[0][threadIdx.x + o];
      sm[1][threadIdx.x] += sm[1][threadIdx.x + o];
      sm[2][threadIdx.x] += sm[2][threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    float ir = Elem<DT>::load(ir_used, t);
    float acc = rnd<DT>(fadd(0.0f, rnd<DT>((float)sm[0][0])));
    acc = rnd<DT>(fsub(acc, rnd<DT>((float)sm[1][0])));
    if (fast_mode) {
      Elem<DT>::store(grad_ir, t, acc);
      return;
    }
    acc = rnd<DT>(fmul(acc, ir));
    if (decay > 0.0f) {
      float numel = (float)((double)M * (double)(tt.hi(t) - tt.lo(t)));
      float pct = fsub(1.0f, fdiv((float)sm[2][0], numel));
      float flag = pct > input_min_percentage ? 1.0f : 0.0f;
      float term = rnd<DT>(fmul(rnd<DT>(fmul(decay, ir)), flag));
      acc = rnd<DT>(fadd(acc, term));
    }
    Elem<DT>::store(grad_ir, t, acc);
  }
}

// Backward of the learned per-channel weight range (`quant_utils.py:125-151`, learn_res branch).
// One warp per (channel, tile) segment.  grad_w arrives as the gradient of the clipped /
// discretised weights and leaves as the gradient of the weights themselves (zero outside the
// range); grad_clip[t, n] is the fp32 row sum of (-Q | +Q | round(q) - q) * grad_w * grad_scale
// (below, above, inside the range), rounded to the layer dtype, and divided by n_states when the
// range entered the quantiser as range / n_states.  The reference builds its indicator tensors in
// fp32, so products and the row sum are fp32; the order of the row sum is this warp's.
template <int DT>
__global__ void __launch_bounds__(256)
learn_clip_backward_kernel(const void* __restrict__ w, const void* __restrict__ clip,
                           const int32_t* __restrict__ all_gt1, int N, int K, TileTable tt, int discretize,
                           float n_states, double max_state_d, int no_rounding,
                           void* __restrict__ grad_w, void* __restrict__ grad_clip) {
  const unsigned seg = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (seg >= (unsigned)N * (unsigned)tt.T) return;
  const int n = (int)(seg / (unsigned)tt.T), t = (int)(seg - (unsigned)n * (unsigned)tt.T);
  const int lo = tt.lo(t), len = tt.hi(t) - lo;
  const int64_t start = (int64_t)n * K + lo;
  const float c = Elem<DT>::load(clip, (int64_t)t * N + n);
  float res;
  if (discretize) {
    const float arg = rnd<DT>(fdiv(c, n_states));
    res = all_gt1[t] ? rnd<DT>(fdiv(2.0f, arg)) : rnd<DT>(fmul(2.0f, arg));
  } else {
    res = all_gt1[t] ? rnd<DT>(fdiv(1.0f, c)) : c;
  }
  if (res == 0.0f) res = 1.0f;
  const float resc = res < kTiny ? kTiny : res;
  const float q_max = discretize ? (float)max_state_d : 1.0f;  // as a Python float in the products
  const float q_cmp = rnd<DT>(q_max);                  // as the layer dtype in the comparisons
  const bool skip = !discretize || no_rounding != 0;
  // 1 / sqrt(numel) without rounding, 2 * sqrt(max_state / numel) with it, evaluated in double
  // like the Python expression and then used as an fp32 scalar (`quant_utils.py:103-106`)
  const double numel = (double)N * (double)len;
  const float grad_scale = (float)(skip ? 1.0 / sqrt(numel) : 2.0 * sqrt(max_state_d / numel));
  float acc = 0.0f;
  for (int i = lane; i < len; i += 32) {
    const float wv = Elem<DT>::load(w, start + i);
    const float g = Elem<DT>::load(grad_w, start + i);
    const float q = rnd<DT>(fdiv(wv, resc));
    const bool small = q < -q_cmp, big = q > q_cmp;
    float a;
    if (small) a = -q_max;
    else if (big) a = q_max;
    else a = skip ? 0.0f : rnd<DT>(fadd(-q, rnd<DT>(frint(q))));
    acc = fadd(acc, fmul(fmul(a, g), grad_scale));
    if (small || big) Elem<DT>::store(grad_w, start + i, 0.0f);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc = fadd(acc, __shfl_xor_sync(0xffffffffu, acc, o));
  if (lane == 0) {
    float r = rnd<DT>(acc);
    if (discretize) r = rnd<DT>(fdiv(r, n_states));
    Elem<DT>::store(grad_clip, (int64_t)t * N + n, r);
  }
}

}  // namespace

int launch_learn_clip_backward(int dtype, const void* w, const void* clip, const int32_t* all_gt1, int N,
                               int K, const TileTable& tt, int discretize, float n_states, double max_state,
                               int no_rounding, void* grad_w, void* grad_clip, cudaStream_t s) {
  ProfScope prof(AL_K_CLIP, s);
  int64_t segs = (int64_t)N * tt.T;
  unsigned blocks = (unsigned)((segs + 7) / 8);
  if (dtype == AL_F32)
    learn_clip_backward_kernel<kF32><<<blocks, 256, 0, s>>>(w, clip, all_gt1, N, K, tt, discretize, n_states, max_state, no_rounding, grad_w, grad_clip);
  else
    learn_clip_backward_kernel<kBF16><<<blocks, 256, 0, s>>>(w, clip, all_gt1, N, K, tt, discretize, n_states, max_state, no_rounding, grad_w, grad_clip);
  return check_launch("learn_clip_backward");
}

int launch_bias_grad(int dtype, const void* g, int M, int N, void* grad_bias, float* scratch,
                     cudaStream_t s) {
  ProfScope prof(AL_K_BIAS_GRAD, s, 2);
  int chunks = M < kBiasChunks ? M : kBiasChunks;
  int rows_per_chunk = (M + chunks - 1) / chunks;
  chunks = (M + rows_per_chunk - 1) / rows_per_chunk;
  dim3 grid((N + 127) / 128, chunks);
  if (dtype == AL_F32) {
    bias_partial_kernel<kF32><<<grid, 128, 0, s>>>(g, M, N, rows_per_chunk, scratch);
    bias_final_kernel<kF32><<<(N + 127) / 128, 128, 0, s>>>(scratch, chunks, N, grad_bias);
  } else {
    bias_partial_kernel<kBF16><<<grid, 128, 0, s>>>(g, M, N, rows_per_chunk, scratch);
    bias_final_kernel<kBF16><<<(N + 127) / 128, 128, 0, s>>>(scratch, chunks, N, grad_bias);
  }
  return check_launch("bias_grad");
}

int launch_static_ir_backward(int dtype, const void* x, const void* ir_used, void* grad_x, int M,
                              int K, const TileTable& tt, float decay, float input_min_percentage,
                              void* grad_ir, float* scratch, int fast_mode, cudaStream_t s) {
  ProfScope prof(AL_K_IR_BACKWARD, s, grad_ir ? 2 : 1);
  int64_t segs = (int64_t)M * tt.T;
  unsigned blocks = (unsigned)((segs + 7) / 8);
  if (dtype == AL_F32) {
    static_ir_partial_kernel<kF32><<<blocks, 256, 0, s>>>(x, ir_used, grad_x, M, K, tt, scratch, fast_mode);
    if (grad_ir) static_ir_final_kernel<kF32><<<tt.T, 256, 0, s>>>(scratch, ir_used, M, tt, decay, input_min_percentage, grad_ir, fast_mode);
  } else {
    static_ir_partial_kernel<kBF16><<<blocks, 256, 0, s>>>(x, ir_used, grad_x, M, K, tt, scratch, fast_mode);
    if (grad_ir) static_ir_final_kernel<kBF16><<<tt.T, 256, 0, s>>>(scratch, ir_used, M, tt, decay, input_min_percentage, grad_ir, fast_mode);
  }
  return check_launch("static_ir_backward");
}

}  // namespace al
