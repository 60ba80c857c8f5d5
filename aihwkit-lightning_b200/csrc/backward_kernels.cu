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

}  // namespace

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
