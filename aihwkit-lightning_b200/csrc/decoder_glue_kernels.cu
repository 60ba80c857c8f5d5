// Element-wise operators of a decoder layer that sit between the analog linear layers: the gated
// activation behind the fused gate / up projection and the rotary embedding behind the fused qkv
// projection.  Both read a slice-structured activation ([.., 2 D] halves, [.., 3, H, hd] thirds); as
// chains of PyTorch element-wise kernels over strided views they run at about 1 TB/s and cost more
// than the attention itself, so each direction is one pass here: 16-byte vectors, fp32 arithmetic,
// one rounding to the tensor's dtype per result.  HBM-bound: bytes = every operand once.
#include <cuda_bf16.h>

#include "analog_math.cuh"
#include "internal.h"

namespace al {

namespace {

// eight consecutive elements (bf16) or four (fp32) of a row: one 16-byte vector
template <int DT>
struct Vec {
  static constexpr int N = DT == kF32 ? 4 : 8;
  __device__ static void load(const void* p, int64_t idx, float out[N]) {
    if (DT == kF32) {
      const float4 f = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx);
      out[0] = f.x; out[1] = f.y; out[2] = f.z; out[3] = f.w;
    } else {
      const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p) + idx);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    }
  }
  __device__ static void store(void* p, int64_t idx, const float v[N]) {
    if (DT == kF32) {
      *reinterpret_cast<float4*>(static_cast<float*>(p) + idx) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[i] = (uint32_t)f32_to_bf16_bits(v[2 * i]) | ((uint32_t)f32_to_bf16_bits(v[2 * i + 1]) << 16);
      *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
};

__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + __expf(-x)); }

// out[m, d] = silu(gu[m, d]) * gu[m, D + d]
template <int DT>
__global__ void __launch_bounds__(256)
swiglu_forward_kernel(const void* __restrict__ gu, int64_t rows, int D, void* __restrict__ out) {
  constexpr int VN = Vec<DT>::N;
  const int vec_per_row = D / VN;
  const int64_t total = rows * vec_per_row;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = v / vec_per_row;
    const int d = (int)(v - m * vec_per_row) * VN;
    float gate[VN], up[VN], o[VN];
    Vec<DT>::load(gu, m * 2 * D + d, gate);
    Vec<DT>::load(gu, m * 2 * D + D + d, up);
#pragma unroll
    for (int i = 0; i < VN; ++i) o[i] = gate[i] * sigmoidf(gate[i]) * up[i];
    Vec<DT>::store(out, m * D + d, o);
  }
}

// dgu[m, d] = g * up * silu'(gate),  dgu[m, D + d] = g * silu(gate)
template <int DT>
__global__ void __launch_bounds__(256)
swiglu_backward_kernel(const void* __restrict__ gu, const void* __restrict__ g, int64_t rows, int D,
                       void* __restrict__ dgu) {
  constexpr int VN = Vec<DT>::N;
  const int vec_per_row = D / VN;
  const int64_t total = rows * vec_per_row;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = v / vec_per_row;
    const int d = (int)(v - m * vec_per_row) * VN;
    float gate[VN], up[VN], go[VN], dgate[VN], dup[VN];
    Vec<DT>::load(gu, m * 2 * D + d, gate);
    Vec<DT>::load(gu, m * 2 * D + D + d, up);
    Vec<DT>::load(g, m * D + d, go);
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      const float s = sigmoidf(gate[i]);
      dup[i] = go[i] * gate[i] * s;
      dgate[i] = go[i] * up[i] * s * (1.0f + gate[i] * (1.0f - s));
    }
    Vec<DT>::store(dgu, m * 2 * D + d, dgate);
    Vec<DT>::store(dgu, m * 2 * D + D + d, dup);
  }
}

// Rotary embedding of the q and k thirds of qkv [B*S rows][3][H][hd] (position = row % S):
//   (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin) over the two halves of hd, angle table [S][hd / 2]
// forward: reads qkv, writes q, k, v [rows][H][hd] each; backward (INVERSE: the transposed rotation): reads
// the three gradients, writes dqkv.
template <int DT, bool INVERSE>
__global__ void __launch_bounds__(256)
rotary_kernel(const void* __restrict__ in_q, const void* __restrict__ in_k, const void* __restrict__ in_v,
              int64_t in_row_stride, const float* __restrict__ cos_t,
              const float* __restrict__ sin_t, int64_t rows, int S, int H, int hd, void* __restrict__ out_q,
              void* __restrict__ out_k, void* __restrict__ out_v, int64_t out_row_stride) {
  constexpr int VN = Vec<DT>::N;
  const int half = hd / 2;
  const int vec_per_head = half / VN;  // vectors of the first half of one head
  const int64_t total = rows * H * vec_per_head;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = v / ((int64_t)H * vec_per_head);
    const int rem = (int)(v - row * H * vec_per_head);
    const int h = rem / vec_per_head, e = (rem - h * vec_per_head) * VN;
    const int pos = (int)(row % S);
    float c[VN], s[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      c[i] = cos_t[(int64_t)pos * half + e + i];
      s[i] = sin_t[(int64_t)pos * half + e + i];
      if (INVERSE) s[i] = -s[i];
    }
    const int64_t in_off = row * in_row_stride + (int64_t)h * hd + e;
    const int64_t out_off = row * out_row_stride + (int64_t)h * hd + e;
    const void* ins[2] = {in_q, in_k};
    void* outs[2] = {out_q, out_k};
#pragma unroll
    for (int part = 0; part < 2; ++part) {
      float x1[VN], x2[VN], y1[VN], y2[VN];
      Vec<DT>::load(ins[part], in_off, x1);
      Vec<DT>::load(ins[part], in_off + half, x2);
#pragma unroll
      for (int i = 0; i < VN; ++i) {
        y1[i] = x1[i] * c[i] - x2[i] * s[i];
        y2[i] = x2[i] * c[i] + x1[i] * s[i];
      }
      Vec<DT>::store(outs[part], out_off, y1);
      Vec<DT>::store(outs[part], out_off + half, y2);
    }
    float a[VN], b[VN];
    Vec<DT>::load(in_v, in_off, a);
    Vec<DT>::load(in_v, in_off + half, b);
    Vec<DT>::store(out_v, out_off, a);
    Vec<DT>::store(out_v, out_off + half, b);
  }
}

inline unsigned glue_grid(int64_t work) {
  const int64_t blocks = (work + 255) / 256;
  return (unsigned)(blocks < 1 ? 1 : blocks < 148 * 16 ? blocks : 148 * 16);
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

}  // namespace al

using namespace al;

extern "C" {

int al_swiglu_forward(int32_t dtype, const void* gate_up, int64_t rows, int32_t width, void* out, void* stream) {
  const int vn = dtype == AL_F32 ? 4 : 8;
  if ((dtype != AL_F32 && dtype != AL_BF16) || !gate_up || !out || rows < 0 || width < vn || width % vn != 0 ||
      !aligned16(gate_up) || !aligned16(out)) {
    set_error("al_swiglu_forward: dtype, pointers (16-byte aligned) or width (a multiple of %d)", vn);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (rows == 0) return AL_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = glue_grid(rows * (width / vn));
  if (dtype == AL_F32) swiglu_forward_kernel<kF32><<<grid, 256, 0, s>>>(gate_up, rows, width, out);
  else swiglu_forward_kernel<kBF16><<<grid, 256, 0, s>>>(gate_up, rows, width, out);
  return check_launch("swiglu_forward");
}

int al_swiglu_backward(int32_t dtype, const void* gate_up, const void* grad_out, int64_t rows, int32_t width,
                       void* grad_gate_up, void* stream) {
  const int vn = dtype == AL_F32 ? 4 : 8;
  if ((dtype != AL_F32 && dtype != AL_BF16) || !gate_up || !grad_out || !grad_gate_up || rows < 0 || width < vn ||
      width % vn != 0 || !aligned16(gate_up) || !aligned16(grad_out) || !aligned16(grad_gate_up)) {
    set_error("al_swiglu_backward: dtype, pointers (16-byte aligned) or width (a multiple of %d)", vn);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (rows == 0) return AL_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = glue_grid(rows * (width / vn));
  if (dtype == AL_F32) swiglu_backward_kernel<kF32><<<grid, 256, 0, s>>>(gate_up, grad_out, rows, width, grad_gate_up);
  else swiglu_backward_kernel<kBF16><<<grid, 256, 0, s>>>(gate_up, grad_out, rows, width, grad_gate_up);
  return check_launch("swiglu_backward");
}

int al_rotary_qkv(int32_t dtype, int32_t inverse, const void* in_q, const void* in_k, const void* in_v,
                  int64_t in_row_stride, const float* cos_table, const float* sin_table, int64_t rows, int32_t seq_len,
                  int32_t heads, int32_t head_dim, void* out_q, void* out_k, void* out_v, int64_t out_row_stride,
                  void* stream) {
  const int vn = dtype == AL_F32 ? 4 : 8;
  const int es = dtype == AL_F32 ? 4 : 2;
  if ((dtype != AL_F32 && dtype != AL_BF16) || !in_q || !in_k || !in_v || !out_q || !out_k || !out_v || !cos_table ||
      !sin_table || rows < 0 || seq_len < 1 || heads < 1 || head_dim < 2 * vn || (head_dim / 2) % vn != 0 ||
      head_dim % 2 != 0 || (in_row_stride * es) % 16 != 0 || (out_row_stride * es) % 16 != 0 || !aligned16(in_q) ||
      !aligned16(in_k) || !aligned16(in_v) || !aligned16(out_q) || !aligned16(out_k) || !aligned16(out_v)) {
    set_error("al_rotary_qkv: dtype, pointers and row strides (16-byte aligned) or head_dim (half of it a multiple of %d)",
              vn);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (rows == 0) return AL_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = glue_grid(rows * heads * (head_dim / 2 / vn));
#define AL_ROTARY(DT_, INV_)                                                                                          \
  rotary_kernel<DT_, INV_><<<grid, 256, 0, s>>>(in_q, in_k, in_v, in_row_stride, cos_table, sin_table, rows, seq_len, \
                                                heads, head_dim, out_q, out_k, out_v, out_row_stride)
  if (dtype == AL_F32) {
    if (inverse) AL_ROTARY(kF32, true);
    else AL_ROTARY(kF32, false);
  } else {
    if (inverse) AL_ROTARY(kBF16, true);
    else AL_ROTARY(kBF16, false);
  }
#undef AL_ROTARY
  return check_launch("rotary_qkv");
}

}  // extern "C"
