// Operand pre-passes of the fp32 layers on the tensor cores.
//
// The tcgen05 GEMMs multiply bf16 operands and accumulate in fp32.  An fp32 operand v is fed as
// kPlanes bf16 "planes" p0 = RN_bf16(v), p1 = RN_bf16(v - p0), ... (8 significant bits each), and a
// product of two fp32 operands becomes the plane products a0 b0 + a0 b1 + a1 b0.  The DAC codes of
// the inputs are small integers and exact in a single bf16 plane, so the forward GEMM and the
// weight gradient need only the planes of their other operand.
#include "analog_math.cuh"
#include "internal.h"

namespace al {

namespace {

__device__ __forceinline__ void split_planes(float v, uint16_t b[kPlanes]) {
#pragma unroll
  for (int p = 0; p < kPlanes; ++p) {
    b[p] = f32_to_bf16_bits(v);
    v = fsub(v, bf16_bits_to_f32(b[p]));  // exact: the difference fits the remaining significant bits
  }
}

// planes[p][e] of src[e], e < count (count is a multiple of 4 on this path: K % 8 == 0)
__global__ void __launch_bounds__(256)
split_planes_kernel(const float* __restrict__ src, int64_t count4, uint16_t* __restrict__ planes, int64_t plane_stride) {
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < count4; v += (int64_t)gridDim.x * blockDim.x) {
    const float4 x = reinterpret_cast<const float4*>(src)[v];
    const float in[4] = {x.x, x.y, x.z, x.w};
    uint16_t b[kPlanes][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint16_t bp[kPlanes];
      split_planes(in[i], bp);
#pragma unroll
      for (int p = 0; p < kPlanes; ++p) b[p][i] = bp[p];
    }
#pragma unroll
    for (int p = 0; p < kPlanes; ++p)
      *reinterpret_cast<uint2*>(planes + p * plane_stride + v * 4) =
          make_uint2((uint32_t)b[p][0] | ((uint32_t)b[p][1] << 16), (uint32_t)b[p][2] | ((uint32_t)b[p][3] << 16));
  }
}

// Planes of the upstream gradient, one set per analog tile: planes[(t * kPlanes + p)][m][n] of
//   g[m, n] * keep_t(m, n) * scale(m, t)
// keep_t: the ADC clamp mask of tile t (null: all kept); scale: the DAC step of (row m, tile t)
// (ir null: 1), computed from the saved input range with the function the DAC itself used, so that
// scale * code is the de-quantised input the reference multiplies with.  One thread per 4 columns
// (N % 8 == 0), tiles in gridDim.y.
__global__ void __launch_bounds__(256)
split_planes_grad_kernel(const float* __restrict__ g, int M, int N, const uint32_t* __restrict__ keep_mask, int mask_words,
                   const float* __restrict__ ir, int ir_per_row, float inp_res, uint16_t* __restrict__ planes) {
  const int t = blockIdx.y;
  const int64_t quads = (int64_t)M * (N / 4);
  const int64_t plane_stride = (int64_t)M * N;
  uint16_t* out = planes + (int64_t)t * kPlanes * plane_stride;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < quads; v += (int64_t)gridDim.x * blockDim.x) {
    const int m = (int)(v / (N / 4)), n = (int)(v % (N / 4)) * 4;
    const float4 x = reinterpret_cast<const float4*>(g)[v];
    float in[4] = {x.x, x.y, x.z, x.w};
    float scale = 1.0f;
    if (ir != nullptr) scale = quant_step<kF32>(ir[ir_per_row ? (int64_t)t * M + m : t], inp_res);
    uint32_t word = 0xffffffffu;
    if (keep_mask != nullptr) word = keep_mask[((int64_t)t * mask_words + (n >> 5)) * M + m];
    uint16_t b[kPlanes][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float val = ((word >> ((n & 31) + i)) & 1u) ? in[i] : 0.0f;
      if (ir != nullptr) val = fmul(val, scale);
      uint16_t bp[kPlanes];
      split_planes(val, bp);
#pragma unroll
      for (int p = 0; p < kPlanes; ++p) b[p][i] = bp[p];
    }
#pragma unroll
    for (int p = 0; p < kPlanes; ++p)
      *reinterpret_cast<uint2*>(out + p * plane_stride + v * 4) =
          make_uint2((uint32_t)b[p][0] | ((uint32_t)b[p][1] << 16), (uint32_t)b[p][2] | ((uint32_t)b[p][3] << 16));
  }
}

unsigned grid_for(int64_t work_items) {
  const int64_t blocks = (work_items + 255) / 256;
  return (unsigned)(blocks < 148 * 16 ? (blocks < 1 ? 1 : blocks) : 148 * 16);
}

}  // namespace

int launch_split_planes(const float* src, int64_t count, void* planes, cudaStream_t s) {
  ProfScope prof(AL_K_WEIGHT_MODIFY, s);
  split_planes_kernel<<<grid_for(count / 4), 256, 0, s>>>(src, count / 4, static_cast<uint16_t*>(planes), count);
  return check_launch("split_planes");
}

int launch_split_planes_grad(const float* g, int M, int N, const uint32_t* keep_mask, int mask_words, const float* ir,
                       int ir_per_row, float inp_res, int sets, void* planes, cudaStream_t s) {
  ProfScope prof(AL_K_DAC, s);
  dim3 grid(grid_for((int64_t)M * (N / 4)), sets);
  split_planes_grad_kernel<<<grid, 256, 0, s>>>(g, M, N, keep_mask, mask_words, ir, ir_per_row, inp_res,
                                          static_cast<uint16_t*>(planes));
  return check_launch("split_planes_grad");
}

}  // namespace al
