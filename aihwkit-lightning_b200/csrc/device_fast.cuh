// Device-only helpers shared by the streaming kernels and the GEMM epilogues: the fast
// output/weight-noise generator and small bf16x2 utilities.
#pragma once

#include <cuda_bf16.h>

#include "analog_math.cuh"

namespace al {

__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 h) { return *reinterpret_cast<uint32_t*>(&h); }

// Noise generator of the hot kernels: one Philox4x32-7 call (seven rounds are the fewest that
// pass BigCrush in Salmon et al.) yields eight 16-bit uniforms, i.e. four Box-Muller pairs =
// eight standard normals for eight consecutive elements.  Uniforms become floats by bit
// manipulation; logarithm, square root and sine/cosine use the approximate hardware
// functions.  The 16-bit radius limits a draw to |z| < 4.71.
__device__ __forceinline__ void box_muller16(uint32_t ab, float* z0, float* z1) {
  // low 16 bits -> radius, high 16 bits -> angle
  const float u1 = 2.0f - __uint_as_float(0x3f800000u | ((ab & 0xffffu) << 7));  // (0, 1], step 2^-16
  const float u2 = __uint_as_float(0x3f800000u | ((ab >> 16) << 7)) - 1.0f;      // [0, 1)
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(-1.3862943611198906f * __log2f(u1)));
  float s, c;
  __sincosf(6.283185307179586f * u2, &s, &c);
  *z0 = r * c;
  *z1 = r * s;
}
// Eight normals for elements [8*group8, 8*group8 + 8) of stream `stream` of call (seed, offset).
__device__ __forceinline__ void normal8_fast(uint64_t seed, uint64_t offset, uint32_t stream, uint64_t group8,
                                             float z[8]) {
  const Philox4 p = philox4x32<7>((uint32_t)group8, (uint32_t)(group8 >> 32), (uint32_t)offset,
                                  (uint32_t)(offset >> 32) ^ (stream * 0x85EBCA6Bu) ^ 0x5bd1e995u,
                                  (uint32_t)seed, (uint32_t)(seed >> 32));
#pragma unroll
  for (int i = 0; i < 4; ++i) box_muller16(p.v[i], &z[2 * i], &z[2 * i + 1]);
}

// round-half-even with two additions, without a range guard: only for |x| < 2^22, which holds
// for DAC codes (|x| <= input range  =>  |x / step| <= inp_res / 2 + 1)
__device__ __forceinline__ float rint_small(float x) {
  return __fsub_rn(__fadd_rn(x, 12582912.0f), 12582912.0f);
}

}  // namespace al
