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
  // low 16 bits -> radius, high 16 bits -> angle.  0x4b000000 | k is the float 2^23 + k, so a
  // byte permute turns a 16-bit integer k into the float f = 2^23 + k without a conversion; the
  // 2^23 is folded into the constant of the multiply-add that consumes f.
  const float f1 = __uint_as_float(__byte_perm(ab, 0x4b000000u, 0x7610));  // 2^23 + (0 .. 65535)
  const float f2 = __uint_as_float(__byte_perm(ab, 0x4b000000u, 0x7632));
  const float u1 = fmaf(f1, -1.52587890625e-05f, 129.0f);  // 1 - k1 / 65536, exact: (0, 1], never denormal
  // .ftz forms: single MUFU instructions (the default forms wrap them in denormal handling)
  float lg, r, s, c;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(lg) : "f"(u1));
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(-1.3862943611198906f * lg));
  // 2*pi * k2 / 65536 up to a constant offset below 4e-5 (the rounding of the folded constant),
  // which a uniform angle does not notice
  const float phi = fmaf(f2, 9.587379924285257e-05f, -804.24771931898713f);
  asm("sin.approx.ftz.f32 %0, %1;" : "=f"(s) : "f"(phi));
  asm("cos.approx.ftz.f32 %0, %1;" : "=f"(c) : "f"(phi));
  *z0 = r * c;
  *z1 = r * s;
}
// Philox4x32 with the two 32x32 -> 64 bit products written as 64-bit multiplies (one wide
// multiply-add instruction each instead of separate high and low halves).
template <int ROUNDS>
__device__ __forceinline__ Philox4 philox4x32_wide(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                                   uint32_t k1) {
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ (k0 + (uint32_t)r * 0x9E3779B9u);
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ (k1 + (uint32_t)r * 0xBB67AE85u);
    c0 = n0; c1 = (uint32_t)p1; c2 = n2; c3 = (uint32_t)p0;
  }
  Philox4 out;
  out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}
// The same generator with everything that depends only on (seed, offset, stream) prepared on the
// host: the fourteen round keys and the two fixed counter words.  Passed inside a kernel's
// parameter block they are constant-bank operands of the XORs, so a round costs two wide
// multiplies and two three-input XORs.
struct NoiseKeys {
  uint32_t k[14];  // k[2r] = seed.lo + r * 0x9E3779B9, k[2r+1] = seed.hi + r * 0xBB67AE85
  uint32_t c2, c3;
  // A call counter in device memory (null: none) that is added to `offset` when the kernel starts, so
  // that a captured CUDA graph draws fresh noise on every replay: see noise_counter().
  const uint64_t* offset_base;
  uint64_t offset;
  uint32_t mix;  // what the stream contributes to c3
};
__host__ __device__ inline NoiseKeys make_noise_keys(uint64_t seed, uint64_t offset, uint32_t stream,
                                                     const uint64_t* offset_base = nullptr) {
  NoiseKeys nk;
  nk.offset_base = offset_base;
  nk.offset = offset;
  nk.mix = (stream * 0x85EBCA6Bu) ^ 0x5bd1e995u;
  for (int r = 0; r < 7; ++r) {
    nk.k[2 * r] = (uint32_t)seed + (uint32_t)r * 0x9E3779B9u;
    nk.k[2 * r + 1] = (uint32_t)(seed >> 32) + (uint32_t)r * 0xBB67AE85u;
  }
  nk.c2 = (uint32_t)offset;
  nk.c3 = (uint32_t)(offset >> 32) ^ (stream * 0x85EBCA6Bu) ^ 0x5bd1e995u;
  return nk;
}
// The two counter words the call contributes: the host's values, or (offset + *offset_base) when
// the caller keeps a counter on the device.  Read once per thread; the keys stay in the constant bank.
struct NoiseCounter {
  uint32_t c2, c3;
};
__device__ __forceinline__ NoiseCounter noise_counter(const NoiseKeys& nk) {
  NoiseCounter c = {nk.c2, nk.c3};
  if (nk.offset_base != nullptr) {
    const uint64_t off = nk.offset + *nk.offset_base;
    c.c2 = (uint32_t)off;
    c.c3 = (uint32_t)(off >> 32) ^ nk.mix;
  }
  return c;
}
// same values as normal8_fast(seed, offset, stream, group8, z)
__device__ __forceinline__ void normal8_keyed(const NoiseKeys& nk, const NoiseCounter& ctr, uint64_t group8, float z[8]) {
  uint32_t c0 = (uint32_t)group8, c1 = (uint32_t)(group8 >> 32), c2 = ctr.c2, c3 = ctr.c3;
#pragma unroll
  for (int r = 0; r < 7; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ nk.k[2 * r];
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ nk.k[2 * r + 1];
    c0 = n0; c1 = (uint32_t)p1; c2 = n2; c3 = (uint32_t)p0;
  }
  box_muller16(c0, &z[0], &z[1]);
  box_muller16(c1, &z[2], &z[3]);
  box_muller16(c2, &z[4], &z[5]);
  box_muller16(c3, &z[6], &z[7]);
}
// The four 32-bit words behind normal8_keyed(nk, group8, .): word i feeds elements 2i and 2i + 1.
__device__ __forceinline__ void philox7_keyed(const NoiseKeys& nk, const NoiseCounter& ctr, uint64_t group8, uint32_t w[4]) {
  uint32_t c0 = (uint32_t)group8, c1 = (uint32_t)(group8 >> 32), c2 = ctr.c2, c3 = ctr.c3;
#pragma unroll
  for (int r = 0; r < 7; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ nk.k[2 * r];
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ nk.k[2 * r + 1];
    c0 = n0; c1 = (uint32_t)p1; c2 = n2; c3 = (uint32_t)p0;
  }
  w[0] = c0; w[1] = c1; w[2] = c2; w[3] = c3;
}
// acc + s * (z0, z1) for the two normals of box_muller16(ab, ..) and a scale s, in packed bf16:
// `neg_c` = -2 ln(2) s^2 goes under the square root, so the radius comes out scaled; the unit vector
// (cos, sin) and the radius are rounded to bf16 and meet the accumulator in one fused multiply-add.
__device__ __forceinline__ __nv_bfloat162 box_muller16_fma(uint32_t ab, float neg_c, __nv_bfloat162 acc) {
  const float f1 = __uint_as_float(__byte_perm(ab, 0x4b000000u, 0x7610));
  const float f2 = __uint_as_float(__byte_perm(ab, 0x4b000000u, 0x7632));
  const float u1 = fmaf(f1, -1.52587890625e-05f, 129.0f);
  float lg, r, s, c;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(lg) : "f"(u1));
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(neg_c * lg));
  const float phi = fmaf(f2, 9.587379924285257e-05f, -804.24771931898713f);
  asm("sin.approx.ftz.f32 %0, %1;" : "=f"(s) : "f"(phi));
  asm("cos.approx.ftz.f32 %0, %1;" : "=f"(c) : "f"(phi));
  return __hfma2(__floats2bfloat162_rn(c, s), __floats2bfloat162_rn(r, r), acc);
}
constexpr float kNegTwoLn2 = -1.3862943611198906f;

// ADC quantisation of a bf16x2 pair, all in packed bf16 arithmetic.
//   code = rint(RN_bf16(o / stepc)),  result = RN_bf16(code * step)
// Division: q0 = RN(o y), r = fma(-stepc, q0, o), q = fma(r, y, q0) with y = RN_bf16(1 / stepc) is
// the correctly rounded bf16 quotient for every pair of 8-bit significands (checked exhaustively
// on the host).  Rounding to an integer: (q + s) - s with s = 128 carrying the sign of o -- sums
// with a magnitude in [128, 256) have a spacing of 1 in bf16 and round half to even like rint.
// Exact for |q| < 128 (a zero code comes out as +0 whatever the sign of o); a larger |q| yields
// some value of magnitude >= 128, which is all the caller needs when every code beyond +-127 ends
// on the clamp (see adc_codes_fit_a_byte).
__device__ __forceinline__ __nv_bfloat162 adc_bf16x2(__nv_bfloat162 o, __nv_bfloat162 y, __nv_bfloat162 neg_stepc,
                                                     __nv_bfloat162 step) {
  const __nv_bfloat162 q0 = __hmul2_rn(o, y);
  const __nv_bfloat162 r = __hfma2(neg_stepc, q0, o);
  const __nv_bfloat162 q = __hfma2(r, y, q0);
  const __nv_bfloat162 s128 = as_bf162((as_u32(o) & 0x80008000u) | 0x43004300u);
  const __nv_bfloat162 code = __hsub2_rn(__hadd2_rn(q, s128), s128);
  return __hmul2_rn(code, step);
}

// Eight normals for elements [8*group8, 8*group8 + 8) of stream `stream` of call (seed, offset).
__device__ __forceinline__ void normal8_fast(uint64_t seed, uint64_t offset, uint32_t stream, uint64_t group8,
                                             float z[8]) {
  const Philox4 p = philox4x32_wide<7>((uint32_t)group8, (uint32_t)(group8 >> 32), (uint32_t)offset,
                                       (uint32_t)(offset >> 32) ^ (stream * 0x85EBCA6Bu) ^ 0x5bd1e995u,
                                       (uint32_t)seed, (uint32_t)(seed >> 32));
#pragma unroll
  for (int i = 0; i < 4; ++i) box_muller16(p.v[i], &z[2 * i], &z[2 * i + 1]);
}

// Two fp32 lanes in one 64-bit register: sm_100 executes fma / mul / add on such a pair as one
// instruction with the same per-lane IEEE rounding as the scalar forms.
__device__ __forceinline__ uint64_t f32x2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f32x2_unpack(uint64_t v, float* lo, float* hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(*lo), "=f"(*hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f32x2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f32x2_mul(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t f32x2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// fdiv_rcp on both lanes: y2 = (1/b, 1/b) correctly rounded, nb2 = (-b, -b)
__device__ __forceinline__ uint64_t f32x2_div_rcp(uint64_t a, uint64_t nb2, uint64_t y2) {
  const uint64_t q = f32x2_mul(a, y2);
  return f32x2_fma(f32x2_fma(q, nb2, a), y2, q);
}

// round-half-even with two additions, without a range guard: only for |x| < 2^22, which holds
// for DAC codes (|x| <= input range  =>  |x / step| <= inp_res / 2 + 1)
__device__ __forceinline__ float rint_small(float x) {
  return __fsub_rn(__fadd_rn(x, 12582912.0f), 12582912.0f);
}

}  // namespace al
