// Element-wise arithmetic of the analog linear path, usable from device code and (for the
// CPU-side checks of this arithmetic) from plain host C++.
//
// Every function reproduces the rounding behaviour of the reference's torch backend: an op on
// bf16 tensors is evaluated in fp32 and rounded to bf16 once, a Python scalar operand stays
// fp32, divisions are true IEEE divisions and rounding to integers is half-to-even.  The
// device build uses the *_rn intrinsics so that nvcc never contracts a multiply and an add
// into an FMA; the host build must be compiled with -ffp-contract=off for the same reason.
#pragma once

#include <stdint.h>
#include <math.h>
#include <string.h>

#if defined(__CUDACC__)
#include <cuda_bf16.h>
#define AL_HD __host__ __device__ __forceinline__
#else
#define AL_HD inline
#endif

namespace al {

constexpr int kF32 = 0;
constexpr int kBF16 = 1;
constexpr float kTiny = 1.17549435e-38f;  // finfo(float32).tiny == finfo(bfloat16).tiny

// ---- exact (never contracted) fp32 primitives -------------------------------------------
AL_HD float fmul(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  return a * b;
#endif
}
AL_HD float fadd(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fadd_rn(a, b);
#else
  return a + b;
#endif
}
AL_HD float fsub(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fsub_rn(a, b);
#else
  return a - b;
#endif
}
AL_HD float fdiv(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fdiv_rn(a, b);
#else
  return a / b;
#endif
}
AL_HD float frint(float a) {  // half-to-even, like torch.round
#if defined(__CUDA_ARCH__)
  return rintf(a);
#else
  return nearbyintf(a);
#endif
}

// ---- bf16 <-> fp32 ----------------------------------------------------------------------
AL_HD uint32_t f2u(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
#endif
}
AL_HD float u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}
AL_HD uint16_t f32_to_bf16_bits(float f) {  // round to nearest even
#if defined(__CUDA_ARCH__)
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
#else
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);  // quiet NaN
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
#endif
}
AL_HD float bf16_bits_to_f32(uint16_t b) { return u2f(((uint32_t)b) << 16); }
AL_HD float round_bf16(float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); }

// Round an fp32 intermediate to the tensor dtype DT.
template <int DT>
AL_HD float rnd(float v) {
  if (DT == kBF16) return round_bf16(v);
  return v;
}

// ---- element access by dtype ------------------------------------------------------------
template <int DT>
struct Elem;
template <>
struct Elem<kF32> {
  typedef float type;
  static AL_HD float load(const void* p, int64_t i) { return ((const float*)p)[i]; }
  static AL_HD void store(void* p, int64_t i, float v) { ((float*)p)[i] = v; }
};
template <>
struct Elem<kBF16> {
  typedef uint16_t type;
  static AL_HD float load(const void* p, int64_t i) {
    return bf16_bits_to_f32(((const uint16_t*)p)[i]);
  }
  static AL_HD void store(void* p, int64_t i, float v) {
    ((uint16_t*)p)[i] = f32_to_bf16_bits(v);
  }
};

// ---- uniform quantiser ------------------------------------------------------------------
// step = 2*bound/res for res > 1, 2*bound*res otherwise; each op rounded to DT.
template <int DT>
AL_HD float quant_step(float bound, float res) {
  float alpha = rnd<DT>(fmul(2.0f, bound));
  return res > 1.0f ? rnd<DT>(fdiv(alpha, res)) : rnd<DT>(fmul(alpha, res));
}

// code = rint(v / max(step, tiny)), as a float holding an integer (unless no_rounding).
template <int DT>
AL_HD float quant_code(float v, float step, bool no_rounding) {
  float c = rnd<DT>(fdiv(v, step < kTiny ? kTiny : step));
  return no_rounding ? c : frint(c);
}

// DAC of one input element.  `ir` is the input range of the element's (row, tile).
// static_clamp: clamp to +-ir first (learned / fixed range); dynamic ranges need no clamp.
template <int DT>
AL_HD float dac(float x, float ir, float inp_res, bool static_clamp, bool no_rounding,
                float* code_out) {
  if (static_clamp) x = fminf(fmaxf(x, -ir), ir);
  if (!(inp_res > 0.0f)) {
    if (code_out) *code_out = x;
    return x;
  }
  float step = quant_step<DT>(ir, inp_res);
  float c = quant_code<DT>(x, step, no_rounding);
  if (code_out) *code_out = c;
  return rnd<DT>(fmul(c, step));
}

// ---- same results, fewer instructions: what the streaming kernels actually execute --------
// Rounding to bf16 precision with integer adds (the cvt instruction is quarter rate).  Equal to
// rnd<DT> for every finite value and for infinities; NaN inputs must be patched by the caller.
template <int DT>
AL_HD float rnd_int(float v) {
  if (DT == kBF16) {
    uint32_t u = f2u(v);
    u += 0x7fffu + ((u >> 16) & 1u);
    return u2f(u & 0xffff0000u);
  }
  return v;
}
AL_HD float ffma(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
  return __fmaf_rn(a, b, c);
#else
  return fmaf(a, b, c);
#endif
}
AL_HD float frcp(float b) {
#if defined(__CUDA_ARCH__)
  return __frcp_rn(b);
#else
  return 1.0f / b;
#endif
}
// a / b from y = RN(1/b): q = RN(a*y), r = a - b*q (exact in one FMA), RN(q + r*y).  With a
// correctly rounded reciprocal this is the correctly rounded quotient (Markstein), as long as
// no intermediate over/underflows; the CPU test-suite compares it with the true division.
AL_HD float fdiv_rcp(float a, float b, float y) {
  float q = fmul(a, y);
  return ffma(ffma(-q, b, a), y, q);
}
// round-half-even to an integer with two additions, exact for |x| < 2^22
AL_HD float frint_add(float x) {
  float r = fsub(fadd(x, 12582912.0f), 12582912.0f);
  return fabsf(x) < 4194304.0f ? r : frint(x);
}

// ---- the tensor-core forward's ADC in bf16 arithmetic, one lane, on values held in floats ------
// One bf16 operation = the exact result rounded to bf16 once (what mul / fma.rn.bf16x2 do per lane).
AL_HD float bf16_mul(float a, float b) { return round_bf16(fmul(a, b)); }  // 16-bit product: exact in fp32
AL_HD float bf16_add(float a, float b) { return round_bf16((float)((double)a + (double)b)); }
AL_HD float bf16_fma(float a, float b, float c) { return round_bf16((float)((double)a * (double)b + (double)c)); }
// code of adc_bf16x2 (device_fast.cuh): Markstein division from y = RN_bf16(1 / stepc), then
// (q + s) - s with s = 128 carrying the sign of o.
AL_HD float adc_code_bf16(float o, float stepc, float y) {
  const float q0 = bf16_mul(o, y);
  const float r = bf16_fma(-stepc, q0, o);
  const float q = bf16_fma(r, y, q0);
  const float s128 = u2f((f2u(o) & 0x80000000u) | 0x43000000u);
  return bf16_add(bf16_add(q, s128), -s128);
}
// Whether every ADC code beyond +-127 ends on the clamp: 128 * step > bound for every bound, with
// step = RN_bf16(2 bound / states) >= (2 bound / states)(1 - 2^-8), holds for states < 255.
AL_HD bool adc_codes_fit_a_byte(float out_res, bool has_bound) {
  const float states = out_res > 1.0f ? out_res : (out_res > 0.0f ? 1.0f / out_res : 0.0f);
  return has_bound && states > 0.0f && states < 255.0f;
}

// Quantiser constants of one (row, tile) segment, hoisted out of the element loop.
struct QuantSeg {
  float bound;   // clamp range (input range for the DAC)
  float step;    // quantisation step (0 for an all-zero row)
  float stepc;   // max(step, tiny): the divisor
  float rstep;   // RN(1 / stepc)
  int clampit;   // clamp to +-bound first
  int quantise;  // resolution given
  int no_rounding;
};
template <int DT>
AL_HD QuantSeg dac_prepare(float ir, float inp_res, bool static_clamp, bool no_rounding) {
  QuantSeg q;
  q.bound = ir;
  q.clampit = static_clamp ? 1 : 0;
  q.quantise = inp_res > 0.0f ? 1 : 0;
  q.no_rounding = no_rounding ? 1 : 0;
  q.step = q.quantise ? quant_step<DT>(ir, inp_res) : 1.0f;
  q.stepc = q.step < kTiny ? kTiny : q.step;
  q.rstep = frcp(q.stepc);
  return q;
}
// Same value as dac<DT>(x, ...) for every non-NaN x; NaN passes through unchanged.
template <int DT>
AL_HD float dac_apply(const QuantSeg& q, float x, float* code_out) {
  float v = x;
  if (q.clampit) v = fminf(fmaxf(v, -q.bound), q.bound);
  float c = v;
  if (q.quantise) {
    c = rnd_int<DT>(fdiv_rcp(v, q.stepc, q.rstep));
    if (!q.no_rounding) c = frint_add(c);
    v = rnd_int<DT>(fmul(c, q.step));
  }
  if (x != x) { v = x; c = x; }
  if (code_out) *code_out = c;
  return v;
}

// Weight discretisation of one element.  `scale` = tile abs-max or channel abs-max (already a
// DT value), n_states = float(max(res, 1/res)) and max_state = float(n_states/2) evaluated in
// double by the host like the Python reference does, all_gt1 = whether every scale/n_states
// of the tile (scalar: the one) exceeds 1, which flips the reference between alpha/res and
// alpha*res.
template <int DT>
AL_HD float discretize(float w, float scale, float n_states, float max_state, bool all_gt1,
                       bool no_rounding) {
  float res = rnd<DT>(fdiv(scale, n_states));
  res = all_gt1 ? rnd<DT>(fdiv(2.0f, res)) : rnd<DT>(fmul(2.0f, res));
  if (res == 0.0f) res = 1.0f;
  float v = rnd<DT>(fdiv(w, res < kTiny ? kTiny : res));
  float ms = rnd<DT>(max_state);
  v = fminf(fmaxf(v, -ms), ms);
  if (!no_rounding) v = frint(v);
  return rnd<DT>(fmul(v, res));
}
template <int DT>
AL_HD bool discretize_scale_gt1(float scale, float n_states) {
  return rnd<DT>(fdiv(scale, n_states)) > 1.0f;
}

// Weight-modifier constants of one (channel, tile) segment, hoisted out of the element loop.
struct WeightSeg {
  int quant, noise, no_rounding;
  float res, resc, rres, max_state;  // discretiser: step, max(step, tiny), RN(1/.), clamp
  float amp;                         // noise amplitude rnd(std_dev * scale)
};
template <int DT>
AL_HD WeightSeg weight_prepare(int quant_type, float q_scale, float n_states, float max_state,
                               bool all_gt1, int noise_type, float std_dev, float n_scale,
                               bool no_rounding) {
  WeightSeg s;
  s.quant = quant_type != 0;
  s.noise = noise_type != 0;
  s.no_rounding = no_rounding ? 1 : 0;
  s.res = 1.0f;
  if (s.quant) {
    float res = rnd<DT>(fdiv(q_scale, n_states));
    res = all_gt1 ? rnd<DT>(fdiv(2.0f, res)) : rnd<DT>(fmul(2.0f, res));
    if (res == 0.0f) res = 1.0f;
    s.res = res;
  }
  s.resc = s.res < kTiny ? kTiny : s.res;
  s.rres = frcp(s.resc);
  s.max_state = rnd<DT>(max_state);
  s.amp = rnd<DT>(fmul(std_dev, n_scale));
  return s;
}
// LEARNABLE_PER_CHANNEL clipping without discretisation (`quant_utils.py:190-197`): the quantiser
// is entered with res = the learned range as a tensor, bound = 0.5 (alpha = 1), max state 1 and
// no rounding, i.e. w / range, clamp to +-1, times range -- with the same `(res > 1).all()`
// switch and zero guard as the discretiser.
template <int DT>
AL_HD WeightSeg weight_prepare_learn_clamp(float clip, bool all_gt1, int noise_type, float std_dev,
                                           float n_scale) {
  WeightSeg s;
  s.quant = 1;
  s.noise = noise_type != 0;
  s.no_rounding = 1;
  float res = all_gt1 ? rnd<DT>(fdiv(1.0f, clip)) : clip;
  if (res == 0.0f) res = 1.0f;
  s.res = res;
  s.resc = s.res < kTiny ? kTiny : s.res;
  s.rres = frcp(s.resc);
  s.max_state = 1.0f;
  s.amp = rnd<DT>(fmul(std_dev, n_scale));
  return s;
}
// Same value as discretize<DT> followed by add_weight_noise<DT> for non-NaN weights.
template <int DT>
AL_HD float weight_apply(const WeightSeg& s, float w, float xi) {
  float v = w;
  if (s.quant) {
    v = rnd_int<DT>(fdiv_rcp(v, s.resc, s.rres));
    v = fminf(fmaxf(v, -s.max_state), s.max_state);
    if (!s.no_rounding) v = frint_add(v);
    v = rnd_int<DT>(fmul(v, s.res));
  }
  if (s.noise) v = rnd_int<DT>(fadd(v, rnd_int<DT>(fmul(s.amp, xi))));
  if (w != w) v = w;
  return v;
}

// Additive weight noise: w + (std_dev * s) * xi.
template <int DT>
AL_HD float add_weight_noise(float w, float std_dev, float s, float xi) {
  float a = rnd<DT>(fmul(std_dev, s));
  float nz = rnd<DT>(fmul(a, xi));
  return rnd<DT>(fadd(w, nz));
}

// Per-tile output stage.  acc is the fp32 dot product of the tile.
struct TileEpilogueCfg {
  int has_noise;        // training && out_noise > 0
  int has_bound;        // out_bound > 0
  int has_adc;          // out_res > 0
  int no_rounding;
  float noise_coef;     // float(out_noise / sqrt(T))
  float out_bound;
  float out_res;
};

// RD = dtype the intermediate results are rounded to (bf16 only in reference-rounding mode).
template <int RD>
AL_HD float tile_epilogue(float acc, float ir, float s_noise, float s_bound, float xi,
                          const TileEpilogueCfg& c, bool* keep) {
  float o = rnd<RD>(acc);
  if (c.has_noise) {
    float k = rnd<RD>(fmul(c.noise_coef, ir));
    float sc = rnd<RD>(fmul(s_noise, k));
    float nz = rnd<RD>(fmul(sc, xi));
    o = rnd<RD>(fadd(o, nz));
  }
  *keep = true;
  if (c.has_bound || c.has_adc) {
    float b0 = rnd<RD>(fmul(ir, c.out_bound));
    float bound = rnd<RD>(fmul(b0, s_bound));
    if (c.has_adc) {
      float step = quant_step<RD>(bound, c.out_res);
      float code = quant_code<RD>(o, step, c.no_rounding != 0);
      o = rnd<RD>(fmul(code, step));
    }
    if (c.has_bound) {
      *keep = (o >= -bound) && (o <= bound);
      o = fminf(fmaxf(o, -bound), bound);
    }
  }
  return o;
}

// ---- counter-based generator ------------------------------------------------------------
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
struct Philox4 {
  uint32_t v[4];
};
AL_HD uint32_t mulhi32(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __umulhi(a, b);
#else
  return (uint32_t)(((uint64_t)a * (uint64_t)b) >> 32);
#endif
}
template <int ROUNDS>
AL_HD Philox4 philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    uint32_t hi0 = mulhi32(M0, c0), lo0 = M0 * c0;
    uint32_t hi1 = mulhi32(M1, c2), lo1 = M1 * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  Philox4 out;
  out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}
AL_HD Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                            uint32_t k1) {
  return philox4x32<10>(c0, c1, c2, c3, k0, k1);
}

// Two standard normals from two 32-bit words (Box-Muller).
AL_HD void box_muller(uint32_t a, uint32_t b, float* z0, float* z1) {
  const float two_pow_m32 = 2.3283064365386963e-10f;
  float u1 = ((float)a + 0.5f) * two_pow_m32;  // (0, 1]
  float u2 = ((float)b + 0.5f) * two_pow_m32;
  if (u1 > 1.0f) u1 = 1.0f;
#if defined(__CUDA_ARCH__)
  float r = sqrtf(-2.0f * __logf(u1));
  float s, c;
  __sincosf(6.283185307179586f * u2, &s, &c);
#else
  float r = sqrtf(-2.0f * logf(u1));
  float s = sinf(6.283185307179586f * u2), c = cosf(6.283185307179586f * u2);
#endif
  *z0 = r * c;
  *z1 = r * s;
}

// Four normals for the group of four consecutive elements that contains element `idx` of
// stream `stream` (0: weight noise, 1: output noise) of call (seed, offset).
AL_HD void normal4(uint64_t seed, uint64_t offset, uint32_t stream, uint64_t group, float z[4]) {
  Philox4 p = philox4x32_10((uint32_t)group, (uint32_t)(group >> 32), (uint32_t)offset,
                            (uint32_t)(offset >> 32) ^ (stream * 0x85EBCA6Bu), (uint32_t)seed,
                            (uint32_t)(seed >> 32));
  box_muller(p.v[0], p.v[1], &z[0], &z[1]);
  box_muller(p.v[2], p.v[3], &z[2], &z[3]);
}
AL_HD float normal1(uint64_t seed, uint64_t offset, uint32_t stream, uint64_t idx) {
  float z[4];
  normal4(seed, offset, stream, idx >> 2, z);
  return z[idx & 3];
}

}  // namespace al
