// TEST INFRASTRUCTURE -- host build of the element-wise arithmetic the CUDA kernels use.
//
// The device functions in csrc/analog_math.cuh are written as host/device code.  This file
// compiles them for the CPU and wraps them in plain loops, so that the CPU test-suite can
// compare the kernels' rounding chains with the oracle bit for bit on machines without a GPU.
// Nothing here is linked into, or called by, the CUDA library or the Python package.
//
// build: g++ -O2 -ffp-contract=off -shared -fPIC kernel_math_host.cpp -o _build/libkernel_math_host.so
#include "../aihwkit-lightning_b200/csrc/analog_math.cuh"

using namespace al;

template <int DT>
static void dac_rows(const void* x, int M, int K, const int* ends, int T, int ir_mode,
                     const void* ir_static, float inp_res, int no_rounding, void* xq,
                     void* ir_rows, void* codes) {
  for (int m = 0; m < M; ++m) {
    for (int t = 0; t < T; ++t) {
      int lo = t ? ends[t - 1] : 0, hi = ends[t];
      float ir = 0.0f;
      bool clampit = false;
      if (ir_mode == 2) {
        for (int k = lo; k < hi; ++k) ir = fmaxf(ir, fabsf(Elem<DT>::load(x, (int64_t)m * K + k)));
        Elem<DT>::store(ir_rows, (int64_t)t * M + m, ir);
      } else if (ir_mode == 1) {
        ir = Elem<DT>::load(ir_static, t);
        clampit = true;
      }
      const QuantSeg seg = dac_prepare<DT>(ir, inp_res, clampit, no_rounding != 0);
      for (int k = lo; k < hi; ++k) {
        float c;
        float q = dac_apply<DT>(seg, Elem<DT>::load(x, (int64_t)m * K + k), &c);
        Elem<DT>::store(xq, (int64_t)m * K + k, q);
        if (codes) Elem<DT>::store(codes, (int64_t)m * K + k, c);
      }
    }
  }
}

template <int DT>
static void weight_modify_rows(const void* w, int N, int K, const int* ends, int T, int quant_type,
                               float n_states, float max_state, int noise_type, float std_dev,
                               const void* w_noise, int no_rounding, void* w_mod, void* amax_out,
                               const void* clip) {
  // clip != null: learned per-channel ranges [T,N] stand in for the abs-max; without a
  // discretiser they only clamp
  const bool learn_clamp = clip != nullptr && quant_type == 0;
  for (int t = 0; t < T; ++t) {
    int lo = t ? ends[t - 1] : 0, hi = ends[t];
    float t_max = 0.0f;
    bool all_gt1 = true;
    for (int n = 0; n < N; ++n) {
      float r = 0.0f;
      if (clip) r = Elem<DT>::load(clip, (int64_t)t * N + n);
      else for (int k = lo; k < hi; ++k) r = fmaxf(r, fabsf(Elem<DT>::load(w, (int64_t)n * K + k)));
      Elem<DT>::store(amax_out, (int64_t)t * N + n, r);
      t_max = fmaxf(t_max, r);
      if (quant_type == 2) all_gt1 = all_gt1 && discretize_scale_gt1<DT>(r, n_states);
      if (learn_clamp) all_gt1 = all_gt1 && r > 1.0f;
    }
    if (quant_type == 1) all_gt1 = discretize_scale_gt1<DT>(t_max, n_states);
    if (quant_type == 0 && !learn_clamp) all_gt1 = false;
    for (int n = 0; n < N; ++n) {
      float r = Elem<DT>::load(amax_out, (int64_t)t * N + n);
      const float n_scale = noise_type == 1 ? t_max : r;
      const WeightSeg ws =
          learn_clamp ? weight_prepare_learn_clamp<DT>(r, all_gt1, noise_type, std_dev, n_scale)
                      : weight_prepare<DT>(quant_type, quant_type == 1 ? t_max : r, n_states, max_state, all_gt1,
                                           noise_type, std_dev, n_scale, no_rounding != 0);
      for (int k = lo; k < hi; ++k) {
        float v = Elem<DT>::load(w, (int64_t)n * K + k);
        float xi = noise_type ? Elem<DT>::load(w_noise, (int64_t)n * K + k) : 0.0f;
        Elem<DT>::store(w_mod, (int64_t)n * K + k, weight_apply<DT>(ws, v, xi));
      }
    }
  }
}

// One tile's output stage applied to a given (already accumulated) tile product acc [M,N].
template <int DT>
static void tile_stage(const float* acc, int M, int N, const void* ir, int ir_per_row,
                       const void* s_noise, int s_noise_per_col, const void* s_bound,
                       int s_bound_per_col, const void* xi, const TileEpilogueCfg* cfg, void* out,
                       unsigned char* keep) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float irv = ir ? Elem<DT>::load(ir, ir_per_row ? m : 0) : 0.0f;
      float sn = s_noise ? Elem<DT>::load(s_noise, s_noise_per_col ? n : 0) : 0.0f;
      float sb = s_bound ? Elem<DT>::load(s_bound, s_bound_per_col ? n : 0) : 0.0f;
      float x = xi ? Elem<DT>::load(xi, (int64_t)m * N + n) : 0.0f;
      bool k;
      float o = tile_epilogue<DT>(acc[(int64_t)m * N + n], irv, sn, sb, x, *cfg, &k);
      Elem<DT>::store(out, (int64_t)m * N + n, o);
      keep[(int64_t)m * N + n] = k ? 1 : 0;
    }
}

extern "C" {

void km_dac(int dtype, const void* x, int M, int K, const int* ends, int T, int ir_mode,
            const void* ir_static, float inp_res, int no_rounding, void* xq, void* ir_rows,
            void* codes) {
  if (dtype == kF32) dac_rows<kF32>(x, M, K, ends, T, ir_mode, ir_static, inp_res, no_rounding, xq, ir_rows, codes);
  else dac_rows<kBF16>(x, M, K, ends, T, ir_mode, ir_static, inp_res, no_rounding, xq, ir_rows, codes);
}

void km_weight_modify(int dtype, const void* w, int N, int K, const int* ends, int T,
                      int quant_type, float n_states, float max_state, int noise_type,
                      float std_dev, const void* w_noise, int no_rounding, void* w_mod,
                      void* amax_out, const void* clip) {
  if (dtype == kF32) weight_modify_rows<kF32>(w, N, K, ends, T, quant_type, n_states, max_state, noise_type, std_dev, w_noise, no_rounding, w_mod, amax_out, clip);
  else weight_modify_rows<kBF16>(w, N, K, ends, T, quant_type, n_states, max_state, noise_type, std_dev, w_noise, no_rounding, w_mod, amax_out, clip);
}

void km_tile_stage(int dtype, const float* acc, int M, int N, const void* ir, int ir_per_row,
                   const void* s_noise, int s_noise_per_col, const void* s_bound,
                   int s_bound_per_col, const void* xi, int has_noise, int has_bound, int has_adc,
                   int no_rounding, float noise_coef, float out_bound, float out_res, void* out,
                   unsigned char* keep) {
  TileEpilogueCfg cfg;
  cfg.has_noise = has_noise; cfg.has_bound = has_bound; cfg.has_adc = has_adc;
  cfg.no_rounding = no_rounding; cfg.noise_coef = noise_coef; cfg.out_bound = out_bound;
  cfg.out_res = out_res;
  if (dtype == kF32) tile_stage<kF32>(acc, M, N, ir, ir_per_row, s_noise, s_noise_per_col, s_bound, s_bound_per_col, xi, &cfg, out, keep);
  else tile_stage<kBF16>(acc, M, N, ir, ir_per_row, s_noise, s_noise_per_col, s_bound, s_bound_per_col, xi, &cfg, out, keep);
}

// Reciprocal-based division and add-based rint against the plain operations: returns the
// number of mismatches over n pairs drawn from a xorshift stream (exponents in [-20, 20]).
long long km_check_fast_ops(long long n, unsigned long long seed) {
  unsigned long long s = seed ? seed : 88172645463325252ull;
  long long bad = 0;
  for (long long i = 0; i < n; ++i) {
    uint32_t bits[2];
    for (int j = 0; j < 2; ++j) {
      s ^= s << 13; s ^= s >> 7; s ^= s << 17;
      uint32_t m = (uint32_t)s & 0x7fffffu;
      int e = (int)((s >> 23) % 41) - 20;
      bits[j] = ((uint32_t)(s >> 63) << 31) | ((uint32_t)(e + 127) << 23) | m;
    }
    float a = u2f(bits[0]), b = fabsf(u2f(bits[1]));
    if (fdiv_rcp(a, b, frcp(b)) != fdiv(a, b)) ++bad;
    float x = a * 64.0f;
    if (frint_add(x) != frint(x)) ++bad;
    if (rnd_int<kBF16>(a) != rnd<kBF16>(a)) ++bad;
  }
  return bad;
}

// The tensor-core forward's ADC in bf16 arithmetic (adc_code_bf16) against the reference chain
// rint(RN_bf16(o / max(step, tiny))): every bf16 step significand at a few exponents, every bf16 o
// with |o / step| below about 300.  Codes up to +-127 must be equal (a zero code may differ in
// its sign); where the reference's code is beyond, the fast form must be beyond +-127 as well.
long long km_check_adc_bf16() {
  long long bad = 0;
  const int exps[5] = {-20, -3, 0, 1, 9};
  for (int e = 0; e < 5; ++e)
    for (uint32_t sig = 0; sig < 128; ++sig) {
      const float step = u2f(((uint32_t)(127 + exps[e]) << 23) | (sig << 16));
      const float stepc = step < kTiny ? kTiny : step;
      const float y = round_bf16(frcp(stepc));
      for (uint32_t ob = 0; ob < 65536; ++ob) {
        const float o = bf16_bits_to_f32((uint16_t)ob);
        if (!(fabsf(o) <= 300.0f * step)) continue;  // also skips NaN and infinities
        const float want = quant_code<kBF16>(o, step, false);
        const float got = adc_code_bf16(o, stepc, y);
        if (fabsf(want) < 128.0f ? !(got == want) : !(fabsf(got) >= 128.0f)) ++bad;
      }
    }
  return bad;
}

// n standard normals of stream `stream` of call (seed, offset), element indices [0, n)
void km_normals(unsigned long long seed, unsigned long long offset, unsigned stream, long long n, float* out) {
  for (long long i = 0; i < n; ++i) out[i] = normal1(seed, offset, stream, (uint64_t)i);
}

}  // extern "C"
