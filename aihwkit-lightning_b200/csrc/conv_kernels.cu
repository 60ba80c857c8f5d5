// Patch extraction for AnalogConv2d: unfold2d writes the [B, L, C*kh*kw] patch matrix the
// analog linear operator consumes (patch axis ordered channel, kernel row, kernel column, like
// torch.nn.functional.unfold followed by the transpose the reference applies), fold2d is its
// adjoint for the backward pass (a gather per input pixel: fixed summation order, no atomics).
// Both are pure data movement and HBM bound.
#include <string.h>

#include "analog_math.cuh"
#include "device_fast.cuh"
#include "internal.h"

namespace al {

namespace {

struct ConvGeom {
  int B, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, Ho, Wo;
};

// n / d for 0 <= n, n * d < 2^32 as one multiplication: m = ceil(2^32 / d) from the host (0 stands for d = 1).
// Index arithmetic with run-time divisors is most of what the staging kernels below would otherwise execute.
inline uint32_t magic_of(int d) { return d == 1 ? 0u : (uint32_t)(0xFFFFFFFFull / (uint32_t)d + 1ull); }
__device__ __forceinline__ int fast_div(int n, uint32_t m) { return m ? (int)__umulhi((uint32_t)n, m) : n; }
struct StageDiv {
  uint32_t kw, kh, span, per_row, pads;  // magic numbers of the divisors the staging uses
  int n_pads;                            // padding columns of a slot (16-byte staging)
};

template <int DT>
__global__ void __launch_bounds__(256)
unfold2d_kernel(const void* __restrict__ x, ConvGeom g, void* __restrict__ out) {
  const int ckk = g.C * g.kh * g.kw;
  const int64_t total = (int64_t)g.B * g.Ho * g.Wo * ckk;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int e = (int)(idx % ckk);
    const int64_t bl = idx / ckk;
    const int l = (int)(bl % (g.Ho * g.Wo));
    const int b = (int)(bl / (g.Ho * g.Wo));
    const int j = e % g.kw, i = (e / g.kw) % g.kh, c = e / (g.kw * g.kh);
    const int oh = l / g.Wo, ow = l % g.Wo;
    const int h = oh * g.sh - g.ph + i * g.dh, w = ow * g.sw - g.pw + j * g.dw;
    float v = 0.0f;
    if (h >= 0 && h < g.H && w >= 0 && w < g.W)
      v = Elem<DT>::load(x, (((int64_t)b * g.C + c) * g.H + h) * g.W + w);
    Elem<DT>::store(out, idx, v);
  }
}

template <int DT>
__global__ void __launch_bounds__(256)
fold2d_kernel(const void* __restrict__ gp, ConvGeom g, void* __restrict__ gx) {
  const int ckk = g.C * g.kh * g.kw;
  const int64_t total = (int64_t)g.B * g.C * g.H * g.W;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int w = (int)(idx % g.W);
    const int h = (int)((idx / g.W) % g.H);
    const int c = (int)((idx / ((int64_t)g.W * g.H)) % g.C);
    const int b = (int)(idx / ((int64_t)g.W * g.H * g.C));
    float acc = 0.0f;
    for (int i = 0; i < g.kh; ++i) {
      const int hh = h + g.ph - i * g.dh;
      if (hh < 0 || hh % g.sh != 0) continue;
      const int oh = hh / g.sh;
      if (oh >= g.Ho) continue;
      for (int j = 0; j < g.kw; ++j) {
        const int ww = w + g.pw - j * g.dw;
        if (ww < 0 || ww % g.sw != 0) continue;
        const int ow = ww / g.sw;
        if (ow >= g.Wo) continue;
        acc += Elem<DT>::load(gp, ((int64_t)b * g.Ho * g.Wo + (int64_t)oh * g.Wo + ow) * ckk +
                                      ((int64_t)c * g.kh + i) * g.kw + j);
      }
    }
    Elem<DT>::store(gx, idx, acc);
  }
}

// ---- staged forms ------------------------------------------------------------------------------
// The patch matrix is [B * Ho * Wo, C * kh * kw]: the patches of one output row (b, oh) form one
// contiguous run of Wo * C*kh*kw elements.  A CTA of unfold2d_rows_kernel stages the kh input
// rows that output row reads (for a chunk of channels, zero padding included) in shared memory
// with coalesced loads and writes its part of the run with coalesced stores; where a patch
// element comes from is a table lookup (lut[e], e = position inside the chunk of the patch)
// plus ow * sw.
constexpr int kStageBytes = 40 * 1024;

// DAC fused into the patch extraction (dynamic per-patch input ranges): a warp writes one patch, so it
// has all elements of every analog tile of the patch in the staged rows in front of it -- abs-max of
// each tile by a warp reduction, then the quantised values straight to the GEMM's input matrix.  The
// fp32 patch matrix is never written.  Needs the whole patch in one channel chunk.
struct UnfoldDac {
  TileTable tt;
  float inp_res;
  void* ir_rows;      // [T, B*Ho*Wo] dtype: the ranges, as the DAC pre-pass would write them
  uint16_t* codes16;  // nullable: the integer DAC codes as bf16 (operand of the tensor-core GEMMs of an fp32 layer)
};

// Stages, for the output row `out_row` = (b, oh) and the channels [c0, c0 + cn), the kh input rows each channel's
// patches read (zero padding included) as tile[r * span + col], and fills lut[e] = where element e of a patch that
// starts at column 0 sits in the staged rows.  All threads of the CTA call it; it ends with a barrier.
// `by16`: a thread moves 16 bytes of an input row per load (the host checked that W is a multiple of the vector and
// that the slot of a row, `span` floats, holds the whole padded row).
template <int DT>
__device__ __forceinline__ void stage_patch_rows(const void* __restrict__ x, const ConvGeom& g, int out_row, int c0,
                                                 int cn, int span, float* tile, int* lut, int* row_src,
                                                 const StageDiv& dv, bool by16 = false) {
  const int kk = g.kh * g.kw;
  const int len = cn * kk;       // patch elements of this chunk
  const int rows = cn * g.kh;    // staged input rows
  const int b = out_row / g.Ho, oh = out_row - b * g.Ho;
  for (int e = threadIdx.x; e < len; e += blockDim.x) {
    const int row = fast_div(e, dv.kw);
    lut[e] = row * span + (e - row * g.kw) * g.dw;
  }
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    const int cl = fast_div(r, dv.kh);
    const int c = c0 + cl, i = r - cl * g.kh;
    const int h = oh * g.sh - g.ph + i * g.dh;
    row_src[r] = (h >= 0 && h < g.H) ? (c * g.H + h) * g.W : -1;  // offset of the input row, -1 = padding
  }
  __syncthreads();
  const int64_t image = (int64_t)b * g.C * g.H * g.W;
  if (by16) {
    // the stores are single floats: with an odd slot length the lanes of a warp, 4 (8) floats apart along a row and
    // one slot apart between rows, fall into different banks.  The padding columns are cleared afterwards.
    constexpr int V = DT == kF32 ? 4 : 8;
    const int per_row = g.W / V;
    for (int it = threadIdx.x; it < rows * per_row; it += blockDim.x) {
      const int r = fast_div(it, dv.per_row), at = (it - r * per_row) * V;
      const int src = row_src[r];
      float v[V];
#pragma unroll
      for (int u = 0; u < V; ++u) v[u] = 0.0f;
      if (src >= 0) {
        if (DT == kF32) {
          const float4 raw = *reinterpret_cast<const float4*>(static_cast<const float*>(x) + image + src + at);
          v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
        } else {
          const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + image + src + at);
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            v[2 * u] = __uint_as_float(w[u] << 16);
            v[2 * u + 1] = __uint_as_float(w[u] & 0xffff0000u);
          }
        }
      }
      float* dst = tile + r * span + g.pw + at;
#pragma unroll
      for (int u = 0; u < V; ++u) dst[u] = v[u];
    }
    const int right = g.pw + g.W;  // columns [pw, right) of a slot hold the image
    const int pads = dv.n_pads;
    for (int it = threadIdx.x; it < rows * pads; it += blockDim.x) {
      const int r = fast_div(it, dv.pads), p = it - r * pads;
      tile[r * span + (p < g.pw ? p : right + (p - g.pw))] = 0.0f;
    }
    __syncthreads();
    return;
  }
  // element idx = r * span + col of the staged rows; (r, col) advance without a division, and
  // kBatch loads are in flight per thread before the first one is stored
  constexpr int kBatch = 4;
  const int step_r = fast_div((int)blockDim.x, dv.span), step_col = (int)blockDim.x - step_r * span;
  int r = fast_div((int)threadIdx.x, dv.span), col = (int)threadIdx.x - r * span;
  for (int first = threadIdx.x; first < rows * span; first += blockDim.x * kBatch) {
    float v[kBatch];
    int rr = r, cc = col;
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      v[u] = 0.0f;
      if (rr < rows) {
        const int src = row_src[rr], w = cc - g.pw;
        if (src >= 0 && w >= 0 && w < g.W) v[u] = Elem<DT>::load(x, image + src + w);
      }
      rr += step_r;
      cc += step_col;
      if (cc >= span) { cc -= span; ++rr; }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (r < rows) tile[r * span + col] = v[u];
      r += step_r;
      col += step_col;
      if (col >= span) { col -= span; ++r; }
    }
  }
  __syncthreads();
}

template <int DT, bool DAC>
__global__ void __launch_bounds__(256)
unfold2d_rows_kernel(const void* __restrict__ x, ConvGeom g, int c_chunk, int span, const StageDiv dv,
                     void* __restrict__ out, const UnfoldDac dac) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kk = g.kh * g.kw, ckk = g.C * kk;
  // blockIdx.x = output row * chunks + chunk: CTAs that run together read and write neighbouring memory
  const int chunks = (g.C + c_chunk - 1) / c_chunk;
  const int out_row = blockIdx.x / chunks;
  const int c0 = (blockIdx.x - out_row * chunks) * c_chunk;
  const int cn = g.C - c0 < c_chunk ? g.C - c0 : c_chunk;
  const int len = cn * kk;
  float* tile = reinterpret_cast<float*>(smem_raw);             // [rows][span]
  int* lut = reinterpret_cast<int*>(tile + c_chunk * g.kh * span);  // [len]
  int* row_src = lut + c_chunk * kk;                                  // [rows]
  stage_patch_rows<DT>(x, g, out_row, c0, cn, span, tile, lut, row_src, dv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int64_t base = ((int64_t)out_row * g.Wo) * ckk + (int64_t)c0 * kk;
  for (int ow = warp; ow < g.Wo; ow += n_warps) {
    const int shift = ow * g.sw;
    const int64_t row = base + (int64_t)ow * ckk;
    if (DAC) {
      const int64_t m = (int64_t)out_row * g.Wo + ow, rows_total = (int64_t)g.B * g.Ho * g.Wo;
      for (int t = 0; t < dac.tt.T; ++t) {
        const int lo = dac.tt.lo(t), hi = dac.tt.hi(t);
        float amax = 0.0f;
        for (int e = lo + lane; e < hi; e += 32) amax = fmaxf(amax, fabsf(tile[lut[e] + shift]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) Elem<DT>::store(dac.ir_rows, (int64_t)t * rows_total + m, amax);
        const QuantSeg q = dac_prepare<DT>(amax, dac.inp_res, false, false);
        for (int e = lo + lane; e < hi; e += 32) {
          float code;
          const float v = dac_apply<DT>(q, tile[lut[e] + shift], &code);
          if (out != nullptr) Elem<DT>::store(out, row + e, v);
          if (dac.codes16 != nullptr) dac.codes16[row + e] = f32_to_bf16_bits(code);  // small integers: exact
        }
      }
    } else {
      for (int e = lane; e < len; e += 32) Elem<DT>::store(out, row + e, tile[lut[e] + shift]);
    }
  }
}

// The same patch extraction + DAC for patches whose length and tile ends are multiples of 4 (every convolution of a
// ResNet after the first): the CTA's output, the Wo patches of one output row, is one contiguous run, and a thread
// owns groups of 4 consecutive elements of it -- a group never straddles a patch or an analog tile.  Pass 1 gathers a
// group from the staged rows and folds its abs-max into the (patch, tile) maximum in shared memory; then one thread
// per (patch, tile) derives the quantiser; pass 2 quantises the group and writes it with 8- or 16-byte stores.  HOLD
// groups per thread stay in registers between the passes (HOLD = 0: any number of groups, gathered twice).  The slot
// of a staged row is an odd number of floats, which keeps the gather (lanes 4 elements apart, so 4/kw rows apart)
// at two to three lanes per bank.
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

constexpr int kGroupHold = 5;

template <int DT, int HOLD>
__global__ void __launch_bounds__(256)
unfold2d_dac4_kernel(const void* __restrict__ x, ConvGeom g, int span, const StageDiv dv, uint32_t gpp_magic, int by16,
                     int quads, void* __restrict__ out, const UnfoldDac dac) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kk = g.kh * g.kw, ckk = g.C * kk, T = dac.tt.T;
  const int out_row = blockIdx.x;
  const int gpp = ckk >> 2, n_groups = g.Wo * gpp;  // groups per patch, per CTA
  const int staged = (g.C * g.kh * span + 3) & ~3;
  float* tile = reinterpret_cast<float*>(smem_raw);   // [C * kh][span]
  int* lut = reinterpret_cast<int*>(tile + staged);   // [ckk], 16-byte aligned
  int* row_src = lut + ckk;                           // [C * kh]
  uint32_t* amax_bits = reinterpret_cast<uint32_t*>(row_src + g.C * g.kh);  // [Wo * T]
  float* seg_step = reinterpret_cast<float*>(amax_bits + g.Wo * T);         // [Wo * T]
  float* seg_rstep = seg_step + g.Wo * T;                                   // [Wo * T]
  unsigned char* grp_tile = reinterpret_cast<unsigned char*>(seg_rstep + g.Wo * T);  // [gpp]
  for (int i = threadIdx.x; i < g.Wo * T; i += blockDim.x) amax_bits[i] = 0u;
  for (int i = threadIdx.x; i < gpp; i += blockDim.x) {
    int t = 0;
    while (dac.tt.hi(t) <= i * 4) ++t;
    grp_tile[i] = (unsigned char)t;
  }
  stage_patch_rows<DT>(x, g, out_row, 0, g.C, span, tile, lut, row_src, dv, by16 != 0);

  auto gather = [&](int q, float (&v)[4], int& ow, int& e) {
    ow = fast_div(q, gpp_magic);
    e = (q - ow * gpp) << 2;
    const int shift = ow * g.sw;
    const int4 l = *reinterpret_cast<const int4*>(lut + e);
    v[0] = tile[l.x + shift]; v[1] = tile[l.y + shift]; v[2] = tile[l.z + shift]; v[3] = tile[l.w + shift];
  };
  // every thread of the warp calls this (q >= n_groups: nothing to add).  `quads`: tiles are whole multiples of 16
  // elements, so the 4 lanes of an aligned quad always share their (patch, tile) and one of them speaks for all.
  auto fold_max = [&](bool valid, const float (&v)[4], int ow, int e) {
    float m = valid ? fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))) : 0.0f;
    if (quads) {
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      if ((threadIdx.x & 3) != 0) valid = false;
    }
    // non-negative floats order like their bits
    if (valid) atomicMax(&amax_bits[ow * T + grp_tile[e >> 2]], __float_as_uint(m));
  };
  const int64_t base = ((int64_t)out_row * g.Wo) * ckk;
  // |v| <= the range of its tile, so |v / step| <= inp_res / 2 (or the quotient is NaN): rounding to an integer by
  // adding and subtracting 1.5 * 2^23 needs no large-value case here
  auto emit = [&](const float (&v)[4], int ow, int e) {
    const int seg = ow * T + grp_tile[e >> 2];
    const float step = seg_step[seg], stepc = step < kTiny ? kTiny : step, rstep = seg_rstep[seg];
    float code[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      code[u] = fsub(fadd(rnd_int<DT>(fdiv_rcp(v[u], stepc, rstep)), 12582912.0f), 12582912.0f);
    const int64_t at = base + (int64_t)ow * ckk + e;  // a multiple of 4
    if (dac.codes16 != nullptr)  // small integers: exact in bf16
      *reinterpret_cast<uint2*>(dac.codes16 + at) = make_uint2(cvt_bf16x2(code[0], code[1]), cvt_bf16x2(code[2], code[3]));
    if (out != nullptr) {
      float val[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) val[u] = rnd_int<DT>(fmul(code[u], step));
      if (DT == kF32)
        *reinterpret_cast<float4*>(static_cast<float*>(out) + at) = make_float4(val[0], val[1], val[2], val[3]);
      else  // values already rounded to bf16
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(out) + at) =
            make_uint2(cvt_bf16x2(val[0], val[1]), cvt_bf16x2(val[2], val[3]));
    }
  };

  float held[HOLD > 0 ? HOLD : 1][4];
  if (HOLD > 0) {
#pragma unroll
    for (int h = 0; h < HOLD; ++h) {
      const int q = threadIdx.x + h * 256;
      int ow = 0, e = 0;
      if (q < n_groups) gather(q, held[h], ow, e);
      fold_max(q < n_groups, held[h], ow, e);
    }
  } else {
    for (int q0 = 0; q0 < n_groups; q0 += 256) {
      const int q = q0 + threadIdx.x;
      int ow = 0, e = 0;
      if (q < n_groups) gather(q, held[0], ow, e);
      fold_max(q < n_groups, held[0], ow, e);
    }
  }
  __syncthreads();
  const int64_t rows_total = (int64_t)g.B * g.Ho * g.Wo;
  for (int i = threadIdx.x; i < g.Wo * T; i += blockDim.x) {
    const int t = i / g.Wo, ow = i - t * g.Wo;  // consecutive threads write consecutive ranges
    const float amax = __uint_as_float(amax_bits[ow * T + t]);
    Elem<DT>::store(dac.ir_rows, (int64_t)t * rows_total + (int64_t)out_row * g.Wo + ow, amax);
    const QuantSeg q = dac_prepare<DT>(amax, dac.inp_res, false, false);
    seg_step[ow * T + t] = q.step;
    seg_rstep[ow * T + t] = q.rstep;
  }
  __syncthreads();
  if (HOLD > 0) {
#pragma unroll
    for (int h = 0; h < HOLD; ++h) {
      const int q = threadIdx.x + h * 256;
      if (q < n_groups) {
        const int ow = fast_div(q, gpp_magic);
        emit(held[h], ow, (q - ow * gpp) << 2);
      }
    }
  } else {
    for (int q = threadIdx.x; q < n_groups; q += 256) {
      int ow, e;
      gather(q, held[0], ow, e);
      emit(held[0], ow, e);
    }
  }
}

// The adjoint.  A CTA owns a band of kFoldRows input rows of one image for a chunk of channels,
// stages every patch row (b, oh) that touches the band -- contiguous runs again -- and each
// thread then sums, for its (channel, h, w), the up to kh * kw staged values in the order
// (i, j), the order of the unstaged kernel.
constexpr int kFoldRows = 4;

// UNIT: both strides are 1, which takes the integer divisions out of the inner loop.
template <int DT, bool UNIT>
__global__ void __launch_bounds__(256)
fold2d_band_kernel(const void* __restrict__ gp, ConvGeom g, int c_chunk, int n_oh_max, void* __restrict__ gx) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* tile = reinterpret_cast<float*>(smem_raw);  // [n_oh][Wo][pitch]
  const int kk = g.kh * g.kw, ckk = g.C * kk;
  const int chunks = (g.C + c_chunk - 1) / c_chunk;
  const int band = blockIdx.x / chunks;  // blockIdx.x = band * chunks + chunk
  const int c0 = (blockIdx.x - band * chunks) * c_chunk;
  const int cn = g.C - c0 < c_chunk ? g.C - c0 : c_chunk;
  const int len = cn * kk;
  const int pitch = (c_chunk * kk) | 1;  // odd: threads with consecutive w read distinct banks
  const int bands = (g.H + kFoldRows - 1) / kFoldRows;
  const int b = band / bands, h0 = (band - b * bands) * kFoldRows;
  const int h1 = h0 + kFoldRows < g.H ? h0 + kFoldRows : g.H;
  // output rows that read input rows h0 .. h1 - 1
  int oh_lo = h0 + g.ph - (g.kh - 1) * g.dh;
  oh_lo = oh_lo <= 0 ? 0 : (oh_lo + g.sh - 1) / g.sh;
  int oh_hi = (h1 - 1 + g.ph) / g.sh;
  if (oh_hi > g.Ho - 1) oh_hi = g.Ho - 1;
  const int n_oh = oh_hi - oh_lo + 1 < n_oh_max ? oh_hi - oh_lo + 1 : n_oh_max;  // <= n_oh_max by construction
  // runs of `len` contiguous elements, one per patch row; kBatch loads in flight per thread
  constexpr int kBatch = 8;
  const int64_t src0 = ((int64_t)(b * g.Ho + oh_lo) * g.Wo) * ckk + (int64_t)c0 * kk;
  const int total = n_oh > 0 ? n_oh * g.Wo * len : 0;
  const int step_r = (int)blockDim.x / len, step_e = (int)blockDim.x - step_r * len;
  int r = (int)threadIdx.x / len, e = (int)threadIdx.x - r * len;  // (row, element) advance without a division
  for (int first = threadIdx.x; first < total; first += blockDim.x * kBatch) {
    float v[kBatch];
    int dst[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      dst[u] = -1;
      if (first + u * (int)blockDim.x < total) {
        dst[u] = r * pitch + e;
        v[u] = Elem<DT>::load(gp, src0 + (int64_t)r * ckk + e);
      }
      r += step_r;
      e += step_e;
      if (e >= len) { e -= len; ++r; }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u)
      if (dst[u] >= 0) tile[dst[u]] = v[u];
  }
  __syncthreads();
  const int per_c = (h1 - h0) * g.W;
  for (int idx = threadIdx.x; idx < cn * per_c; idx += blockDim.x) {
    const int cl = idx / per_c, rem = idx - cl * per_c;
    const int h = h0 + rem / g.W, w = rem % g.W;
    float acc = 0.0f;
    for (int i = 0; i < g.kh; ++i) {
      const int hh = h + g.ph - i * g.dh;
      if (hh < 0 || (!UNIT && hh % g.sh != 0)) continue;
      const int oh = UNIT ? hh : hh / g.sh;
      if (oh > oh_hi) continue;
      const float* row = tile + (oh - oh_lo) * g.Wo * pitch + (cl * g.kh + i) * g.kw;
      for (int j = 0; j < g.kw; ++j) {
        const int ww = w + g.pw - j * g.dw;
        if (ww < 0 || (!UNIT && ww % g.sw != 0)) continue;
        const int ow = UNIT ? ww : ww / g.sw;
        if (ow >= g.Wo) continue;
        acc += row[ow * pitch + j];
      }
    }
    Elem<DT>::store(gx, (((int64_t)b * g.C + c0 + cl) * g.H + h) * g.W + w, acc);
  }
}

// Unit-stride fp32 form of the band kernel, built to spend few instructions per byte (the form
// above is bound by instruction issue, not by memory).  The staged block is zero-padded --
// patch rows above / below the image and patch columns left / right of it hold zeros -- so the
// sum of an output needs no validity tests: kh * kw loads at offsets that a table in shared
// memory lists once per CTA.  Patch runs are loaded as 16-byte vectors; the slot walk carries
// (row, column, vector) along without divisions.  Lanes map to (channel mod 4, w): with a pitch
// (floats per staged slot) that is an odd multiple of 4 and an odd kh * kw the 32 lanes of a warp
// then read 32 distinct banks.
// Requires: C-chunk a multiple of 4 channels, 16-byte aligned runs (checked by the host).
__global__ void __launch_bounds__(256)
fold2d_band_unit_kernel(const float* __restrict__ gp, ConvGeom g, int c_chunk, int pitch, float* __restrict__ gx) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kk = g.kh * g.kw, ckk = g.C * kk;
  const int chunks = (g.C + c_chunk - 1) / c_chunk;
  const int band = blockIdx.x / chunks;
  const int c0 = (blockIdx.x - band * chunks) * c_chunk;
  const int cn = g.C - c0 < c_chunk ? g.C - c0 : c_chunk;   // a multiple of 4
  const int len4 = cn * kk / 4;                            // 16-byte vectors per patch run
  const int bands = (g.H + kFoldRows - 1) / kFoldRows;
  const int b = band / bands, h0 = (band - b * bands) * kFoldRows;
  const int h1 = h0 + kFoldRows < g.H ? h0 + kFoldRows : g.H;
  // staged slots: patch rows oh_min .. oh_min + rows - 1, patch columns ow_min .. ow_min + cols - 1
  const int rows = kFoldRows + (g.kh - 1) * g.dh, cols = g.W + (g.kw - 1) * g.dw;
  const int oh_min = h0 + g.ph - (g.kh - 1) * g.dh, ow_min = g.pw - (g.kw - 1) * g.dw;
  float* tile = reinterpret_cast<float*>(smem_raw);             // [rows][cols][pitch]
  int* tap = reinterpret_cast<int*>(tile + rows * cols * pitch);  // [kk]
  // tap (i, j) of output (h, w), channel cl sits at slot (h - h0 + (kh-1-i) dh, w + (kw-1-j) dw), element cl*kk + i*kw + j
  for (int t = threadIdx.x; t < kk; t += blockDim.x) {
    const int i = t / g.kw, j = t - i * g.kw;
    tap[t] = (((g.kh - 1 - i) * g.dh) * cols + (g.kw - 1 - j) * g.dw) * pitch + t;
  }
  const int total = rows * cols * len4;
  const int step_slot = (int)blockDim.x / len4, step_q = (int)blockDim.x - step_slot * len4;
  int slot = (int)threadIdx.x / len4, q = (int)threadIdx.x - slot * len4;
  int row = slot / cols, col = slot - row * cols;
  const int64_t image_rows = (int64_t)b * g.Ho;
  constexpr int kBatch = 4;
  for (int first = threadIdx.x; first < total; first += blockDim.x * kBatch) {
    float4 v[kBatch];
    int dst[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      dst[u] = -1;
      v[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (row < rows) {
        dst[u] = (row * cols + col) * pitch + 4 * q;
        const int oh = oh_min + row, ow = ow_min + col;
        if (oh >= 0 && oh < g.Ho && ow >= 0 && ow < g.Wo)
          v[u] = __ldg(reinterpret_cast<const float4*>(gp + ((image_rows + oh) * g.Wo + ow) * ckk + (int64_t)c0 * kk) + q);
      }
      q += step_q;
      col += step_slot;
      if (q >= len4) { q -= len4; ++col; }
      while (col >= cols) { col -= cols; ++row; }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u)
      if (dst[u] >= 0) *reinterpret_cast<float4*>(tile + dst[u]) = v[u];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int cl_lane = lane & 3, w_lane = lane >> 2;
  const int w_groups = (g.W + 7) >> 3, c_groups = cn >> 2;
  const int band_rows = h1 - h0;
  // items: (channel group, row of the band, group of 8 columns), the last fastest
  const int items = c_groups * band_rows * w_groups;
  int item = warp;
  int wg = item % w_groups, rest = item / w_groups;
  int hr = rest % band_rows, cg = rest / band_rows;
  const int adv_wg = n_warps % w_groups, adv_rest = n_warps / w_groups;
  for (; item < items; item += n_warps) {
    const int cl = cg * 4 + cl_lane, w = wg * 8 + w_lane;
    if (w < g.W) {
      const float* base = tile + (hr * cols + w) * pitch + cl * kk;
      float acc = 0.0f;
      for (int t = 0; t < kk; ++t) acc += base[tap[t]];
      gx[(((int64_t)b * g.C + c0 + cl) * g.H + h0 + hr) * g.W + w] = acc;
    }
    wg += adv_wg;
    int carry = adv_rest;
    if (wg >= w_groups) { wg -= w_groups; ++carry; }
    hr += carry;
    while (hr >= band_rows) { hr -= band_rows; ++cg; }
  }
}

// ---- input gradient of a unit-stride convolution without the patch matrix --------------------------------------
// grad_x[b, c, h, w] = sum over taps (i, j) and output channels n of grad_out[b, h + ph - i, w + pw - j, n] *
// w[n, c, i, j]: the product grad_out @ w followed by the fold, computed in place.  For layers with few output
// channels the patch gradient (kh * kw times the image) costs far more to write and read back than these
// multiplications cost on the CUDA cores.  A CTA owns `R` image rows of one image and a chunk of input channels;
// it stages the R + kh - 1 rows of grad_out it needs as gs[row][n][column] (zero outside the image, so the sums
// need no validity tests) and the weights as ws[tap][n][channel].  A thread accumulates PX pixels (rows hr + k * R / PX,
// same column) times CT channels in packed fp32 pairs: per (tap, n) PX scalar loads of grad_out and CT / 4 16-byte
// broadcast loads of weights feed PX * CT / 2 packed multiply-adds.
struct DirectPlan {
  int R, px, c_chunk, ct, rp, tp, threads;
  size_t smem;
  uint32_t m_w, m_kk, m_ckk, m_per_row, m_n4;
};

template <int CT, int PX>
__global__ void __launch_bounds__(256)
conv2d_dgrad_direct_kernel(const float* __restrict__ go, const float* __restrict__ w, ConvGeom g, int N, DirectPlan pl,
                           float* __restrict__ gx) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kk = g.kh * g.kw, ckk = g.C * kk;
  const int Wp = g.W + g.kw - 1, rows = pl.R + g.kh - 1, part = pl.R / PX;
  const int gs_floats = (rows * pl.rp + 3) & ~3;
  float* gs = reinterpret_cast<float*>(smem_raw);  // [rows] x rp floats, a row = [N][Wp]
  float* ws = gs + gs_floats;                      // [kk] x tp floats, a tap = [N][c_chunk]
  const int bands = (g.H + pl.R - 1) / pl.R;
  const int b = blockIdx.x / bands, h0 = (blockIdx.x - b * bands) * pl.R;
  const int c0 = blockIdx.y * pl.c_chunk;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  for (int i = tid; i < gs_floats / 4; i += nthreads) reinterpret_cast<float4*>(gs)[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  const int run = pl.c_chunk * kk;  // weights of one output channel for this chunk: contiguous in w
  for (int idx = tid; idx < N * run; idx += nthreads) {
    const int n = fast_div(idx, pl.m_ckk), e = idx - n * run;
    const int cl = fast_div(e, pl.m_kk), tap = e - cl * kk;
    ws[tap * pl.tp + n * pl.c_chunk + cl] = w[(int64_t)n * ckk + (int64_t)c0 * kk + e];
  }
  __syncthreads();
  const int oh_min = h0 + g.ph - (g.kh - 1), col0 = g.kw - 1 - g.pw;
  const int n4 = N >> 2, per_row = g.Wo * n4;
  for (int idx = tid; idx < rows * per_row; idx += nthreads) {
    const int r = fast_div(idx, pl.m_per_row), rem = idx - r * per_row;
    const int ow = fast_div(rem, pl.m_n4), q = rem - ow * n4;
    const int oh = oh_min + r;
    if (oh < 0 || oh >= g.Ho) continue;
    const float4 v = *reinterpret_cast<const float4*>(go + (((int64_t)b * g.Ho + oh) * g.Wo + ow) * N + 4 * q);
    float* d = gs + r * pl.rp + (4 * q) * Wp + col0 + ow;
    d[0] = v.x; d[Wp] = v.y; d[2 * Wp] = v.z; d[3 * Wp] = v.w;
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31, n_warps = nthreads >> 5;
  const int pixels = part * g.W, px_chunks = (pixels + 31) >> 5, c_groups = pl.c_chunk / CT;
  for (int item = warp; item < px_chunks * c_groups; item += n_warps) {
    const int cg = item / px_chunks, pc = item - cg * px_chunks;
    const int p = pc * 32 + lane;
    const bool valid = p < pixels;
    const int hr = valid ? fast_div(p, pl.m_w) : 0, wc = valid ? p - hr * g.W : 0;
    uint64_t acc[PX][CT / 2];
#pragma unroll
    for (int k = 0; k < PX; ++k)
#pragma unroll
      for (int u = 0; u < CT / 2; ++u) acc[k][u] = 0ull;  // two +0.0f
    for (int i = 0; i < g.kh; ++i) {
      for (int j = 0; j < g.kw; ++j) {
        const float* gt = gs + (hr + g.kh - 1 - i) * pl.rp + (wc + g.kw - 1 - j);
        const float* wt = ws + (i * g.kw + j) * pl.tp + cg * CT;
#pragma unroll 4
        for (int n = 0; n < N; ++n) {
          uint64_t gp[PX];
#pragma unroll
          for (int k = 0; k < PX; ++k) {
            const float gv = gt[k * part * pl.rp + n * Wp];
            gp[k] = f32x2_pack(gv, gv);
          }
#pragma unroll
          for (int v4 = 0; v4 < CT / 4; ++v4) {
            const ulonglong2 wv = *reinterpret_cast<const ulonglong2*>(wt + n * pl.c_chunk + 4 * v4);
#pragma unroll
            for (int k = 0; k < PX; ++k) {
              acc[k][2 * v4] = f32x2_fma(wv.x, gp[k], acc[k][2 * v4]);
              acc[k][2 * v4 + 1] = f32x2_fma(wv.y, gp[k], acc[k][2 * v4 + 1]);
            }
          }
        }
      }
    }
    if (!valid) continue;
#pragma unroll
    for (int k = 0; k < PX; ++k) {
      const int h = h0 + hr + k * part;
      if (h >= g.H) continue;
#pragma unroll
      for (int u = 0; u < CT / 2; ++u) {
        const int c = c0 + cg * CT + 2 * u;
        float lo, hi;
        f32x2_unpack(acc[k][u], &lo, &hi);
        gx[(((int64_t)b * g.C + c) * g.H + h) * g.W + wc] = lo;
        gx[(((int64_t)b * g.C + c + 1) * g.H + h) * g.W + wc] = hi;
      }
    }
  }
}

constexpr size_t kDirectMaxSmem = 96 * 1024;

// 0 = the direct kernel does not apply
int plan_direct(int dtype, const ConvGeom& g, int N, DirectPlan* pl) {
  if (dtype != AL_F32 || g.sh != 1 || g.sw != 1 || g.dh != 1 || g.dw != 1) return 0;
  if (g.ph > g.kh - 1 || g.pw > g.kw - 1 || N < 4 || N % 4 != 0 || g.C % 4 != 0) return 0;
  const int kk = g.kh * g.kw, Wp = g.W + g.kw - 1;
  pl->ct = g.C % 8 == 0 ? 8 : 4;
  // bands of 8 rows, four pixels per thread; images of fewer than 8 rows: bands of 4, two pixels
  pl->R = g.H >= 8 ? 8 : 4;
  pl->px = g.H >= 8 ? 4 : 2;
  // a warp spans 32 / W rows when the image is narrow: a row pitch of W (mod 32) keeps its lanes in distinct banks
  int rp = N * Wp;
  if (g.W < 32) rp += ((g.W - rp % 32) + 32) % 32;
  pl->rp = rp;
  const size_t gs_bytes = (size_t)(((pl->R + g.kh - 1) * rp + 3) & ~3) * 4;
  int cc = g.C;
  for (;;) {
    pl->tp = N * cc + 4;
    pl->smem = gs_bytes + (size_t)kk * pl->tp * 4;
    if (pl->smem <= kDirectMaxSmem) break;
    if (cc % 2 != 0 || (cc / 2) % pl->ct != 0) return 0;
    cc /= 2;
  }
  pl->c_chunk = cc;
  const int items = (((pl->R / pl->px) * g.W + 31) / 32) * (cc / pl->ct);
  pl->threads = 32 * (items < 8 ? items : 8);
  if ((int64_t)g.B * ((g.H + pl->R - 1) / pl->R) >= 2147483647 || g.C / cc > 65535) return 0;
  pl->m_w = magic_of(g.W);
  pl->m_kk = magic_of(kk);
  pl->m_ckk = magic_of(cc * kk);
  pl->m_per_row = magic_of(g.Wo * (N / 4));
  pl->m_n4 = magic_of(N / 4);
  return 1;
}

constexpr size_t kFoldUnitMaxSmem = 100 * 1024;

// floats per staged slot of the unit-stride kernel: the run, padded to an odd multiple of 4
int fold_unit_pitch(int chunk, int kk) {
  const int run = chunk * kk;  // a multiple of 4
  return (run / 4) % 2 == 1 ? run : run + 4;
}
size_t fold_unit_smem(const ConvGeom& g, int chunk) {
  const size_t slots = (size_t)(kFoldRows + (g.kh - 1) * g.dh) * (g.W + (g.kw - 1) * g.dw);
  return (slots * fold_unit_pitch(chunk, g.kh * g.kw) + g.kh * g.kw) * 4;
}
// channel chunk for the unit-stride kernel: a multiple of 4 whose padded block fits, 0 if none
int fold_unit_chunk(const ConvGeom& g) {
  if (g.sh != 1 || g.sw != 1 || g.C % 4 != 0) return 0;
  int c = g.C;
  while (c >= 4 && fold_unit_smem(g, c) > 48 * 1024) c -= 4;
  // wide images: four channels may still fit the opt-in shared memory (two CTAs per SM)
  if (c < 4 && fold_unit_smem(g, 4) <= kFoldUnitMaxSmem) c = 4;
  if (c < 4) return 0;
  const int chunks = (g.C + c - 1) / c;
  const int even = ((g.C + chunks - 1) / chunks + 3) / 4 * 4;
  return even <= c ? even : c;
}

// channels per CTA (0: does not fit, use the unstaged kernel): the most that fit the staging
// budget, then evened out over the resulting number of chunks
int even_chunk(int C, int most) {
  if (most < 1) return 0;
  if (most >= C) return C;
  const int chunks = (C + most - 1) / most;
  return (C + chunks - 1) / chunks;
}
int unfold_chunk(const ConvGeom& g, int span) {
  if ((int64_t)g.C * g.H * g.W >= 2147483647) return 0;  // row offsets inside one image are ints
  return even_chunk(g.C, kStageBytes / (g.kh * span * 4 + g.kh * g.kw * 4 + g.kh * 4));
}
int fold_max_rows(const ConvGeom& g) { return (kFoldRows - 1 + (g.kh - 1) * g.dh) / g.sh + 1; }
int fold_chunk(const ConvGeom& g) {
  const int64_t rows = (int64_t)fold_max_rows(g) * g.Wo;
  int c = g.C;
  while (c > 0 && rows * ((c * g.kh * g.kw) | 1) * 4 > kStageBytes) --c;
  return even_chunk(g.C, c);
}

StageDiv make_stage_div(const ConvGeom& g, int span, int per_row, int n_pads) {
  StageDiv dv;
  dv.kw = magic_of(g.kw);
  dv.kh = magic_of(g.kh);
  dv.span = magic_of(span);
  dv.per_row = magic_of(per_row > 0 ? per_row : 1);
  dv.pads = magic_of(n_pads > 0 ? n_pads : 1);
  dv.n_pads = n_pads;
  return dv;
}

int make_geom(int B, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
              ConvGeom* g) {
  if (B < 1 || C < 1 || H < 1 || W < 1 || kh < 1 || kw < 1 || sh < 1 || sw < 1 || ph < 0 || pw < 0 || dh < 1 ||
      dw < 1) {
    set_error("conv geometry: non-positive size, stride or dilation");
    return AL_ERR_BAD_ARGUMENT;
  }
  const int Ho = (H + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
  const int Wo = (W + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
  if (Ho < 1 || Wo < 1) {
    set_error("conv geometry: kernel larger than the padded input");
    return AL_ERR_BAD_ARGUMENT;
  }
  *g = ConvGeom{B, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, Ho, Wo};
  return AL_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

unsigned blocks_for(int64_t total) {
  int64_t b = (total + 255) / 256;
  const int64_t cap = 148 * 32;
  return (unsigned)(b < cap ? (b < 1 ? 1 : b) : cap);
}

}  // namespace

}  // namespace al

using namespace al;

extern "C" {

int al_unfold2d(int32_t dtype, const void* x, int32_t B, int32_t C, int32_t H, int32_t W, int32_t kh, int32_t kw,
                int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw, void* out, void* stream) {
  if ((dtype != AL_F32 && dtype != AL_BF16) || !x || !out) {
    set_error("al_unfold2d: bad dtype or null pointer");
    return AL_ERR_BAD_ARGUMENT;
  }
  ConvGeom g;
  int rc = make_geom(B, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, &g);
  if (rc) return rc;
  ProfScope prof(AL_K_UNFOLD, (cudaStream_t)stream);
  const int64_t total = (int64_t)B * g.Ho * g.Wo * C * kh * kw;
  const int span = (g.Wo - 1) * sw + (kw - 1) * dw + 1;
  const int chunk = unfold_chunk(g, span);
  if (chunk >= 1 && (int64_t)B * g.Ho * ((C + chunk - 1) / chunk) < 2147483647) {
    const unsigned grid = (unsigned)((int64_t)B * g.Ho * ((C + chunk - 1) / chunk));
    const size_t smem = (size_t)chunk * (kh * span + kh * kw + kh) * 4;
    const StageDiv dv = make_stage_div(g, span, 1, 0);
    if (dtype == AL_F32) unfold2d_rows_kernel<kF32, false><<<grid, 256, smem, (cudaStream_t)stream>>>(x, g, chunk, span, dv, out, UnfoldDac());
    else unfold2d_rows_kernel<kBF16, false><<<grid, 256, smem, (cudaStream_t)stream>>>(x, g, chunk, span, dv, out, UnfoldDac());
    return check_launch("unfold2d_rows");
  }
  if (dtype == AL_F32) unfold2d_kernel<kF32><<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(x, g, out);
  else unfold2d_kernel<kBF16><<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(x, g, out);
  return check_launch("unfold2d");
}

int al_unfold2d_dac(int32_t dtype, const void* x, int32_t B, int32_t C, int32_t H, int32_t W, int32_t kh, int32_t kw,
                    int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw,
                    const int32_t* tile_ends_host, int32_t T, double inp_res, void* xq, void* ir_rows, void* codes16,
                    void* stream) {
  if ((dtype != AL_F32 && dtype != AL_BF16) || !x || (!xq && !codes16) || !ir_rows || !tile_ends_host) {
    set_error("al_unfold2d_dac: bad dtype or null pointer");
    return AL_ERR_BAD_ARGUMENT;
  }
  ConvGeom g;
  int rc = make_geom(B, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, &g);
  if (rc) return rc;
  const int ckk = C * kh * kw;
  if (T < 1 || T > kMaxTiles || !(inp_res > 0) || tile_ends_host[T - 1] != ckk) {
    set_error("al_unfold2d_dac: tile table (T=%d, last end %d, patch length %d) or inp_res", T,
              T >= 1 && T <= kMaxTiles ? tile_ends_host[T - 1] : -1, ckk);
    return AL_ERR_BAD_ARGUMENT;
  }
  const int span = (g.Wo - 1) * sw + (kw - 1) * dw + 1;
  const int chunk = unfold_chunk(g, span);
  if (chunk < C || (int64_t)B * g.Ho >= 2147483647 || (int64_t)B * g.Ho * g.Wo * T >= 2147483647) {
    set_error("al_unfold2d_dac: the patch does not fit one staged block (use al_unfold2d and the DAC of al_forward)");
    return AL_ERR_UNSUPPORTED;
  }
  UnfoldDac host;
  memset(&host, 0, sizeof(host));
  host.tt.T = T;
  int prev = 0;
  for (int t = 0; t < T; ++t) {
    if (tile_ends_host[t] <= prev) {
      set_error("al_unfold2d_dac: tile ends must be strictly increasing");
      return AL_ERR_BAD_ARGUMENT;
    }
    host.tt.ends[t] = prev = tile_ends_host[t];
  }
  host.inp_res = (float)inp_res;
  host.ir_rows = ir_rows;
  host.codes16 = static_cast<uint16_t*>(codes16);
  cudaStream_t st = (cudaStream_t)stream;
  ProfScope prof(AL_K_UNFOLD, st);
  const unsigned grid = (unsigned)((int64_t)B * g.Ho);
  // patches and analog tiles in whole groups of 4 elements: the kernel with vector stores
  bool by4 = ckk % 4 == 0 && (!xq || aligned16(xq)) && (!codes16 || aligned16(codes16));
  bool quads = true;  // tiles in whole multiples of 16 elements: four neighbouring lanes always share a tile
  for (int t = 0; t < T; ++t) {
    by4 = by4 && tile_ends_host[t] % 4 == 0;
    quads = quads && tile_ends_host[t] % 16 == 0;
  }
  // 16-byte loads of the image rows need rows that start aligned and a slot that holds the whole padded row; the
  // slot length is odd either way (bank spread of the stores and of the gather)
  const int vec = dtype == AL_F32 ? 4 : 8;
  const bool by16 = W % vec == 0 && aligned16(x);
  const int pitch = (by16 && pw + W > span ? pw + W : span) | 1;
  const size_t smem4 = ((size_t)((C * kh * pitch + 3) & ~3) + ckk + C * kh + 3 * (size_t)g.Wo * T) * 4 + ckk / 4;
  if (by4 && smem4 <= 48 * 1024) {
    const bool hold = (int64_t)g.Wo * (ckk / 4) <= kGroupHold * 256;
    const StageDiv dv = make_stage_div(g, pitch, W / vec, by16 ? pw + (pitch - (pw + W)) : 0);
    const uint32_t gm = magic_of(ckk / 4);
    if (dtype == AL_F32) {
      if (hold) unfold2d_dac4_kernel<kF32, kGroupHold><<<grid, 256, smem4, st>>>(x, g, pitch, dv, gm, by16, quads, xq, host);
      else unfold2d_dac4_kernel<kF32, 0><<<grid, 256, smem4, st>>>(x, g, pitch, dv, gm, by16, quads, xq, host);
    } else {
      if (hold) unfold2d_dac4_kernel<kBF16, kGroupHold><<<grid, 256, smem4, st>>>(x, g, pitch, dv, gm, by16, quads, xq, host);
      else unfold2d_dac4_kernel<kBF16, 0><<<grid, 256, smem4, st>>>(x, g, pitch, dv, gm, by16, quads, xq, host);
    }
    return check_launch("unfold2d_dac4");
  }
  const size_t smem = (size_t)chunk * (kh * span + kh * kw + kh) * 4;
  const StageDiv dv_rows = make_stage_div(g, span, 1, 0);
  if (dtype == AL_F32) unfold2d_rows_kernel<kF32, true><<<grid, 256, smem, st>>>(x, g, chunk, span, dv_rows, xq, host);
  else unfold2d_rows_kernel<kBF16, true><<<grid, 256, smem, st>>>(x, g, chunk, span, dv_rows, xq, host);
  return check_launch("unfold2d_dac");
}

int al_fold2d(int32_t dtype, const void* grad_patches, int32_t B, int32_t C, int32_t H, int32_t W, int32_t kh,
              int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw, void* grad_x,
              void* stream) {
  if ((dtype != AL_F32 && dtype != AL_BF16) || !grad_patches || !grad_x) {
    set_error("al_fold2d: bad dtype or null pointer");
    return AL_ERR_BAD_ARGUMENT;
  }
  ConvGeom g;
  int rc = make_geom(B, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, &g);
  if (rc) return rc;
  ProfScope prof(AL_K_FOLD, (cudaStream_t)stream);
  const int64_t total = (int64_t)B * C * H * W;
  const int64_t bands = (int64_t)B * ((H + kFoldRows - 1) / kFoldRows);
  const int unit_chunk = dtype == AL_F32 && aligned16(grad_patches) ? fold_unit_chunk(g) : 0;
  if (unit_chunk >= 4 && bands * ((C + unit_chunk - 1) / unit_chunk) < 2147483647) {
    const unsigned grid = (unsigned)(bands * ((C + unit_chunk - 1) / unit_chunk));
    const size_t smem = fold_unit_smem(g, unit_chunk);
    if (smem > 48 * 1024) {  // per device and cheap: no caching
      const cudaError_t attr = cudaFuncSetAttribute(fold2d_band_unit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    (int)kFoldUnitMaxSmem);
      if (attr != cudaSuccess) {
        set_error("fold2d: shared-memory opt-in failed: %s", cudaGetErrorString(attr));
        return AL_ERR_CUDA;
      }
    }
    fold2d_band_unit_kernel<<<grid, 256, smem, (cudaStream_t)stream>>>(
        reinterpret_cast<const float*>(grad_patches), g, unit_chunk, fold_unit_pitch(unit_chunk, kh * kw),
        reinterpret_cast<float*>(grad_x));
    return check_launch("fold2d_band_unit");
  }
  const int chunk = fold_chunk(g);
  if (chunk >= 1 && bands * ((C + chunk - 1) / chunk) < 2147483647) {
    const int n_oh = fold_max_rows(g);
    const unsigned grid = (unsigned)(bands * ((C + chunk - 1) / chunk));
    const size_t smem = (size_t)n_oh * g.Wo * ((chunk * kh * kw) | 1) * 4;
    const bool unit = sh == 1 && sw == 1;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == AL_F32 && unit) fold2d_band_kernel<kF32, true><<<grid, 256, smem, st>>>(grad_patches, g, chunk, n_oh, grad_x);
    else if (dtype == AL_F32) fold2d_band_kernel<kF32, false><<<grid, 256, smem, st>>>(grad_patches, g, chunk, n_oh, grad_x);
    else if (unit) fold2d_band_kernel<kBF16, true><<<grid, 256, smem, st>>>(grad_patches, g, chunk, n_oh, grad_x);
    else fold2d_band_kernel<kBF16, false><<<grid, 256, smem, st>>>(grad_patches, g, chunk, n_oh, grad_x);
    return check_launch("fold2d_band");
  }
  if (dtype == AL_F32) fold2d_kernel<kF32><<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(grad_patches, g, grad_x);
  else fold2d_kernel<kBF16><<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(grad_patches, g, grad_x);
  return check_launch("fold2d");
}

int al_conv2d_input_grad_supported(int32_t dtype, int32_t N, int32_t B, int32_t C, int32_t H, int32_t W, int32_t kh,
                                   int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw) {
  ConvGeom g;
  DirectPlan pl;
  if (make_geom(B, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, &g)) return 0;
  return plan_direct(dtype, g, N, &pl);
}

int al_conv2d_input_grad(int32_t dtype, const void* grad_out, const void* w_mod, int32_t N, int32_t B, int32_t C,
                         int32_t H, int32_t W, int32_t kh, int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw,
                         int32_t dh, int32_t dw, void* grad_x, void* stream) {
  if (!grad_out || !w_mod || !grad_x) {
    set_error("al_conv2d_input_grad: null pointer");
    return AL_ERR_BAD_ARGUMENT;
  }
  ConvGeom g;
  int rc = make_geom(B, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, &g);
  if (rc) return rc;
  DirectPlan pl;
  if (!plan_direct(dtype, g, N, &pl) || !aligned16(grad_out)) {
    set_error("al_conv2d_input_grad: not a unit-stride fp32 convolution the direct kernel covers "
              "(ask al_conv2d_input_grad_supported; use al_backward and al_fold2d)");
    return AL_ERR_UNSUPPORTED;
  }
  ProfScope prof(AL_K_DGRAD_GEMM, (cudaStream_t)stream);
  const dim3 grid((unsigned)((int64_t)B * ((H + pl.R - 1) / pl.R)), (unsigned)(C / pl.c_chunk));
  const float* go = static_cast<const float*>(grad_out);
  const float* wm = static_cast<const float*>(w_mod);
  float* gx = static_cast<float*>(grad_x);
  cudaError_t attr = cudaSuccess;
#define AL_LAUNCH_DIRECT(CT_, PX_)                                                                                   \
  do {                                                                                                               \
    if (pl.smem > 48 * 1024)                                                                                         \
      attr = cudaFuncSetAttribute(conv2d_dgrad_direct_kernel<CT_, PX_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                  (int)kDirectMaxSmem);                                                              \
    if (attr == cudaSuccess)                                                                                         \
      conv2d_dgrad_direct_kernel<CT_, PX_><<<grid, pl.threads, pl.smem, (cudaStream_t)stream>>>(go, wm, g, N, pl, gx); \
  } while (0)
  if (pl.ct == 8 && pl.px == 4) AL_LAUNCH_DIRECT(8, 4);
  else if (pl.ct == 8) AL_LAUNCH_DIRECT(8, 2);
  else if (pl.px == 4) AL_LAUNCH_DIRECT(4, 4);
  else AL_LAUNCH_DIRECT(4, 2);
#undef AL_LAUNCH_DIRECT
  if (attr != cudaSuccess) {
    set_error("al_conv2d_input_grad: cudaFuncSetAttribute: %s", cudaGetErrorString(attr));
    return AL_ERR_CUDA;
  }
  return check_launch("conv2d_dgrad_direct");
}

}  // extern "C"
