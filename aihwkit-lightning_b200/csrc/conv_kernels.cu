// Patch extraction for AnalogConv2d: unfold2d writes the [B, L, C*kh*kw] patch matrix the
// analog linear operator consumes (patch axis ordered channel, kernel row, kernel column, like
// torch.nn.functional.unfold followed by the transpose the reference applies), fold2d is its
// adjoint for the backward pass (a gather per input pixel: fixed summation order, no atomics).
// Both are pure data movement and HBM bound.
#include "analog_math.cuh"
#include "internal.h"

namespace al {

namespace {

struct ConvGeom {
  int B, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, Ho, Wo;
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
  if (dtype == AL_F32) unfold2d_kernel<kF32><<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(x, g, out);
  else unfold2d_kernel<kBF16><<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(x, g, out);
  return check_launch("unfold2d");
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
  if (dtype == AL_F32) fold2d_kernel<kF32><<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(grad_patches, g, grad_x);
  else fold2d_kernel<kBF16><<<blocks_for(total), 256, 0, (cudaStream_t)stream>>>(grad_patches, g, grad_x);
  return check_launch("fold2d");
}

}  // extern "C"
