// Internal declarations shared by the translation units of libanalog_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/analog_b200.h"

namespace al {

constexpr int kMaxTiles = 256;

// Tile boundaries travel to the kernels by value (kernel parameter space), so that no device
// allocation or copy is needed for them.
struct TileTable {
  int32_t T;
  int32_t ends[kMaxTiles];  // cumulative, ends[T-1] == K
  __host__ __device__ int lo(int t) const { return t == 0 ? 0 : ends[t - 1]; }
  __host__ __device__ int hi(int t) const { return ends[t]; }
};

// Host-side derived constants of a forward/backward call (double -> float narrowing happens
// here, once, the way the Python reference narrows its scalars).
struct Derived {
  float inp_res, out_res, out_bound, noise_coef, std_dev, n_states, max_state;
  float decay, input_min_percentage, init_std_alpha;
  int has_dac, has_noise, has_bound, has_adc, bound_pc, noise_pc;
  int weight_noise;   // noise type active in this call (training only)
  int weight_quant;   // quant type
  int round_dt;       // dtype intermediate results are rounded to
};

// Everything the per-tile output stage of a forward GEMM kernel needs.
struct FwdEpilogueParams {
  int32_t M, N, T;
  int32_t ir_mode;
  const void* ir_rows;       // [T,M] (dynamic) or [T] (static), dtype
  const void* w_amax;        // [T,N] dtype
  const float* w_tile_max;   // [T]
  const void* bias;          // [N] dtype or null
  const void* out_noise;     // [T,M,N] dtype or null (replay)
  uint32_t* keep_mask;       // [T,mask_words,M] or null
  int32_t mask_words;
  int32_t has_noise, has_bound, has_adc, bound_pc, noise_pc, no_rounding;
  float noise_coef, out_bound, out_res;
  uint64_t seed, offset;
  const uint64_t* offset_base;  // call counter on the device, added to offset by the kernels (null: none)
};

// Internal weight-quantiser mode next to AlQuantType: the learned per-channel range used as a
// clamp only (LEARNABLE_PER_CHANNEL clipping without discretisation, `quant_utils.py:184-201`).
constexpr int kQuantLearnClamp = 100;

void set_error(const char* fmt, ...);

// Launch accounting: every launch_* function opens one scope.  Launch counts are always kept;
// when profiling is enabled (al_profile_enable) the scope also brackets the launches with CUDA
// events on the launching stream.
struct ProfScope {
  ProfScope(int kernel_class, cudaStream_t s, int launches = 1);
  ~ProfScope();
  int cls;
  cudaStream_t stream;
  void* slot;
};
int check_launch(const char* what);

// SMs the calling thread asked the backward GEMMs to leave unoccupied (al_reserve_sms), so that a
// communication kernel enqueued beside them finds room to run.
int comm_reserved_sms();

// ---- reductions (reduce_kernels.cu) -------------------------------------------------------
int launch_abs_max_tiles(int dtype, const void* a, int rows, int K, const TileTable& tt,
                         void* out, cudaStream_t s);
int launch_tile_max(int dtype, const void* amax, int rows, const TileTable& tt, int quant_type,
                    float n_states, float* tile_max, int32_t* flags, cudaStream_t s);
int launch_std_tiles(int dtype, const void* a, int rows, int K, const TileTable& tt, float* out,
                     float* scratch, cudaStream_t s);
int launch_ir_update(int dtype, void* input_range, void* update_idx, const float* std, int T,
                     int init_from_data, float init_std_alpha, int do_update, void* ir_used,
                     cudaStream_t s);
// fast mode: per-tile min / max over all rows and the momentum update of x_min, x_max, the
// range and its counter, all on the device; ir_used receives the ranges of this call
int launch_ir_fast_update(int dtype, const void* x, int M, int K, const TileTable& tt, void* input_range,
                          void* update_idx, void* x_min, void* x_max, int init_from_data, float momentum,
                          float one_minus_momentum, int minmax_mode, int do_update, float* scratch,
                          void* ir_used, cudaStream_t s);
int launch_clip_weights(int dtype, void* w, int rows, int cols, int clip_type, float sigma,
                        float* scratch, cudaStream_t s);

// ---- operand pre-passes (prepass_kernels.cu) ----------------------------------------------
// codes16 (fp32 layers only, nullable): the integer DAC codes as bf16 [M,K], the A operand of the
// tensor-core GEMMs of an fp32 layer
int launch_dac(int dtype, const void* x, int M, int K, const TileTable& tt, int ir_mode,
               const void* ir_static, float inp_res, int no_rounding, void* xq, void* ir_rows,
               void* codes, cudaStream_t s, void* codes16 = nullptr,
               void* zero_words = nullptr, int zero_count = 0, bool* zeroed = nullptr);

// ---- bf16 planes of fp32 operands (split_kernels.cu) ----------------------------------------
// An fp32 operand v travels to the tensor cores as kPlanes bf16 planes p0 = RN(v), p1 = RN(v - p0), ...
// Two planes carry 16 significant bits: the value is off by at most 2^-18 (2.2e-6 rms), which keeps a
// GEMM inside the 1e-5 relative bar of fp32 layers at two (one exact operand) or three (both split)
// plane products.
constexpr int kPlanes = 2;
// planes [kPlanes][count] bf16 (count % 4 == 0)
int launch_split_planes(const float* src, int64_t count, void* planes, cudaStream_t s);
// planes [sets][kPlanes][M][N] of g * keep_t * step(row, tile t): keep_mask null = nothing masked (sets
// may then be 1), ir null = no scaling; ir_per_row: ir is [T,M] (dynamic ranges), else [T]
int launch_split_planes_grad(const float* g, int M, int N, const uint32_t* keep_mask, int mask_words, const float* ir,
                       int ir_per_row, float inp_res, int sets, void* planes, cudaStream_t s);
int launch_weight_modify(int dtype, const void* w, int N, int K, const TileTable& tt,
                         const void* w_amax, const float* tile_max, const int32_t* flags,
                         int quant_type, float n_states, float max_state, int noise_type,
                         float std_dev, const void* w_noise, uint64_t seed, uint64_t offset,
                         int no_rounding, void* w_mod, cudaStream_t s, const uint64_t* offset_base = nullptr);

// abs-max + tile max + (per-channel-scaled) noise in one sweep; w_mod may be null when noise is off
int launch_weight_fused(int dtype, const void* w, int N, int K, const TileTable& tt, void* w_amax,
                        float* tile_max, int noise_type, float std_dev, const void* w_noise,
                        uint64_t seed, uint64_t offset, void* w_mod, cudaStream_t s,
                        const uint64_t* offset_base = nullptr, bool tile_max_zeroed = false);

// ---- SIMT GEMMs (gemm_simt.cu) ------------------------------------------------------------
// c_out[e] = sum over s of partial[s][e], e < count, added in the order of s
int launch_sum_partials(int dtype, const float* partial, int splits, int64_t count, void* c_out, cudaStream_t s);
int launch_fwd_simt(int dtype, int round_dt, const void* xq, const void* w_mod, int K,
                    const TileTable& tt, const FwdEpilogueParams& ep, void* out, cudaStream_t s);
// grad_x[:, tile] = (g * keep_t) @ w_mod[:, tile]
int launch_dgrad_simt(int dtype, const void* g, const void* w_mod, const uint32_t* keep_mask,
                      int mask_words, int M, int K, int N, const TileTable& tt, void* grad_x,
                      cudaStream_t s);
// grad_w[:, tile] = (g * keep_t)^T @ xq[:, tile].  `partial` holds wgrad_simt_partial_floats()
// floats (fp32 partial sums of the reduction over the rows when it is split over CTAs; may be
// null when that count is zero).
// Both take the LAYER's tile count (`layer_T`), not the tile table of the launch: the launch runs
// with a one-tile table when there is no clamp mask, and the split count must be the one the
// buffer was sized with.  `partial_capacity` is what the caller's buffer holds, in floats; a launch
// that would need more is refused on the host.
void wgrad_simt_plan(int M, int K, int N, int layer_T, int* splits, int* chunk_rows);
int64_t wgrad_simt_partial_floats(int M, int K, int N, int layer_T);
int launch_wgrad_simt(int dtype, const void* g, const void* xq, const uint32_t* keep_mask,
                      int mask_words, int M, int K, int N, const TileTable& tt, int layer_T, float* partial,
                      int64_t partial_capacity, void* grad_w, cudaStream_t s);

// ---- backward element-wise parts (backward_kernels.cu) ------------------------------------
int launch_bias_grad(int dtype, const void* g, int M, int N, void* grad_bias, float* scratch,
                     cudaStream_t s);
// learned per-channel weight ranges: grad_w -> gradient of the unclipped weights (in place),
// grad_clip [T,N]; all_gt1 = the per-tile flags launch_tile_max wrote for the ranges
int launch_learn_clip_backward(int dtype, const void* w, const void* clip, const int32_t* all_gt1, int N,
                               int K, const TileTable& tt, int discretize, float n_states, double max_state,
                               int no_rounding, void* grad_w, void* grad_clip, cudaStream_t s);
int launch_static_ir_backward(int dtype, const void* x, const void* ir_used, void* grad_x, int M,
                              int K, const TileTable& tt, float decay, float input_min_percentage,
                              void* grad_ir, float* scratch, int fast_mode, cudaStream_t s);

// ---- few-rows forward (gemm_smallm.cu): M <= 16, bf16, unmodified weights, no output noise ----
int64_t smallm_scratch_floats(int N, int T);
bool smallm_forward_supported(int M, int K, int N, const TileTable& tt);
int launch_fwd_smallm(int round_dt, const void* xq, const void* w, int K, const TileTable& tt,
                      const FwdEpilogueParams& ep, void* w_amax, float* tile_max, float* scratch, void* out,
                      cudaStream_t s, int dac_in_kernel, const void* ir_static, float inp_res, int no_rounding);

// ---- tcgen05 GEMMs (gemm_tcgen05_fwd.cu, gemm_tcgen05_bwd.cu) -----------------------------
bool tc_forward_supported(const AlDesc& d, const TileTable& tt);
// pairing: 0 = CTA pairs when they fill the machine, 1 = always pairs, -1 = never
int launch_fwd_tc(int round_dt, const void* xq, const void* w_mod, int K, const TileTable& tt,
                  const FwdEpilogueParams& ep, int pairing, void* out, cudaStream_t s);
bool tc_backward_supported(const AlDesc& d, const TileTable& tt);
void tc_pair_work_item(int num_work, int n_pairs, int item, int* total, int* block, int* half);
// pairing: 0 = CTA pairs when they fill the machine, 1 = always pairs, -1 = never
int launch_dgrad_tc(const void* g, const void* w_mod, const uint32_t* keep_mask, int mask_words,
                    int M, int K, int N, const TileTable& tt, int pairing, void* grad_x, cudaStream_t s);
int launch_wgrad_tc(const void* g, const void* xq, const uint32_t* keep_mask, int mask_words,
                    int M, int K, int N, const TileTable& tt, int pairing, void* grad_w, cudaStream_t s);
// fp32 layers on the tensor cores: operands as bf16 planes (split_kernels.cu)
bool tc_f32_supported(const AlDesc& d, const TileTable& tt);
int launch_fwd_tc_f32(const void* codes16, const void* w_planes, int K, const TileTable& tt,
                      const FwdEpilogueParams& ep, float inp_res, void* out, cudaStream_t s);
int launch_dgrad_tc_f32(const void* g_planes, int sets, const void* w_planes, int M, int K, int N, const TileTable& tt,
                        int pairing, void* grad_x, cudaStream_t s);
int launch_wgrad_tc_f32(const void* g_planes, int sets, const void* codes16, int M, int K, int N, const TileTable& tt,
                        const float* scale_ir, float inp_res, int pairing, void* grad_w, cudaStream_t s, int splits = 1,
                        float* partial = nullptr);
int tc_read_device_error(cudaStream_t s, uint32_t* code);
// limit of the device-side waits of all tcgen05 kernels (both translation units)
int tc_set_wait_limit(unsigned long long ns);
cudaError_t tc_fwd_set_wait_limit(unsigned long long ns);
// test aid: the forward kernel's MMA issuer withholds its "accumulator full" signal
cudaError_t tc_fwd_set_withhold_acc_signal(uint32_t on);
// the forward translation unit's own error word (read and cleared); the stream must be idle
cudaError_t tc_fwd_take_error_word(uint32_t* code);

}  // namespace al
