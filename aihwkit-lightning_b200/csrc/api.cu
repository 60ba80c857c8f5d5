// extern "C" entry points of libanalog_b200.so (declared in include/analog_b200.h): argument
// checking, narrowing of the configuration scalars, and the launch sequence of one forward /
// backward call.  No device memory is allocated here and nothing synchronises the stream.
#include <cuda.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include <nvtx3/nvToolsExt.h>

#include "analog_math.cuh"
#include "internal.h"

namespace al {

// NVTX range around an entry point: a timeline profiler shows which kernels belong to which call
// (the header-only NVTX loader does nothing unless a tool is attached).
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};

static thread_local char g_last_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  return AL_OK;
}

static int make_tile_table(const int32_t* ends, int T, int K, TileTable* tt) {
  if (ends == nullptr || T < 1) {
    set_error("tile table missing (T=%d)", T);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (T > kMaxTiles) {
    set_error("T=%d exceeds the maximum of %d analog tiles", T, kMaxTiles);
    return AL_ERR_TOO_LARGE;
  }
  int prev = 0;
  for (int t = 0; t < T; ++t) {
    if (ends[t] <= prev) {
      set_error("tile ends must be strictly increasing (tile %d: %d after %d)", t, ends[t], prev);
      return AL_ERR_BAD_ARGUMENT;
    }
    tt->ends[t] = ends[t];
    prev = ends[t];
  }
  if (prev != K) {
    set_error("last tile end %d != K=%d", prev, K);
    return AL_ERR_BAD_ARGUMENT;
  }
  tt->T = T;
  return AL_OK;
}

static int check_dtype(int dtype) {
  if (dtype != AL_F32 && dtype != AL_BF16) {
    set_error("unknown dtype %d", dtype);
    return AL_ERR_BAD_ARGUMENT;
  }
  return AL_OK;
}

static int derive(const AlDesc& d, Derived* o) {
  memset(o, 0, sizeof(*o));
  if (d.M < 1 || d.K < 1 || d.N < 1) {
    set_error("non-positive size M=%d K=%d N=%d", d.M, d.K, d.N);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (check_dtype(d.dtype)) return AL_ERR_BAD_ARGUMENT;
  if ((int64_t)(d.M > d.N ? d.M : d.N) * (int64_t)(d.T > 0 ? d.T : 1) >= (1ll << 31)) {
    set_error("rows * tiles = %lld exceeds 2^31 - 1 segments", (long long)(d.M > d.N ? d.M : d.N) * d.T);
    return AL_ERR_TOO_LARGE;
  }
  if (d.ir_mode < AL_IR_OFF || d.ir_mode > AL_IR_FAST) {
    set_error("unknown input-range mode %d", d.ir_mode);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (d.clip_type == AL_CLIP_LEARNABLE_PER_CHANNEL && d.quant_type != AL_QUANT_NONE &&
      d.quant_type != AL_QUANT_DISCRETIZE_PER_CHANNEL) {
    set_error("You can't learn weight ranges per column but quantize per tensor");
    return AL_ERR_BAD_ARGUMENT;
  }
  o->has_dac = d.inp_res > 0;
  if (o->has_dac && d.ir_mode == AL_IR_OFF) {
    set_error("inp_res > 0 needs an input range");
    return AL_ERR_BAD_ARGUMENT;
  }
  o->has_adc = d.out_res > 0;
  o->has_bound = d.out_bound > 0;
  if (o->has_adc && (!o->has_bound || d.ir_mode == AL_IR_OFF)) {
    set_error("out_res > 0 needs out_bound > 0 and an input range");
    return AL_ERR_BAD_ARGUMENT;
  }
  if (o->has_bound && d.ir_mode == AL_IR_OFF) {
    set_error("out_bound > 0 needs an input range");
    return AL_ERR_BAD_ARGUMENT;
  }
  o->has_noise = d.training && d.out_noise > 0;
  if (o->has_noise && d.ir_mode == AL_IR_OFF) {
    set_error("out_noise > 0 needs an input range");
    return AL_ERR_BAD_ARGUMENT;
  }
  o->inp_res = (float)d.inp_res;
  o->out_res = (float)d.out_res;
  o->out_bound = (float)d.out_bound;
  o->noise_coef = (float)(d.out_noise / sqrt((double)d.T));
  o->std_dev = (float)d.std_dev;
  o->decay = (float)d.decay;
  o->input_min_percentage = (float)d.input_min_percentage;
  o->init_std_alpha = (float)d.init_std_alpha;
  o->weight_quant = d.quant_type;
  o->weight_noise = d.training ? d.noise_type : AL_NOISE_NONE;
  if (o->weight_quant != AL_QUANT_NONE) {
    if (!(d.mod_res > 0)) {
      set_error("weight discretisation needs modifier.res > 0");
      return AL_ERR_BAD_ARGUMENT;
    }
    double n_states = d.mod_res > 1.0 / d.mod_res ? d.mod_res : 1.0 / d.mod_res;
    o->n_states = (float)n_states;
    o->max_state = (float)(n_states / 2.0);
  }
  o->bound_pc = d.clip_type == AL_CLIP_LAYER_GAUSSIAN_PER_CHANNEL ||
                d.clip_type == AL_CLIP_LEARNABLE_PER_CHANNEL;
  o->noise_pc = d.out_noise_per_channel != 0;
  o->round_dt = (d.dtype == AL_BF16 && d.ref_rounding) ? AL_BF16 : AL_F32;
  return AL_OK;
}

static bool needs_wmax(const Derived& dv) {
  return dv.has_adc || dv.has_bound || dv.has_noise || dv.weight_noise != AL_NOISE_NONE ||
         dv.weight_quant != AL_QUANT_NONE;
}
static size_t elem_size(int dtype) { return dtype == AL_BF16 ? 2 : 4; }

static bool pick_tc(const AlDesc& d, const TileTable& tt, bool backward) {
  if (d.engine == AL_ENGINE_SIMT) return false;
  return backward ? tc_backward_supported(d, tt) : tc_forward_supported(d, tt);
}

// fp32 layers: tensor cores (bf16 planes) when the configuration allows it and, under AUTO, when
// the layer is large enough for 128-wide blocks and the extra operand pre-passes to pay; layers
// with few output channels (convolutions) stay on the CUDA cores, they are bound by memory
static bool pick_tc_f32(const AlDesc& d, const TileTable& tt) {
  if (d.engine == AL_ENGINE_SIMT || !tc_f32_supported(d, tt)) return false;
  if (d.engine >= AL_ENGINE_TCGEN05) return true;
  // few output channels (convolutions): the 128-column blocks are mostly empty, but the forward and the
  // weight gradient still run 1.5-3 times faster than on the CUDA cores once there are enough rows
  return d.M >= 128 && d.N >= 16 && d.K >= 128 && (double)d.M * d.N * d.K >= 134217728.0;
}

}  // namespace al

namespace {
thread_local int g_reserved_sms = 0;
}  // namespace

namespace al {
int comm_reserved_sms() { return g_reserved_sms; }
}  // namespace al

using namespace al;

// The weight pre-pass of a large layer runs beside the DAC pass of its input on a second stream (both stream
// through HBM once and neither fills it alone): the caller's stream forks before the DAC launch and joins before
// the GEMM.  One stream and two events per device and host thread, made on first use.
namespace {
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool ready = false;
};
SideStream* side_stream() {
  // AL_B200_SERIAL_PREPASS=1 in the environment keeps both passes on the caller's stream (for A/B timing)
  static const bool serial = [] {
    const char* v = getenv("AL_B200_SERIAL_PREPASS");
    return v != nullptr && v[0] == '1';
  }();
  if (serial) return nullptr;
  thread_local SideStream table[64];  // per host thread: two threads never share the fork / join events
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  SideStream& ss = table[dev];
  if (!ss.ready) {
    if (cudaStreamCreateWithFlags(&ss.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&ss.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&ss.join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    ss.ready = true;
  }
  return &ss;
}
// both passes move at least this many elements: below that the fork and join cost more than they hide
constexpr int64_t kOverlapMinElems = (int64_t)1 << 22;
}  // namespace

extern "C" {

int al_version(void) { return 1; }

const char* al_last_error(void) { return g_last_error; }

const char* al_status_str(int status) {
  switch (status) {
    case AL_OK: return "ok";
    case AL_ERR_BAD_ARGUMENT: return "bad argument";
    case AL_ERR_UNSUPPORTED: return "unsupported configuration";
    case AL_ERR_CUDA: return "CUDA error";
    case AL_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case AL_ERR_TOO_LARGE: return "size beyond the stated maximum";
    default: return "unknown status";
  }
}

int al_abs_max_tiles(int32_t dtype, const void* a, int32_t rows, int32_t K,
                     const int32_t* tile_ends_host, int32_t T, void* out, void* stream) {
  if (check_dtype(dtype)) return AL_ERR_BAD_ARGUMENT;
  if (!a || !out || rows < 1 || K < 1) {
    set_error("al_abs_max_tiles: null pointer or empty matrix");
    return AL_ERR_BAD_ARGUMENT;
  }
  if ((int64_t)rows * (int64_t)(T > 0 ? T : 1) >= (1ll << 31)) {
    set_error("al_abs_max_tiles: rows * tiles exceeds 2^31 - 1 segments");
    return AL_ERR_TOO_LARGE;
  }
  TileTable tt;
  int rc = make_tile_table(tile_ends_host, T, K, &tt);
  if (rc) return rc;
  return launch_abs_max_tiles(dtype, a, rows, K, tt, out, (cudaStream_t)stream);
}

int64_t al_std_scratch_floats(int32_t rows, int32_t T) { return 2 * (int64_t)rows * T + T + 4; }

int al_std_tiles(int32_t dtype, const void* a, int32_t rows, int32_t K,
                 const int32_t* tile_ends_host, int32_t T, float* out, float* scratch,
                 void* stream) {
  if (check_dtype(dtype)) return AL_ERR_BAD_ARGUMENT;
  if (!a || !out || !scratch || rows < 1 || K < 1) {
    set_error("al_std_tiles: null pointer or empty matrix");
    return AL_ERR_BAD_ARGUMENT;
  }
  if ((int64_t)rows * (int64_t)(T > 0 ? T : 1) >= (1ll << 31)) {
    set_error("al_std_tiles: rows * tiles exceeds 2^31 - 1 segments");
    return AL_ERR_TOO_LARGE;
  }
  TileTable tt;
  int rc = make_tile_table(tile_ends_host, T, K, &tt);
  if (rc) return rc;
  return launch_std_tiles(dtype, a, rows, K, tt, out, scratch, (cudaStream_t)stream);
}

int32_t al_f32_planes(void) { return kPlanes; }

int al_uses_tcgen05(const AlDesc* desc, const int32_t* tile_ends_host) {
  if (!desc) return 0;
  TileTable tt;
  if (make_tile_table(tile_ends_host, desc->T, desc->K, &tt)) return 0;
  return (pick_tc(*desc, tt, false) || pick_tc_f32(*desc, tt)) ? 1 : 0;
}

int64_t al_backward_plane_elems(const AlDesc* desc, const int32_t* tile_ends_host) {
  if (!desc) return 0;
  TileTable tt;
  if (make_tile_table(tile_ends_host, desc->T, desc->K, &tt) || !pick_tc_f32(*desc, tt)) return 0;
  const int64_t plane = (int64_t)desc->M * desc->N;
  const int64_t sets_d = desc->out_bound > 0 ? desc->T : 1;                    // masked: one set per tile
  const int64_t sets_w = desc->ir_mode == AL_IR_DYNAMIC ? desc->T : 0;          // per-row DAC steps folded in
  return kPlanes * plane * (sets_d + sets_w);
}

int al_forward(const AlDesc* desc, const AlForwardArgs* a, void* stream) {
  if (!desc || !a) {
    set_error("al_forward: null descriptor");
    return AL_ERR_BAD_ARGUMENT;
  }
  NvtxRange range("al_forward");
  const AlDesc& d = *desc;
  Derived dv;
  int rc = derive(d, &dv);
  if (rc) return rc;
  TileTable tt;
  rc = make_tile_table(a->tile_ends, d.T, d.K, &tt);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const bool prequantised = a->x_prequantised != 0;
  const bool prequantised_codes = a->x_prequantised == 2;
  if (prequantised && (d.ir_mode != AL_IR_DYNAMIC || !(d.inp_res > 0) || !a->ir_rows ||
                       (prequantised_codes ? !a->codes16 : !a->xq))) {
    set_error("al_forward: x_prequantised needs a dynamic input range with the DAC on, xq and ir_rows");
    return AL_ERR_BAD_ARGUMENT;
  }
  if ((!a->x && !prequantised) || !a->w || !a->out) {
    set_error("al_forward: x, w and out must be given");
    return AL_ERR_BAD_ARGUMENT;
  }

  // 1. input range (static mode): optional init-from-data update, then copy the ranges used
  const void* ir_static = nullptr;
  if (d.ir_mode == AL_IR_FAST) {
    if (!a->input_range || !a->input_range_update_idx || !a->x_min || !a->x_max || !a->ir_rows) {
      set_error("fast input-range mode needs input_range, input_range_update_idx, x_min, x_max and ir_rows");
      return AL_ERR_BAD_ARGUMENT;
    }
    int do_update = d.training && d.init_from_data > 0;
    if (do_update && !a->std_scratch) {
      set_error("init_from_data > 0 needs std_scratch");
      return AL_ERR_BAD_ARGUMENT;
    }
    rc = launch_ir_fast_update(d.dtype, a->x, d.M, d.K, tt, a->input_range, a->input_range_update_idx,
                               a->x_min, a->x_max, d.init_from_data, (float)d.act_range_momentum,
                               (float)(1.0 - d.act_range_momentum), d.act_range_momentum == -1.0, do_update,
                               a->std_scratch, a->ir_rows, s);
    if (rc) return rc;
    ir_static = a->ir_rows;
  }
  if (d.ir_mode == AL_IR_STATIC) {
    if (!a->input_range || !a->input_range_update_idx || !a->ir_rows) {
      set_error("static input range needs input_range, input_range_update_idx and ir_rows");
      return AL_ERR_BAD_ARGUMENT;
    }
    int do_update = d.training && d.init_from_data > 0;
    if (do_update) {
      const float* std_in = a->std_override;  // given: the caller's (replica-averaged) statistics
      if (!std_in) {
        if (!a->std_scratch) {
          set_error("init_from_data > 0 needs std_scratch");
          return AL_ERR_BAD_ARGUMENT;
        }
        float* std_out = a->std_scratch + 2 * (int64_t)d.M * d.T;
        rc = launch_std_tiles(d.dtype, a->x, d.M, d.K, tt, std_out, a->std_scratch, s);
        if (rc) return rc;
        std_in = std_out;
      }
      rc = launch_ir_update(d.dtype, a->input_range, a->input_range_update_idx, std_in, d.T,
                            d.init_from_data, dv.init_std_alpha, 1, a->ir_rows, s);
    } else {
      rc = launch_ir_update(d.dtype, a->input_range, a->input_range_update_idx, nullptr, d.T, 0,
                            0.0f, 0, a->ir_rows, s);
    }
    if (rc) return rc;
    ir_static = a->ir_rows;
  }

  // fp32 layer on the tensor cores: needs the bf16 workspaces
  const bool tc_f32 = pick_tc_f32(d, tt) && a->codes16 != nullptr && a->w_planes != nullptr && a->x_prequantised != 1;
  if (prequantised_codes && !tc_f32) {
    set_error("al_forward: x_prequantised = 2 (bf16 codes) is for fp32 layers on the tensor cores (al_uses_tcgen05)");
    return AL_ERR_UNSUPPORTED;
  }
  if (d.dtype == AL_F32 && d.engine >= AL_ENGINE_TCGEN05 && !tc_f32) {
    set_error("tcgen05 engine requested for an fp32 layer that does not qualify (DAC on, rounding on, aligned tiles, "
              "codes16 and w_planes given)");
    return AL_ERR_UNSUPPORTED;
  }

  // A handful of rows, nothing to modify in the weights, no backward to prepare: the layer is
  // bound by streaming W once; one kernel takes abs-max and tile products from the same read and
  // quantises its slice of the inputs itself.
  const bool smallm = a->smallm_scratch && d.dtype == AL_BF16 && d.engine == AL_ENGINE_AUTO && !dv.has_noise &&
                      dv.weight_quant == AL_QUANT_NONE && dv.weight_noise == AL_NOISE_NONE &&
                      d.clip_type != AL_CLIP_LEARNABLE_PER_CHANNEL && !d.save_for_backward && a->w_amax &&
                      a->w_tile_max && smallm_forward_supported(d.M, d.K, d.N, tt) && ((uintptr_t)a->w % 16) == 0;
  // Every block of 64 output channels quantises the rows again, so the in-kernel DAC pays while
  // rows x channels is small (measured on B200: 3-13 % off a single-row call at every size, about even at
  // 16 rows x 4096 channels, slower beyond that, where the stand-alone pass is used).
  const bool smallm_dac = smallm && !prequantised && d.ir_mode != AL_IR_OFF && a->codes == nullptr &&
                          ((uintptr_t)a->x % 16) == 0 && (d.ir_mode != AL_IR_DYNAMIC || a->ir_rows != nullptr) &&
                          (int64_t)d.M * d.N <= 65536;

  // 2. DAC: x -> xq (+ per-row ranges in dynamic mode)
  const void* xq = a->x;
  bool tile_max_zeroed = false;
  SideStream* side = nullptr;  // non-null: forked, the weight pre-pass goes there
  if (prequantised) {
    xq = a->xq;
  } else if (d.ir_mode != AL_IR_OFF && !smallm_dac) {
    if (!a->xq || (d.ir_mode == AL_IR_DYNAMIC && !a->ir_rows)) {
      set_error("al_forward: xq / ir_rows workspace missing");
      return AL_ERR_BAD_ARGUMENT;
    }
    // the fused weight pre-pass that follows accumulates tile maxima into w_tile_max: the DAC kernel
    // clears those words on its way (no memset between the two kernels)
    bool fused_weights_next = !smallm && d.clip_type != AL_CLIP_LEARNABLE_PER_CHANNEL && needs_wmax(dv) &&
                              dv.weight_quant == AL_QUANT_NONE && dv.weight_noise != AL_NOISE_ADD_NORMAL &&
                              a->w_amax && a->w_tile_max;
    if (fused_weights_next && (int64_t)d.M * d.K >= kOverlapMinElems && (int64_t)d.N * d.K >= kOverlapMinElems &&
        a->w_mod && a->w_mod != a->w) {
      side = side_stream();
      if (side && cudaEventRecord(side->fork, s) == cudaSuccess && cudaStreamWaitEvent(side->stream, side->fork, 0) == cudaSuccess)
        fused_weights_next = false;  // the weight pass clears its own words: it no longer runs behind the DAC kernel
      else
        side = nullptr;
    }
    rc = launch_dac(d.dtype, a->x, d.M, d.K, tt, d.ir_mode == AL_IR_FAST ? AL_IR_STATIC : d.ir_mode, ir_static, dv.has_dac ? dv.inp_res : -1.0f,
                    d.no_rounding, a->xq, a->ir_rows, a->codes, s, tc_f32 ? a->codes16 : nullptr,
                    fused_weights_next ? a->w_tile_max : nullptr, 2 * d.T, &tile_max_zeroed);
    if (rc) return rc;
    xq = a->xq;
  }

  // 2b. the few-rows forward
  if (smallm && ((uintptr_t)xq % 16) == 0) {
    FwdEpilogueParams ep;
    memset(&ep, 0, sizeof(ep));
    ep.M = d.M; ep.N = d.N; ep.T = d.T;
    ep.ir_mode = d.ir_mode == AL_IR_FAST ? AL_IR_STATIC : d.ir_mode;
    ep.ir_rows = a->ir_rows;
    ep.bias = a->bias;
    ep.has_bound = dv.has_bound; ep.has_adc = dv.has_adc;
    ep.bound_pc = dv.bound_pc; ep.noise_pc = dv.noise_pc; ep.no_rounding = d.no_rounding;
    ep.noise_coef = dv.noise_coef; ep.out_bound = dv.out_bound; ep.out_res = dv.out_res;
    return launch_fwd_smallm(dv.round_dt, xq, a->w, d.K, tt, ep, a->w_amax, (float*)a->w_tile_max,
                             a->smallm_scratch, a->out, s, smallm_dac ? 1 : 0, ir_static,
                             dv.has_dac ? dv.inp_res : -1.0f, d.no_rounding);
  }

  // 3. weight statistics and modifier
  const void* w_mod = a->w;
  float* tile_max = nullptr;
  const bool learn_clip = d.clip_type == AL_CLIP_LEARNABLE_PER_CHANNEL;
  if (learn_clip) {
    // `quant_utils.py:184-233`, `torch_linear.py:236-246`: the weights are clamped to (or
    // discretised on the scale of) the learned ranges, which then stand in for the per-channel
    // abs-max everywhere downstream
    if (!a->learnable_weight_clip || !a->w_amax || !a->w_tile_max || !a->w_mod || a->w_mod == a->w) {
      set_error("al_forward: learnable_weight_clip, w_amax, w_tile_max and a separate w_mod are needed");
      return AL_ERR_BAD_ARGUMENT;
    }
    cudaError_t e = cudaMemcpyAsync(a->w_amax, a->learnable_weight_clip, elem_size(d.dtype) * d.T * d.N,
                                    cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess) {
      set_error("al_forward: copying the learned weight ranges: %s", cudaGetErrorString(e));
      return AL_ERR_CUDA;
    }
    tile_max = (float*)a->w_tile_max;
    int32_t* flags = (int32_t*)(tile_max + d.T);
    const int quant = dv.weight_quant == AL_QUANT_NONE ? kQuantLearnClamp : dv.weight_quant;
    rc = launch_tile_max(d.dtype, a->w_amax, d.N, tt, quant, dv.n_states, tile_max, flags, s);
    if (rc) return rc;
    rc = launch_weight_modify(d.dtype, a->w, d.N, d.K, tt, a->w_amax, tile_max, flags, quant, dv.n_states,
                              dv.max_state, dv.weight_noise, dv.std_dev, a->w_noise, a->seed, a->offset,
                              d.no_rounding, a->w_mod, s, a->offset_base);
    if (rc) return rc;
    w_mod = a->w_mod;
  } else if (needs_wmax(dv)) {
    if (!a->w_amax || !a->w_tile_max) {
      set_error("al_forward: w_amax / w_tile_max workspace missing");
      return AL_ERR_BAD_ARGUMENT;
    }
    tile_max = (float*)a->w_tile_max;
    int32_t* flags = (int32_t*)(tile_max + d.T);
    const bool modifies = dv.weight_quant != AL_QUANT_NONE || dv.weight_noise != AL_NOISE_NONE;
    if (modifies && (!a->w_mod || a->w_mod == a->w)) {
      set_error("al_forward: w_mod workspace missing (the modifier never writes into w)");
      return AL_ERR_BAD_ARGUMENT;
    }
    if (dv.weight_quant == AL_QUANT_NONE && dv.weight_noise != AL_NOISE_ADD_NORMAL) {
      // every scale the modifier needs is the segment's own abs-max: one sweep over w
      rc = launch_weight_fused(d.dtype, a->w, d.N, d.K, tt, a->w_amax, tile_max, dv.weight_noise,
                               dv.std_dev, a->w_noise, a->seed, a->offset, modifies ? a->w_mod : nullptr,
                               side ? side->stream : s, a->offset_base, tile_max_zeroed);
      if (side) {  // join, also after a failed launch: the caller's stream must not stay forked
        const cudaError_t ej = cudaEventRecord(side->join, side->stream);
        const cudaError_t ew = ej == cudaSuccess ? cudaStreamWaitEvent(s, side->join, 0) : ej;
        if (ew != cudaSuccess && !rc) {
          set_error("al_forward: joining the weight pre-pass: %s", cudaGetErrorString(ew));
          rc = AL_ERR_CUDA;
        }
        side = nullptr;
      }
      if (rc) return rc;
    } else {
      rc = launch_abs_max_tiles(d.dtype, a->w, d.N, d.K, tt, a->w_amax, s);
      if (rc) return rc;
      rc = launch_tile_max(d.dtype, a->w_amax, d.N, tt, dv.weight_quant, dv.n_states, tile_max, flags, s);
      if (rc) return rc;
      if (modifies) {
        rc = launch_weight_modify(d.dtype, a->w, d.N, d.K, tt, a->w_amax, tile_max, flags,
                                  dv.weight_quant, dv.n_states, dv.max_state, dv.weight_noise,
                                  dv.std_dev, a->w_noise, a->seed, a->offset, d.no_rounding, a->w_mod, s,
                                  a->offset_base);
        if (rc) return rc;
      }
    }
    if (modifies) w_mod = a->w_mod;
  }

  // 4. tiled GEMM with the per-tile output stage
  FwdEpilogueParams ep;
  memset(&ep, 0, sizeof(ep));
  ep.M = d.M; ep.N = d.N; ep.T = d.T;
  ep.ir_mode = d.ir_mode == AL_IR_FAST ? AL_IR_STATIC : d.ir_mode;  // one range per tile either way
  ep.ir_rows = a->ir_rows;
  ep.w_amax = a->w_amax;
  ep.w_tile_max = tile_max;
  ep.bias = a->bias;
  ep.out_noise = a->out_noise;
  ep.mask_words = (d.N + 31) / 32;
  ep.keep_mask = (dv.has_bound && d.save_for_backward) ? a->keep_mask : nullptr;
  if (dv.has_bound && d.save_for_backward && !a->keep_mask) {
    set_error("al_forward: keep_mask workspace missing");
    return AL_ERR_BAD_ARGUMENT;
  }
  ep.has_noise = dv.has_noise; ep.has_bound = dv.has_bound; ep.has_adc = dv.has_adc;
  ep.bound_pc = dv.bound_pc; ep.noise_pc = dv.noise_pc; ep.no_rounding = d.no_rounding;
  ep.noise_coef = dv.noise_coef; ep.out_bound = dv.out_bound; ep.out_res = dv.out_res;
  ep.seed = a->seed; ep.offset = a->offset;
  ep.offset_base = a->offset_base;

  if (tc_f32) {
    rc = launch_split_planes(static_cast<const float*>(w_mod), (int64_t)d.N * d.K, a->w_planes, s);
    if (rc) return rc;
    return launch_fwd_tc_f32(a->codes16, a->w_planes, d.K, tt, ep, dv.inp_res, a->out, s);
  }
  if (d.engine >= AL_ENGINE_TCGEN05 && !tc_forward_supported(d, tt)) {
    set_error("tcgen05 engine requested but the problem does not qualify (bf16, 16-byte aligned tiles)");
    return AL_ERR_UNSUPPORTED;
  }
  const int pairing = d.engine == AL_ENGINE_TCGEN05_PAIR ? 1 : d.engine == AL_ENGINE_TCGEN05_SINGLE ? -1 : 0;
  if (pick_tc(d, tt, false)) return launch_fwd_tc(dv.round_dt, xq, w_mod, d.K, tt, ep, pairing, a->out, s);
  return launch_fwd_simt(d.dtype, dv.round_dt, xq, w_mod, d.K, tt, ep, a->out, s);
}

int64_t al_smallm_scratch_floats(int32_t M, int32_t N, int32_t T) {
  // 0: the problem does not take the few-rows path (more than 16 rows), no scratch needed
  if (M < 1 || M > 16 || N < 1 || T < 1) return 0;
  return smallm_scratch_floats(N, T);
}

namespace {
// reductions of the bias / range / clip gradients, rounded up to 16 bytes; the partial sums of
// a split CUDA-core weight gradient follow
int64_t backward_reduce_floats(int32_t M, int32_t N, int32_t T) {
  const int64_t n = 256 * (int64_t)N + 3 * (int64_t)T * M + 16 + 2 * (int64_t)T + 16;
  return (n + 3) / 4 * 4;
}
}  // namespace

int64_t al_backward_scratch_floats(int32_t M, int32_t K, int32_t N, int32_t T) {
  if (M <= 0 || K <= 0 || N <= 0 || T <= 0) return 0;
  return backward_reduce_floats(M, N, T) + al::wgrad_simt_partial_floats(M, K, N, T);
}

int al_pair_work_item(int32_t num_blocks, int32_t n_pairs, int32_t item, int32_t* total, int32_t* block, int32_t* half) {
  if (num_blocks < 1 || n_pairs < 1 || !total || !block || !half) {
    set_error("al_pair_work_item: non-positive size or null output");
    return AL_ERR_BAD_ARGUMENT;
  }
  int t = 0, b = -1, h = -1;
  tc_pair_work_item(num_blocks, n_pairs, item, &t, &b, &h);
  *total = t;
  *block = b;
  *half = h;
  return AL_OK;
}

int al_wgrad_split_plan(int32_t M, int32_t K, int32_t N, int32_t T, int32_t* splits, int32_t* rows_per_split) {
  if (M <= 0 || K <= 0 || N <= 0 || T <= 0 || !splits || !rows_per_split) {
    set_error("al_wgrad_split_plan: non-positive size or null output");
    return AL_ERR_BAD_ARGUMENT;
  }
  int s = 1, c = 0;
  al::wgrad_simt_plan(M, K, N, T, &s, &c);
  *splits = s;
  *rows_per_split = c;
  return AL_OK;
}

int al_backward(const AlDesc* desc, const AlBackwardArgs* a, void* stream) {
  if (!desc || !a) {
    set_error("al_backward: null descriptor");
    return AL_ERR_BAD_ARGUMENT;
  }
  NvtxRange range("al_backward");
  const AlDesc& d = *desc;
  Derived dv;
  int rc = derive(d, &dv);
  if (rc) return rc;
  TileTable tt;
  rc = make_tile_table(a->tile_ends, d.T, d.K, &tt);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (!a->grad_out) {
    set_error("al_backward: grad_out missing");
    return AL_ERR_BAD_ARGUMENT;
  }
  if (a->reduce_scratch && a->reduce_scratch_floats < al_backward_scratch_floats(d.M, d.K, d.N, d.T)) {
    set_error("al_backward: reduce_scratch holds %lld floats, al_backward_scratch_floats asks for %lld",
              (long long)a->reduce_scratch_floats, (long long)al_backward_scratch_floats(d.M, d.K, d.N, d.T));
    return AL_ERR_BAD_ARGUMENT;
  }
  const uint32_t* mask = dv.has_bound ? a->keep_mask : nullptr;
  if (dv.has_bound && !mask) {
    set_error("al_backward: keep_mask missing although out_bound > 0");
    return AL_ERR_BAD_ARGUMENT;
  }
  int mask_words = (d.N + 31) / 32;
  // Without a clamp mask every tile sees the same gradient: one GEMM over the whole K range.
  TileTable one;
  one.T = 1;
  one.ends[0] = d.K;
  const TileTable& gt = mask ? tt : one;
  const int pairing = d.engine == AL_ENGINE_TCGEN05_PAIR ? 1 : d.engine == AL_ENGINE_TCGEN05_SINGLE ? -1 : 0;
  // fp32 layer whose forward ran on the tensor cores: bf16 planes of the upstream gradient
  const bool tc_f32 = pick_tc_f32(d, tt) && a->codes16 != nullptr && a->w_planes != nullptr && a->g_planes != nullptr;
  const int sets_d = mask ? d.T : 1;
  const int64_t plane_elems = kPlanes * (int64_t)d.M * d.N;
  if (tc_f32 && a->g_planes_elems < al_backward_plane_elems(desc, a->tile_ends)) {
    set_error("al_backward: g_planes holds %lld elements, al_backward_plane_elems asks for %lld",
              (long long)a->g_planes_elems, (long long)al_backward_plane_elems(desc, a->tile_ends));
    return AL_ERR_BAD_ARGUMENT;
  }
  if (d.engine >= AL_ENGINE_TCGEN05 && !tc_f32 && !tc_backward_supported(d, tt)) {
    set_error("tcgen05 engine requested but the problem does not qualify");
    return AL_ERR_UNSUPPORTED;
  }
  bool tc = !tc_f32 && pick_tc(d, tt, true);
  // an fp32 layer with fewer than 64 output channels: the input gradient reduces over those few channels
  // only, which the CUDA-core kernel does faster (52 against 76 us at 65536 x 288 x 32); it needs w_mod
  const bool dgrad_tc_f32 = tc_f32 && (d.N >= 64 || d.engine >= AL_ENGINE_TCGEN05 || !a->w_mod);
  if (tc_f32 && ((a->grad_x && dgrad_tc_f32) || (a->grad_w && d.ir_mode != AL_IR_DYNAMIC))) {
    // planes of g (masked per tile when the ADC clamped), shared by the input gradient and -- with
    // one input range per tile -- by the weight gradient
    rc = launch_split_planes_grad(static_cast<const float*>(a->grad_out), d.M, d.N, mask, mask_words, nullptr, 0, 0.0f,
                            sets_d, a->g_planes, s);
    if (rc) return rc;
  }

  if (a->grad_x) {
    if (!a->w_mod && !tc_f32) {
      set_error("al_backward: w_mod missing");
      return AL_ERR_BAD_ARGUMENT;
    }
    rc = dgrad_tc_f32 ? launch_dgrad_tc_f32(a->g_planes, sets_d, a->w_planes, d.M, d.K, d.N, tt, pairing, a->grad_x, s)
         : tc   ? launch_dgrad_tc(a->grad_out, a->w_mod, mask, mask_words, d.M, d.K, d.N, gt, pairing, a->grad_x, s)
                : launch_dgrad_simt(d.dtype, a->grad_out, a->w_mod, mask, mask_words, d.M, d.K, d.N, gt, a->grad_x, s);
    if (rc) return rc;
    if (d.ir_mode == AL_IR_STATIC || d.ir_mode == AL_IR_FAST) {
      if (!a->x || !a->ir_rows || !a->reduce_scratch) {
        set_error("al_backward: static input range needs x, ir_rows and reduce_scratch");
        return AL_ERR_BAD_ARGUMENT;
      }
      rc = launch_static_ir_backward(d.dtype, a->x, a->ir_rows, a->grad_x, d.M, d.K, tt, dv.decay,
                                     dv.input_min_percentage, a->grad_input_range,
                                     a->reduce_scratch + 256 * (int64_t)d.N, d.ir_mode == AL_IR_FAST, s);
      if (rc) return rc;
    }
  } else if (a->grad_input_range) {
    set_error("al_backward: grad_input_range needs grad_x");
    return AL_ERR_BAD_ARGUMENT;
  }
  if (a->grad_w && tc_f32) {
    // few output blocks (layers with few channels): the reduction over the batch rows is split over CTAs
    // exactly as the CUDA-core kernel splits it, into the same caller-sized buffer
    int w_splits = 1, w_chunk = 0;
    wgrad_simt_plan(d.M, d.K, d.N, d.T, &w_splits, &w_chunk);
    float* w_partial = nullptr;
    if (w_splits > 1) {
      const int64_t fixed = backward_reduce_floats(d.M, d.N, d.T);
      w_partial = a->reduce_scratch ? a->reduce_scratch + fixed : nullptr;
      const int64_t capacity = a->reduce_scratch ? a->reduce_scratch_floats - fixed : 0;
      if (w_partial == nullptr || (int64_t)w_splits * d.N * d.K > capacity) {
        set_error("al_backward: the partial-sum buffer holds %lld floats, %d splits x %d x %d need %lld",
                  (long long)capacity, w_splits, d.N, d.K, (long long)w_splits * d.N * d.K);
        return AL_ERR_BAD_ARGUMENT;
      }
    }
    if (d.ir_mode == AL_IR_DYNAMIC) {
      // per-row DAC steps: a second set of planes, one per tile, with the step (and the mask) folded in
      uint16_t* planes_w = static_cast<uint16_t*>(a->g_planes) + plane_elems * sets_d;
      rc = launch_split_planes_grad(static_cast<const float*>(a->grad_out), d.M, d.N, mask, mask_words,
                              static_cast<const float*>(a->ir_rows), 1, dv.inp_res, d.T, planes_w, s);
      if (rc) return rc;
      rc = launch_wgrad_tc_f32(planes_w, d.T, a->codes16, d.M, d.K, d.N, tt, nullptr, 0.0f, pairing, a->grad_w, s,
                               w_splits, w_partial);
    } else {
      rc = launch_wgrad_tc_f32(a->g_planes, sets_d, a->codes16, d.M, d.K, d.N, tt,
                               static_cast<const float*>(a->ir_rows), dv.inp_res, pairing, a->grad_w, s, w_splits,
                               w_partial);
    }
    if (rc) return rc;
  } else if (a->grad_w) {
    if (!a->xq) {
      set_error("al_backward: xq missing");
      return AL_ERR_BAD_ARGUMENT;
    }
    // the partial sums of a split CUDA-core weight gradient sit behind the reductions; what is
    // left of the caller's buffer there is the capacity the launch may use
    const int64_t fixed = backward_reduce_floats(d.M, d.N, d.T);
    float* partial = a->reduce_scratch ? a->reduce_scratch + fixed : nullptr;
    const int64_t partial_capacity = a->reduce_scratch ? a->reduce_scratch_floats - fixed : 0;
    rc = tc ? launch_wgrad_tc(a->grad_out, a->xq, mask, mask_words, d.M, d.K, d.N, gt, pairing, a->grad_w, s)
            : launch_wgrad_simt(d.dtype, a->grad_out, a->xq, mask, mask_words, d.M, d.K, d.N, gt, d.T, partial,
                                partial_capacity, a->grad_w, s);
    if (rc) return rc;
  }
  if (d.clip_type == AL_CLIP_LEARNABLE_PER_CHANNEL && (a->grad_w || a->grad_weight_clip)) {
    // `quant_utils.py:125-151`: straight-through inside the learned range, range gradient outside
    if (!a->grad_w || !a->grad_weight_clip || !a->w || !a->learnable_weight_clip || !a->reduce_scratch) {
      set_error("al_backward: learnable weight ranges need grad_w, grad_weight_clip, w, learnable_weight_clip "
                "and reduce_scratch");
      return AL_ERR_BAD_ARGUMENT;
    }
    float* tile_max = a->reduce_scratch + 256 * (int64_t)d.N + 3 * (int64_t)d.T * d.M + 16;
    int32_t* flags = (int32_t*)(tile_max + d.T);
    const int discretize = dv.weight_quant == AL_QUANT_DISCRETIZE_PER_CHANNEL;
    rc = launch_tile_max(d.dtype, a->learnable_weight_clip, d.N, tt, discretize ? dv.weight_quant : kQuantLearnClamp,
                         dv.n_states, tile_max, flags, s);
    if (rc) return rc;
    const double n_states_d = d.mod_res > 0 ? (d.mod_res > 1.0 / d.mod_res ? d.mod_res : 1.0 / d.mod_res) : 1.0;
    rc = launch_learn_clip_backward(d.dtype, a->w, a->learnable_weight_clip, flags, d.N, d.K, tt, discretize,
                                    dv.n_states, n_states_d / 2.0, d.no_rounding, a->grad_w, a->grad_weight_clip, s);
    if (rc) return rc;
  }
  if (a->grad_bias) {
    if (!a->reduce_scratch) {
      set_error("al_backward: reduce_scratch missing");
      return AL_ERR_BAD_ARGUMENT;
    }
    rc = launch_bias_grad(d.dtype, a->grad_out, d.M, d.N, a->grad_bias, a->reduce_scratch, s);
    if (rc) return rc;
  }
  return AL_OK;
}

int al_clip_weights(int32_t dtype, void* w, int32_t rows, int32_t cols, int32_t clip_type,
                    float sigma, float* scratch, void* stream) {
  if (check_dtype(dtype)) return AL_ERR_BAD_ARGUMENT;
  if (clip_type == AL_CLIP_NONE || clip_type == AL_CLIP_LEARNABLE_PER_CHANNEL) return AL_OK;
  if (!w || rows < 1 || cols < 1 || !scratch) {
    set_error("al_clip_weights: null pointer or empty matrix");
    return AL_ERR_BAD_ARGUMENT;
  }
  if (!(sigma > 0)) {
    set_error("Clip sigma must be greater than 0");
    return AL_ERR_BAD_ARGUMENT;
  }
  if (clip_type != AL_CLIP_LAYER_GAUSSIAN && clip_type != AL_CLIP_LAYER_GAUSSIAN_PER_CHANNEL) {
    set_error("Unknown clip type %d", clip_type);
    return AL_ERR_BAD_ARGUMENT;
  }
  return launch_clip_weights(dtype, w, rows, cols, clip_type, sigma, scratch, (cudaStream_t)stream);
}

int al_set_device_wait_limit_ns(uint64_t ns) { return tc_set_wait_limit(ns == 0 ? 2000000000ull : ns); }

int al_debug_withhold_forward_signal(int32_t on) {
  cudaError_t e = tc_fwd_set_withhold_acc_signal(on != 0 ? 1u : 0u);
  if (e != cudaSuccess) {
    set_error("al_debug_withhold_forward_signal: %s", cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  return AL_OK;
}

int al_read_device_error(void* stream, uint32_t* out_code) {
  if (!out_code) return AL_ERR_BAD_ARGUMENT;
  return tc_read_device_error((cudaStream_t)stream, out_code);
}

}  // extern "C"

// ---- launch accounting / per-kernel event timing ------------------------------------------
#include <mutex>
#include <vector>

namespace al {
namespace {
struct EventPair {
  cudaEvent_t start, stop;
  int cls;
};
std::mutex g_prof_mu;
bool g_prof_on = false;
uint32_t g_prof_classes = 0xffffffffu;
AlProfileEntry g_prof[AL_K_COUNT];
std::vector<EventPair*> g_pending, g_free;
}  // namespace

ProfScope::ProfScope(int kernel_class, cudaStream_t s, int launches)
    : cls(kernel_class), stream(s), slot(nullptr) {
  std::lock_guard<std::mutex> lock(g_prof_mu);
  g_prof[cls].launches += launches;
  if (!g_prof_on || !((g_prof_classes >> cls) & 1u)) return;
  EventPair* ep = nullptr;
  if (!g_free.empty()) {
    ep = g_free.back();
    g_free.pop_back();
  } else {
    ep = new EventPair();
    if (cudaEventCreate(&ep->start) != cudaSuccess || cudaEventCreate(&ep->stop) != cudaSuccess) {
      delete ep;
      cudaGetLastError();
      return;
    }
  }
  ep->cls = cls;
  cudaEventRecord(ep->start, stream);
  slot = ep;
}

ProfScope::~ProfScope() {
  if (!slot) return;
  EventPair* ep = static_cast<EventPair*>(slot);
  cudaEventRecord(ep->stop, stream);
  std::lock_guard<std::mutex> lock(g_prof_mu);
  g_pending.push_back(ep);
}
}  // namespace al

extern "C" {

int al_reserve_sms(int32_t n) {
  const int before = g_reserved_sms;
  g_reserved_sms = n < 0 ? 0 : n;
  return before;
}

int al_profile_enable(int on) {
  std::lock_guard<std::mutex> lock(g_prof_mu);
  g_prof_on = on != 0;
  return AL_OK;
}

int al_profile_select(uint32_t class_mask) {
  std::lock_guard<std::mutex> lock(g_prof_mu);
  g_prof_classes = class_mask;
  return AL_OK;
}

int al_profile_read(AlProfileEntry* out, int reset) {
  if (!out) return AL_ERR_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_prof_mu);
  for (EventPair* ep : g_pending) {
    float ms = 0.0f;
    if (cudaEventSynchronize(ep->stop) == cudaSuccess &&
        cudaEventElapsedTime(&ms, ep->start, ep->stop) == cudaSuccess) {
      g_prof[ep->cls].timed += 1;
      g_prof[ep->cls].total_ms += ms;
    } else {
      cudaGetLastError();
    }
    g_free.push_back(ep);
  }
  g_pending.clear();
  memcpy(out, g_prof, sizeof(g_prof));
  if (reset) memset(g_prof, 0, sizeof(g_prof));
  return AL_OK;
}

const char* al_kernel_class_name(int k) {
  static const char* names[AL_K_COUNT] = {
      "abs_max_tiles", "tile_max", "std_tiles", "ir_update", "dac", "weight_modify",
      "fwd_gemm", "dgrad_gemm", "wgrad_gemm", "bias_grad", "ir_backward", "clip_weights",
      "unfold2d", "fold2d"};
  return (k >= 0 && k < AL_K_COUNT) ? names[k] : "?";
}

}  // extern "C"
