/*
 * analog_b200.h -- C ABI of libanalog_b200.so: the noisy, quantised, input-tiled analog
 * linear forward/backward for NVIDIA B200 (sm_100a).
 *
 * The reference (IBM/aihwkit-lightning) is pure Python: it has no native library and no FFI
 * for this path.  The functions below therefore replace *Python* call sites of the reference;
 * each one cites the call site it stands in for (paths inside the reference project,
 * `P = src/aihwkit_lightning/nn/modules`).
 *
 * Conventions
 *  - every pointer is a device pointer on the current CUDA device unless stated otherwise;
 *    the caller owns all memory, the library allocates nothing on the device;
 *  - `stream` is a `cudaStream_t` passed as `void*`; all work is enqueued on it and the
 *    functions return without synchronising;
 *  - matrices are row-major and contiguous: x [M,K], w [N,K], out [M,N];
 *  - "dtype" tensors have the layer's element type (AL_F32 or AL_BF16);
 *  - return value 0 = success, anything else is an `AlStatus` (see al_status_str);
 *  - functions are re-entrant; the only process-wide state is a cache of TMA tensor maps.
 */
#ifndef ANALOG_B200_H_
#define ANALOG_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum AlDtype { AL_F32 = 0, AL_BF16 = 1 };

enum AlStatus {
  AL_OK = 0,
  AL_ERR_BAD_ARGUMENT = 1,   /* null pointer, non-positive size, inconsistent tile table   */
  AL_ERR_UNSUPPORTED = 2,    /* configuration outside what the kernels implement           */
  AL_ERR_CUDA = 3,           /* a CUDA runtime / driver call failed (launch, tensor map)    */
  AL_ERR_DEVICE_TIMEOUT = 4, /* a bounded device-side wait gave up (al_read_device_error)   */
  AL_ERR_TOO_LARGE = 5       /* size beyond a stated maximum                               */
};

/* reference enums, `simulator/parameters/enums.py:46-90` */
enum AlNoiseType { AL_NOISE_NONE = 0, AL_NOISE_ADD_NORMAL = 1, AL_NOISE_ADD_NORMAL_PER_CHANNEL = 2 };
enum AlQuantType { AL_QUANT_NONE = 0, AL_QUANT_DISCRETIZE = 1, AL_QUANT_DISCRETIZE_PER_CHANNEL = 2 };
enum AlClipType {
  AL_CLIP_NONE = 0,
  AL_CLIP_LAYER_GAUSSIAN = 1,
  AL_CLIP_LAYER_GAUSSIAN_PER_CHANNEL = 2,
  AL_CLIP_LEARNABLE_PER_CHANNEL = 3
};
/* STATIC: learned / fixed range with init-from-data (std based); DYNAMIC: per-row abs-max;
 * FAST: the reference's fast_mode (min/max tracking, plain clamp, `torch_linear.py:361-423`) */
enum AlInputRangeMode { AL_IR_OFF = 0, AL_IR_STATIC = 1, AL_IR_DYNAMIC = 2, AL_IR_FAST = 3 };

/* GEMM engine selection.  AUTO picks the tcgen05/TMA kernels whenever dtype and alignment
 * allow and the SIMT kernels otherwise; SIMT and TCGEN05 force one of them (tests).  The
 * tcgen05 backward GEMMs run on CTA pairs (cta_group::2) when the problem has a 256 x 256 block
 * per pair of SMs and on single CTAs otherwise; TCGEN05_PAIR / TCGEN05_SINGLE force that choice
 * as well (tests, comparisons). */
enum AlEngine {
  AL_ENGINE_AUTO = 0, AL_ENGINE_SIMT = 1, AL_ENGINE_TCGEN05 = 2,
  AL_ENGINE_TCGEN05_PAIR = 3, AL_ENGINE_TCGEN05_SINGLE = 4
};

/*
 * Flattened `TorchInferenceRPUConfig` (`simulator/configs/configs.py:27-88`) plus the problem
 * size.  Field meaning is the reference's; see `simulator/parameters/{io,inference,mapping,
 * pre_post}.py`.
 */
/* Python floats of the configuration are carried as doubles so that derived constants
 * (out_noise/sqrt(T), max(res, 1/res), ...) are evaluated in double and narrowed to float
 * once, exactly like the Python reference does. */
typedef struct AlDesc {
  int32_t M, K, N, T;        /* rows, in_features, out_features, number of analog tiles     */
  int32_t dtype;             /* AlDtype                                                     */
  int32_t training;          /* module.training                                            */
  int32_t ir_mode;           /* AlInputRangeMode                                           */
  int32_t init_from_data;    /* InputRangeParameter.init_from_data                         */
  double init_std_alpha;      /* InputRangeParameter.init_std_alpha                         */
  double decay;               /* InputRangeParameter.decay                                  */
  double input_min_percentage;
  double act_range_momentum;  /* InputRangeParameter.act_range_momentum (fast mode)          */
  double inp_res;             /* IOParameters.inp_res  (<=0: DAC off)                        */
  double out_res;             /* IOParameters.out_res  (<=0: ADC quantisation off)           */
  double out_bound;           /* IOParameters.out_bound (<=0: no clipping)                   */
  double out_noise;           /* IOParameters.out_noise                                     */
  int32_t out_noise_per_channel;
  int32_t noise_type;        /* AlNoiseType                                                 */
  int32_t quant_type;        /* AlQuantType                                                 */
  double std_dev;             /* WeightModifierParameter.std_dev                            */
  double mod_res;             /* WeightModifierParameter.res                                */
  int32_t clip_type;         /* AlClipType (selects per-channel ADC bounds)                 */
  int32_t no_rounding;       /* skip rint in every quantiser (`quant_utils.py:60,88`)       */
  int32_t ref_rounding;      /* bf16: round to bf16 after every op like the reference does */
  int32_t engine;            /* AlEngine                                                    */
  int32_t save_for_backward; /* write `keep_mask` (forward) so that al_backward can run     */
} AlDesc;

/*
 * Buffers of one forward call.  Nullable entries say so.  Sizes in elements.
 */
typedef struct AlForwardArgs {
  const void* x;             /* [M,K] dtype                                                 */
  const void* w;             /* [N,K] dtype                                                 */
  const void* bias;          /* [N] dtype, nullable                                         */
  void* input_range;         /* [T] dtype, static mode: read, and updated while
                                 init_from_data is active; null otherwise                  */
  void* input_range_update_idx; /* [T] dtype, static mode                                   */
  void* x_min;               /* [T] dtype, fast mode: running minimum (updated)             */
  void* x_max;               /* [T] dtype, fast mode: running maximum (updated)             */
  const void* learnable_weight_clip; /* [T,N] dtype, clip type LEARNABLE_PER_CHANNEL: the learned
                                 per-tile per-channel weight ranges; null otherwise        */
  const int32_t* tile_ends;  /* HOST pointer, [T] cumulative tile ends (last == K)         */
  void* out;                 /* [M,N] dtype                                                 */
  /* saved for backward / intermediates (caller-allocated workspace) */
  void* xq;                  /* [M,K] dtype: DAC output fed to the GEMM. May equal x when
                                 the input range and the DAC are both off                  */
  void* ir_rows;             /* [T,M] dtype (dynamic mode) or [T] dtype (static mode: the
                                 ranges actually used by this call)                        */
  void* w_amax;              /* [T,N] dtype per-tile per-channel abs-max of w               */
  void* w_tile_max;          /* [T] float  per-tile abs-max of w + [T] int32 flags behind it */
  void* w_mod;               /* [N,K] dtype modified weights; may equal w when the modifier
                                 does nothing in this call                                  */
  uint32_t* keep_mask;       /* [T, ceil(N/32), M] word (t, n/32, m), bit n%32 = 1 where the
                                 ADC clamp of tile t passes the gradient of out[m, n];
                                 nullable if out_bound <= 0                                 */
  float* std_scratch;        /* >= al_std_scratch_floats(M, T) floats, static mode with
                                 init_from_data > 0 in training; nullable otherwise        */
  const float* std_override; /* [T] float, nullable: per-tile standard deviations to use for the
                                 init-from-data update of a static input range instead of
                                 computing them from x -- data-parallel callers pass the mean
                                 of al_std_tiles over all replicas so that every replica
                                 updates its ranges identically (the reference updates from
                                 the local batch, P/torch_utils/torch_linear.py:338-352)   */
  float* smallm_scratch;     /* >= al_smallm_scratch_floats(M, N, T) floats, nullable: lets a
                                 call with M <= 16 rows that modifies no weights and prepares
                                 no backward stream the weights once (abs-max and tile
                                 products from the same read)                               */
  /* fp32 layers on the tensor cores (al_uses_tcgen05): workspace for the bf16 operands of the GEMMs,
   * both nullable (the layer then runs on the CUDA cores) */
  void* codes16;             /* [M,K] bf16: the integer DAC codes                           */
  void* w_planes;            /* [al_f32_planes(),N,K] bf16: planes whose sum approximates
                                 w_mod to 2^-18 relative                                    */
  /* shared-noise parity mode: standard normals to use instead of the internal generator */
  const void* w_noise;       /* [N,K] dtype, nullable                                       */
  const void* out_noise;     /* [T,M,N] dtype, nullable                                     */
  /* optional debug output */
  void* codes;               /* [M,K] dtype integer DAC codes, nullable                     */
  uint64_t seed, offset;     /* counter-based generator: (seed, call counter)              */
  int32_t x_prequantised;    /* 1: xq and ir_rows already hold the DAC's output (al_unfold2d_dac);
                                 x may then be null and the DAC stage is skipped (dynamic
                                 input ranges only).  2: codes16 and ir_rows hold it (the codes
                                 as bf16, for an fp32 layer that al_uses_tcgen05 reports on the
                                 tensor cores); x and xq may be null                          */
  const uint64_t* offset_base; /* nullable: one counter in DEVICE memory that every noise kernel of the
                                 call adds to `offset` when it starts.  A caller that captures its
                                 calls in a CUDA graph (where `offset` is frozen) advances this
                                 counter between replays and so draws fresh noise every time      */
} AlForwardArgs;

typedef struct AlBackwardArgs {
  const void* grad_out;      /* [M,N] dtype                                                 */
  const void* x;             /* [M,K] dtype (static mode: clip positions)                   */
  const void* xq;            /* [M,K] dtype from the forward                                */
  const void* w_mod;         /* [N,K] dtype from the forward                                */
  const void* ir_rows;       /* as written by the forward                                   */
  const uint32_t* keep_mask; /* as written by the forward, nullable if out_bound <= 0      */
  const int32_t* tile_ends;  /* HOST pointer                                                */
  void* grad_x;              /* [M,K] dtype, nullable                                       */
  void* grad_w;              /* [N,K] dtype, nullable                                       */
  void* grad_bias;           /* [N] dtype, nullable                                         */
  void* grad_input_range;    /* [T] dtype, nullable (static mode, learn_input_range)       */
  float* reduce_scratch;     /* >= al_backward_scratch_floats(M,K,N,T) floats               */
  int64_t reduce_scratch_floats; /* floats the caller's reduce_scratch holds; a call that would need
                                 more than that is refused before anything is launched     */
  /* fp32 layers on the tensor cores: codes16 and w_planes as written by the forward, g_planes a
   * workspace of g_planes_elems >= al_backward_plane_elems(desc) bf16 elements; all null / 0 when
   * the forward ran on the CUDA cores */
  const void* codes16;
  const void* w_planes;
  void* g_planes;
  int64_t g_planes_elems;
  /* clip type LEARNABLE_PER_CHANNEL (`quant_utils.py:125-151`): grad_w becomes the gradient of
   * the unclipped weights and grad_weight_clip that of the learned ranges; null otherwise */
  const void* w;             /* [N,K] dtype weights of the forward                          */
  const void* learnable_weight_clip; /* [T,N] dtype                                         */
  void* grad_weight_clip;    /* [T,N] dtype                                                 */
} AlBackwardArgs;

/* Per-tile, per-row abs-max: out[t, r] = max_k |a[r, k]|, k in tile t.  a is [rows, K] dtype,
 * out [T, rows] dtype.  Replaces `sliced_abs_max` (P/torch_utils/torch_abs_max.py:17-39), the
 * in-loop `abs().amax(-1)` (P/torch_utils/torch_linear.py:220), the dynamic input range
 * `abs().max(-1)` (torch_linear.py:156) and the Triton `sliced_fast_abs_max`
 * (P/triton_utils/triton_abs_max.py:273-327). */
int al_abs_max_tiles(int32_t dtype, const void* a, int32_t rows, int32_t K,
                     const int32_t* tile_ends_host, int32_t T, void* out, void* stream);

/* Per-tile unbiased standard deviation over all rows: out[t] = std(a[:, tile t]) as float.
 * Replaces `values.std()` of the init-from-data update (torch_linear.py:342) and the Triton
 * `sliced_fast_std` (P/triton_utils/triton_std.py:184-245).  scratch: al_std_scratch_floats. */
int al_std_tiles(int32_t dtype, const void* a, int32_t rows, int32_t K,
                 const int32_t* tile_ends_host, int32_t T, float* out, float* scratch,
                 void* stream);
int64_t al_std_scratch_floats(int32_t rows, int32_t T);

/* Same result as al_std_tiles, for callers that have no way to hand over a scratch buffer.
 * This entry point has no counterpart in the reference.  It is meant for hosts that must not
 * (or cannot) allocate device memory when they need the statistic -- a serving process whose
 * device arena is fixed at start-up and where a later cudaMalloc would stall every stream of
 * the device, or a hook running inside another component's forward pass that owns no
 * allocator.  The stage-1 partials go to a 2 MiB array built into the library image (resident
 * on every GPU that loads the library, until the process exits), so the problem is limited
 * to rows*T <= AL_STD_STATIC_MAX_SEGMENTS; larger ones return AL_ERR_TOO_LARGE.  The call
 * allocates nothing.  The first call on each device looks the array's device address up
 * (with that device current); make that first call outside of any stream capture.  All calls
 * on a device share the array: calls whose kernels may overlap on the GPU race and must be
 * serialised by the caller.  `a` and `out` are the caller's, as for al_std_tiles. */
#define AL_STD_STATIC_MAX_SEGMENTS 262144
int al_std_tiles_static(int32_t dtype, const void* a, int32_t rows, int32_t K,
                        const int32_t* tile_ends_host, int32_t T, float* out, void* stream);

/* Whole forward of one analog layer.  Replaces `TorchLinear.linear`
 * (P/torch_utils/torch_linear.py:116-314) and `TritonLinear.forward`
 * (P/triton_utils/triton_linear.py:446-690). */
int al_forward(const AlDesc* desc, const AlForwardArgs* args, void* stream);

/* Whole backward.  Replaces what autograd derives from `TorchLinear.linear` (custom pieces:
 * torch_linear.py:44-54, 81-108; quant_utils.py:113-156) and `TritonLinear.backward`
 * (triton_linear.py:695-764). */
int al_backward(const AlDesc* desc, const AlBackwardArgs* args, void* stream);
int64_t al_backward_scratch_floats(int32_t M, int32_t K, int32_t N, int32_t T);
/* How the CUDA-core weight gradient (fp32 layers, unaligned tilings) cuts its reduction over the M
 * rows of the batch: `splits` CTAs per output block, `rows_per_split` rows each; with more than one
 * split, splits * N * K floats of reduce_scratch (behind the reductions) hold the partial sums.  A
 * function of the layer's sizes alone: the same whether or not the call carries a clamp mask. */
int al_wgrad_split_plan(int32_t M, int32_t K, int32_t N, int32_t T, int32_t* splits, int32_t* rows_per_split);
/* Work list of the backward GEMMs on CTA pairs: `num_blocks` output blocks of 256 x 256 walked by `n_pairs` pairs
 * (pair p takes items p, p + n_pairs, ...).  When the last round would keep at most half of the pairs busy (and at
 * most three full rounds precede it) its blocks are listed as two half blocks of 128 columns each (bf16 layers; the
 * plane products of fp32 layers always take whole blocks).  Returns the
 * length of the list in *total and, for 0 <= item < *total, the block of that item and which half of it (-1: the
 * whole block); *block = -1 for an item outside the list.  Host arithmetic, the functions the kernel itself calls. */
int al_pair_work_item(int32_t num_blocks, int32_t n_pairs, int32_t item, int32_t* total, int32_t* block, int32_t* half);
/* bf16 elements of AlBackwardArgs.g_planes for an fp32 layer on the tensor cores: the upstream
 * gradient as bf16 planes, per analog tile when the ADC clamp mask or a per-row DAC step has
 * to be folded in.  tile_ends_host as in the forward.  0 when the layer runs on the CUDA cores. */
int64_t al_backward_plane_elems(const AlDesc* desc, const int32_t* tile_ends_host);
/* Number of bf16 planes an fp32 operand is split into for the tensor cores (first dimension of w_planes). */
int32_t al_f32_planes(void);
/* floats of AlForwardArgs.smallm_scratch; 0 when the problem has more than 16 rows */
int64_t al_smallm_scratch_floats(int32_t M, int32_t N, int32_t T);

/* In-place weight clipping w <- clamp(w, +-sigma*std(w)), std over the whole tensor
 * (AL_CLIP_LAYER_GAUSSIAN) or per row (AL_CLIP_LAYER_GAUSSIAN_PER_CHANNEL).  Replaces
 * `AnalogLinear.clip_weights` (P/linear.py:269-283) / `_AnalogConvNd.clip_weights`
 * (P/conv.py:647-663).  scratch: >= 2*rows + 4 floats. */
int al_clip_weights(int32_t dtype, void* w, int32_t rows, int32_t cols, int32_t clip_type,
                    float sigma, float* scratch, void* stream);

/* Patch matrix of a 2-D convolution: out[b, l, c*kh*kw + i*kw + j] = x[b, c, oh*sh - ph + i*dh,
 * ow*sw - pw + j*dw] (zero outside the image), l = oh*Wo + ow.  x is [B,C,H,W] contiguous, out
 * [B, Ho*Wo, C*kh*kw].  Replaces `unfold(...).transpose(-1, -2).contiguous()` in
 * `_AnalogConvNd.forward` (P/conv.py:312-322).  al_fold2d is its adjoint (the backward of that
 * expression): grad_x[b,c,h,w] = sum of grad_patches over every patch position that read x[b,c,h,w]. */
int al_unfold2d(int32_t dtype, const void* x, int32_t B, int32_t C, int32_t H, int32_t W, int32_t kh, int32_t kw,
                int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw, void* out, void* stream);
/* al_unfold2d with the DAC of a dynamic input range fused in: writes the quantised patches xq
 * [B*Ho*Wo, C*kh*kw] and the per-(tile, patch) ranges ir_rows [T, B*Ho*Wo] that al_forward would
 * otherwise compute from the patch matrix (P/conv.py:312-322 followed by P/torch_utils/torch_linear.py:
 * 156, 182-192); the unquantised patch matrix is never written.  al_forward then runs with
 * AlForwardArgs.x_prequantised = 1.  codes16 (nullable): the integer DAC codes as bf16, same shape as
 * xq, for fp32 layers whose GEMMs run on the tensor cores (x_prequantised = 2); xq may be null when
 * codes16 is given.  AL_ERR_UNSUPPORTED when a patch does not fit one staged block: use al_unfold2d then. */
int al_unfold2d_dac(int32_t dtype, const void* x, int32_t B, int32_t C, int32_t H, int32_t W, int32_t kh, int32_t kw,
                    int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw,
                    const int32_t* tile_ends_host, int32_t T, double inp_res, void* xq, void* ir_rows, void* codes16,
                    void* stream);
int al_fold2d(int32_t dtype, const void* grad_patches, int32_t B, int32_t C, int32_t H, int32_t W, int32_t kh,
              int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw, void* grad_x,
              void* stream);
/* Input gradient of a convolution without the patch matrix: grad_x[b,c,h,w] = sum over taps (i, j) and output
 * channels n of grad_out[b, h+ph-i, w+pw-j, n] * w_mod[n, (c*kh+i)*kw+j] -- the same values as the product
 * grad_out @ w_mod of al_backward followed by al_fold2d (the autograd of P/conv.py:312-322 + P/torch_utils/
 * torch_linear.py:253), summed in another order.  For layers with few output channels the patch gradient costs more
 * to write and read back than these multiplications.  grad_out [B*Ho*Wo, N] and w_mod [N, C*kh*kw] (the modified
 * weights the forward multiplied with) are fp32; only for layers without an ADC clamp mask (out_bound <= 0), unit
 * stride, no dilation, padding smaller than the kernel, N and C multiples of 4: al_conv2d_input_grad_supported
 * returns 1 for those, and al_conv2d_input_grad returns AL_ERR_UNSUPPORTED otherwise. */
int al_conv2d_input_grad_supported(int32_t dtype, int32_t N, int32_t B, int32_t C, int32_t H, int32_t W, int32_t kh,
                                   int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw, int32_t dh, int32_t dw);
int al_conv2d_input_grad(int32_t dtype, const void* grad_out, const void* w_mod, int32_t N, int32_t B, int32_t C,
                         int32_t H, int32_t W, int32_t kh, int32_t kw, int32_t sh, int32_t sw, int32_t ph, int32_t pw,
                         int32_t dh, int32_t dw, void* grad_x, void* stream);

/* Element-wise operators of a decoder layer that sit between its analog linear layers, one pass each
 * (16-byte vectors, fp32 arithmetic, one rounding per result); the reference leaves them to PyTorch
 * (HF Phi-3 `modeling_phi3.py`: `apply_rotary_pos_emb`, `Phi3MLP.forward`), where the strided views of the
 * fused projections make them chains of slow element-wise kernels.
 *   al_swiglu_forward:  out[m, d] = silu(gate_up[m, d]) * gate_up[m, width + d],  gate_up [rows, 2 width]
 *   al_swiglu_backward: grad_gate_up [rows, 2 width] from gate_up and grad_out [rows, width]
 *   al_rotary_qkv: the rotary embedding of q and k (rotation of the two halves of each head by the angle
 *     of the row's position, position = row % seq_len, tables [seq_len, head_dim / 2] fp32) and a copy of
 *     v, from three [rows, heads, head_dim] inputs with a common row stride (the thirds of a fused qkv
 *     activation: in_k = in_q + heads * head_dim, row stride 3 * heads * head_dim) into three outputs with
 *     their own row stride.  inverse != 0: the transposed rotation, which is the backward (inputs: the
 *     three gradients, outputs: the thirds of the qkv gradient).
 * dtype AL_F32 or AL_BF16; pointers and row strides 16-byte aligned; width and head_dim / 2 multiples of
 * the vector length (4 fp32, 8 bf16). */
int al_swiglu_forward(int32_t dtype, const void* gate_up, int64_t rows, int32_t width, void* out, void* stream);
int al_swiglu_backward(int32_t dtype, const void* gate_up, const void* grad_out, int64_t rows, int32_t width,
                       void* grad_gate_up, void* stream);
int al_rotary_qkv(int32_t dtype, int32_t inverse, const void* in_q, const void* in_k, const void* in_v,
                  int64_t in_row_stride, const float* cos_table, const float* sin_table, int64_t rows, int32_t seq_len,
                  int32_t heads, int32_t head_dim, void* out_q, void* out_k, void* out_v, int64_t out_row_stride,
                  void* stream);

/* Device-side error word of the tcgen05 kernels (a bounded wait that gave up).  Reads and
 * clears it; synchronises `stream`.  0 = no error. */
int al_read_device_error(void* stream, uint32_t* out_code);

/* Every wait inside the tcgen05 kernels (on an mbarrier: a TMA copy, an MMA commit, a peer CTA) is
 * bounded by a wall-clock limit, 2 s by default; a wait that runs out sets the error word above,
 * the CTA drains its copies in flight, frees its tensor memory and returns -- the context stays
 * usable.  al_set_device_wait_limit_ns changes the limit for kernels launched afterwards on the
 * current device (0 restores the default).  al_debug_withhold_forward_signal(1) is a test aid:
 * the forward kernel then withholds the signal its output-stage warps wait for, so that their
 * wait runs out after the limit and the path above can be exercised; (0) restores normal
 * operation.  Neither has a counterpart in the reference. */
int al_set_device_wait_limit_ns(uint64_t ns);
int al_debug_withhold_forward_signal(int32_t on);

/* 1 if the given problem would run on the tcgen05/TMA kernels under AL_ENGINE_AUTO. */
int al_uses_tcgen05(const AlDesc* desc, const int32_t* tile_ends_host);

/* Launch accounting and optional per-kernel timing (no counterpart in the reference, whose
 * only timing aids are ad-hoc `triton.testing.do_bench` scripts, P/triton_utils/triton_abs_max.py:358-404).
 * Launch counts are always kept.  With profiling enabled every launch is bracketed by CUDA
 * events on its stream; al_profile_read waits for the recorded events (host-side wait only),
 * adds their elapsed times to the totals, copies AL_K_COUNT entries to `out` and optionally
 * resets the totals. */
enum AlKernelClass {
  AL_K_ABS_MAX = 0, AL_K_TILE_MAX, AL_K_STD, AL_K_IR_UPDATE, AL_K_DAC, AL_K_WEIGHT_MODIFY,
  AL_K_FWD_GEMM, AL_K_DGRAD_GEMM, AL_K_WGRAD_GEMM, AL_K_BIAS_GRAD, AL_K_IR_BACKWARD, AL_K_CLIP,
  AL_K_UNFOLD, AL_K_FOLD,
  AL_K_COUNT
};
typedef struct AlProfileEntry {
  int64_t launches;   /* kernel launches issued for this class                              */
  int64_t timed;      /* scopes that were timed with events                                 */
  double total_ms;    /* summed event time of the timed scopes                              */
} AlProfileEntry;
/* Data-parallel training overlaps the exchange of a layer's weight gradient with the computation
 * of its input gradient (the reference leaves that to DeepSpeed / DDP around
 * `TorchLinear.linear`'s autograd, P/torch_linear.py:116-314).  The backward GEMMs are persistent
 * kernels that occupy every SM, so a communication kernel enqueued beside them would only start
 * when they end: after al_reserve_sms(n) the backward GEMMs launched by the calling thread leave
 * n SMs unoccupied (n = 0 restores the default).  Returns the previous value. */
int al_reserve_sms(int32_t n);

/* Sum of a gradient buffer over the replicas of data-parallel training, over peer memory (NVLink /
 * NVSwitch), as one small kernel that runs beside the backward GEMMs.  The reference leaves gradient
 * exchange to DDP / DeepSpeed around its autograd (P/torch_utils/torch_linear.py:116-314 has no
 * exchange of its own); this entry point is what a data-parallel caller of this library uses
 * instead of a library all-reduce.
 *   buffer_ptrs[r], signal_pad_ptrs[r] (HOST arrays of `world` device addresses): rank r's copy of the
 *   exchanged buffer and its signal pad, as mapped into this process (symmetric memory: same size and
 *   layout on every rank; pads zero-initialised, at least 4 * (AL_PEER_SIGNAL_SLOT + 9) bytes, the
 *   32-bit words from AL_PEER_SIGNAL_SLOT on belong to this library);
 *   multicast_ptr: multicast address of the buffer (switch reduction, multimem) or 0 for plain peer
 *   loads and stores;  byte_offset / count: the part of the buffer to reduce (16-byte aligned, count a
 *   multiple of 8 bf16 / 4 fp32 elements);  call_index: 0, 1, 2, ... -- every rank passes the same
 *   number for the same exchange and a larger one for each later exchange on these pads;
 *   scale: factor applied to the sum (1 / world for the mean).
 * Every rank launches it on its own GPU; the kernels of the ranks signal and wait for one another
 * through the pads (waits bounded at 4 s: al_peer_read_error).  On return of the kernel the part of
 * the buffer holds the same bits on every rank.  Exchanges that share pads must not overlap. */
#define AL_PEER_SIGNAL_SLOT 192
int al_peer_allreduce(int32_t dtype, int32_t world, int32_t rank, const uint64_t* buffer_ptrs,
                      const uint64_t* signal_pad_ptrs, uint64_t multicast_ptr, int64_t byte_offset, int64_t count,
                      uint32_t call_index, float scale, int32_t n_ctas, void* stream);
/* Reads and clears the error word of al_peer_allreduce (a wait for a peer ran out): AL_ERR_DEVICE_TIMEOUT
 * if set.  The streams that ran the exchange must be idle. */
int al_peer_read_error(uint32_t* out_code);

int al_profile_enable(int on);
/* Which kernel classes are bracketed by events while profiling is on: bit c = class c (default: all).
 * Launches are counted for every class either way.  An event pair costs about a microsecond of stream
 * time, so a caller that times a whole step and one kernel inside it selects that kernel only. */
int al_profile_select(uint32_t class_mask);
int al_profile_read(AlProfileEntry* out, int reset);
const char* al_kernel_class_name(int kernel_class);

const char* al_status_str(int status);
const char* al_last_error(void); /* thread-local detail of the last non-zero status */
int al_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ANALOG_B200_H_ */
