// Gradient exchange of data-parallel training over peer memory (NVLink / NVSwitch), as a kernel of
// a few CTAs that runs beside the input-gradient GEMM instead of a library collective.
//
// Every rank holds the gradients in a buffer that all ranks have mapped (symmetric memory).  One
// launch per rank: (1) tell every peer "my buffer is complete" and wait for the same from all of
// them; (2) reduce this rank's 1/world slice -- read the slice from every rank (or let the switch
// add them up: multimem.ld_reduce), add in fp32 in rank order, scale, round once -- and write the
// result into every rank's buffer (or once to the multicast address: multimem.st); (3) tell every
// peer "my slice is written everywhere" and wait for all of them.  All ranks end with bit-identical
// gradients: each element is reduced by exactly one rank, in a fixed order, and broadcast.
//
// The signals are 32-bit counters in each rank's signal pad, one slot per source rank, that only
// grow: call number c uses the values 2c+1 (begin) and 2c+2 (end), so no slot is ever reset.
// Every wait is bounded (wall clock); a wait that runs out sets an error word, the kernel skips
// what depends on it and returns.
#include "analog_math.cuh"
#include "internal.h"

namespace al {

namespace {

constexpr int kMaxRanks = 8;
constexpr int kPeerThreads = 512;
constexpr unsigned long long kPeerWaitLimitNs = 4000000000ull;

__device__ uint32_t g_peer_error_word = 0;

struct PeerParams {
  int32_t world, rank, dtype;
  void* buf[kMaxRanks];       // the exchanged buffer in every rank (this rank's own at [rank])
  uint32_t* pad[kMaxRanks];   // signal slots of every rank: pad[r][s] = last value rank s sent to rank r
  uint32_t* counter;          // this rank's CTA counter (own memory, returns to 0)
  void* mc;                   // multicast address of the buffer (null: plain peer loads and stores)
  int64_t nvec;               // 16-byte vectors in the buffer
  uint32_t epoch;             // value of the begin signal; end signal = epoch + 1
  float scale;                // applied to the sum (1 / world for an average)
};

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void signal_peer(uint32_t* slot, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(slot), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t read_signal(const uint32_t* slot) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(slot) : "memory");
  return v;
}
// true when every rank's slot in this rank's pad has reached `value`
__device__ __forceinline__ bool wait_all(const PeerParams& p, uint32_t value, bool* shared_ok) {
  if (threadIdx.x < (unsigned)p.world) {
    const uint32_t* slot = p.pad[p.rank] + threadIdx.x;
    const uint64_t t0 = timer_ns();
    bool ok = true;
    // signed distance: the counters wrap after 2^31 calls
    while ((int32_t)(read_signal(slot) - value) < 0) {
      if (timer_ns() - t0 > kPeerWaitLimitNs) {
        ok = false;
        break;
      }
      __nanosleep(200);
    }
    if (!ok) {
      atomicOr(&g_peer_error_word, 1u);
      *shared_ok = false;
    }
  }
  __syncthreads();
  return *shared_ok;
}

__device__ __forceinline__ uint4 ld_peer(const void* base, int64_t v) {
  uint4 d;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(d.x), "=r"(d.y), "=r"(d.z), "=r"(d.w)
               : "l"(reinterpret_cast<const uint4*>(base) + v)
               : "memory");
  return d;
}
__device__ __forceinline__ void st_peer(void* base, int64_t v, uint4 d) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(reinterpret_cast<uint4*>(base) + v),
               "r"(d.x), "r"(d.y), "r"(d.z), "r"(d.w)
               : "memory");
}

template <int DT>
__device__ __forceinline__ void accumulate(uint4 d, float acc[8]) {
  const uint32_t w[4] = {d.x, d.y, d.z, d.w};
  if (DT == kBF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] = fadd(acc[2 * i], __uint_as_float(w[i] << 16));
      acc[2 * i + 1] = fadd(acc[2 * i + 1], __uint_as_float(w[i] & 0xffff0000u));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = fadd(acc[i], __uint_as_float(w[i]));
  }
}
template <int DT>
__device__ __forceinline__ uint4 finish(const float acc[8], float scale) {
  uint32_t w[4];
  if (DT == kBF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = (uint32_t)f32_to_bf16_bits(fmul(acc[2 * i], scale)) | ((uint32_t)f32_to_bf16_bits(fmul(acc[2 * i + 1], scale)) << 16);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __float_as_uint(fmul(acc[i], scale));
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <int DT>
__global__ void __launch_bounds__(kPeerThreads)
peer_allreduce_kernel(const PeerParams p) {
  __shared__ bool ok;
  __shared__ bool last;
  if (threadIdx.x == 0) ok = true;
  __syncthreads();
  // (1) this rank's buffer is complete (the kernel runs after the kernels that wrote it): tell everyone
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)p.world) {
    __threadfence_system();
    signal_peer(p.pad[threadIdx.x] + p.rank, p.epoch);
  }
  const bool ready = wait_all(p, p.epoch, &ok);

  // (2) this rank's slice: sum over the ranks in rank order, one rounding, broadcast
  if (ready) {
    const int64_t per = (p.nvec + p.world - 1) / p.world;
    const int64_t begin = (int64_t)p.rank * per;
    const int64_t end = begin + per < p.nvec ? begin + per : p.nvec;
    const int64_t stride = (int64_t)gridDim.x * kPeerThreads;
    if (p.mc != nullptr) {
      // the switch adds the ranks' copies (fp32 accumulation) and delivers the result to every rank
      constexpr int kUnroll = 4;  // reduced loads in flight per thread
      for (int64_t v0 = begin + ((int64_t)blockIdx.x * kPeerThreads + threadIdx.x) * kUnroll; v0 < end;
           v0 += stride * kUnroll) {
        uint4 d[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (v0 + u >= end) break;
          uint4* addr = reinterpret_cast<uint4*>(p.mc) + v0 + u;
          if (DT == kBF16)
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                         : "=r"(d[u].x), "=r"(d[u].y), "=r"(d[u].z), "=r"(d[u].w) : "l"(addr) : "memory");
          else
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(d[u].x), "=r"(d[u].y), "=r"(d[u].z), "=r"(d[u].w) : "l"(addr) : "memory");
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (v0 + u >= end) break;
          uint4* addr = reinterpret_cast<uint4*>(p.mc) + v0 + u;
          uint4 o = d[u];
          if (p.scale != 1.0f) {
            float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            accumulate<DT>(o, acc);
            o = finish<DT>(acc, p.scale);
          }
          if (DT == kBF16)
            asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(o.x),
                         "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
          else
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(o.x), "r"(o.y),
                         "r"(o.z), "r"(o.w) : "memory");
        }
      }
    } else {
      constexpr int kUnroll = 2;  // vectors per thread and turn: 2 x world 16-byte loads in flight
      for (int64_t v0 = begin + ((int64_t)blockIdx.x * kPeerThreads + threadIdx.x) * kUnroll; v0 < end;
           v0 += stride * kUnroll) {
        uint4 in[kUnroll][kMaxRanks];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r)
            if (r < p.world && v0 + u < end) in[u][r] = ld_peer(p.buf[r], v0 + u);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (v0 + u >= end) break;
          float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r)
            if (r < p.world) accumulate<DT>(in[u][r], acc);
          const uint4 out = finish<DT>(acc, p.scale);
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r)
            if (r < p.world) st_peer(p.buf[r], v0 + u, out);
        }
      }
    }
  }

  // (3) all of this rank's CTAs have written their part everywhere: tell everyone, wait for everyone
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(p.counter, 1u) + 1u;
    last = done == gridDim.x;
    if (last) atomicExch(p.counter, 0u);
  }
  __syncthreads();
  if (last && threadIdx.x < (unsigned)p.world) signal_peer(p.pad[threadIdx.x] + p.rank, p.epoch + 1u);
  wait_all(p, p.epoch + 1u, &ok);
}

}  // namespace

}  // namespace al

using namespace al;

extern "C" {

int al_peer_allreduce(int32_t dtype, int32_t world, int32_t rank, const uint64_t* buffer_ptrs,
                      const uint64_t* signal_pad_ptrs, uint64_t multicast_ptr, int64_t byte_offset, int64_t count,
                      uint32_t call_index, float scale, int32_t n_ctas, void* stream) {
  if (dtype != AL_F32 && dtype != AL_BF16) {
    set_error("al_peer_allreduce: unknown dtype %d", dtype);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || !buffer_ptrs || !signal_pad_ptrs) {
    set_error("al_peer_allreduce: world %d (1..%d), rank %d, or a null pointer table", world, kMaxRanks, rank);
    return AL_ERR_BAD_ARGUMENT;
  }
  const int64_t per_vec = dtype == AL_BF16 ? 8 : 4;
  if (count < 0 || count % per_vec != 0 || byte_offset % 16 != 0) {
    set_error("al_peer_allreduce: count %lld must be a multiple of %lld elements and the offset of 16 bytes",
              (long long)count, (long long)per_vec);
    return AL_ERR_BAD_ARGUMENT;
  }
  if (count == 0) return AL_OK;
  PeerParams p;
  p.world = world;
  p.rank = rank;
  p.dtype = dtype;
  for (int r = 0; r < kMaxRanks; ++r) {
    p.buf[r] = r < world ? reinterpret_cast<void*>(buffer_ptrs[r] + (uint64_t)byte_offset) : nullptr;
    p.pad[r] = r < world ? reinterpret_cast<uint32_t*>(signal_pad_ptrs[r]) + AL_PEER_SIGNAL_SLOT : nullptr;
  }
  p.counter = reinterpret_cast<uint32_t*>(signal_pad_ptrs[rank]) + AL_PEER_SIGNAL_SLOT + kMaxRanks;
  p.mc = multicast_ptr ? reinterpret_cast<void*>(multicast_ptr + (uint64_t)byte_offset) : nullptr;
  p.nvec = count / per_vec;
  p.epoch = 2u * call_index + 1u;
  p.scale = scale;
  int grid = n_ctas < 1 ? 1 : (n_ctas > 64 ? 64 : n_ctas);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == AL_BF16) peer_allreduce_kernel<kBF16><<<grid, kPeerThreads, 0, s>>>(p);
  else peer_allreduce_kernel<kF32><<<grid, kPeerThreads, 0, s>>>(p);
  return check_launch("peer_allreduce");
}

int al_peer_read_error(uint32_t* out_code) {
  if (!out_code) return AL_ERR_BAD_ARGUMENT;
  uint32_t zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out_code, g_peer_error_word, sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_peer_error_word, &zero, sizeof(uint32_t));
  if (e != cudaSuccess) {
    set_error("al_peer_read_error: %s", cudaGetErrorString(e));
    return AL_ERR_CUDA;
  }
  if (*out_code != 0) {
    set_error("a wait for a peer's signal ran out in al_peer_allreduce");
    return AL_ERR_DEVICE_TIMEOUT;
  }
  return AL_OK;
}

}  // extern "C"
