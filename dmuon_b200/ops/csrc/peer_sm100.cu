// Peer-memory kernels: flag signalling, bounded flag waits, reduce-to-owner
// fused with the Muon prologue, and owner -> reader pulls of published weights.
//
// Data moves with ordinary ld/st.global on peer-mapped symmetric memory; the
// only synchronisation is a monotonically increasing epoch per (rank, purpose)
// flag word written with st.release.sys and read with ld.acquire.sys.  Every
// wait has a cycle budget; when it runs out the kernel records status 4 and
// returns (the result of that launch is then invalid and the host raises).
//
// Replaces the reference's NCCL reduce-to-owner followed by a clone and a chain
// of elementwise kernels (dmuon/_backends/fsdp2/group.py:1095-1109, :1348-1352,
// dmuon/optim/muon.py:1687-1694) and its NCCL owner broadcast
// (dmuon/_backends/fsdp2/group.py:791-807).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "peer_sm100.cuh"
#include "ptx_sm100.cuh"

namespace dmuon {
void count_launch();

namespace {

constexpr int kBlock = 256;
constexpr int kVec = 8;

template <typename T>
struct Cv;
template <>
struct Cv<__nv_bfloat16> {
  static __device__ __forceinline__ float to(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from(float x) { return __float2bfloat16_rn(x); }
};
template <>
struct Cv<__half> {
  static __device__ __forceinline__ float to(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from(float x) { return __float2half_rn(x); }
};
template <>
struct Cv<float> {
  static __device__ __forceinline__ float to(float x) { return x; }
  static __device__ __forceinline__ float from(float x) { return x; }
};

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&v)[kVec]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < kVec; ++i) v[i] = Cv<T>::to(e[i]);
  } else {
    float4 a = reinterpret_cast<const float4*>(p)[0];
    float4 b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}

template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&v)[kVec]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < kVec; ++i) e[i] = Cv<T>::from(v[i]);
    *reinterpret_cast<uint4*>(p) = raw;
  } else {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

__device__ __forceinline__ bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ float blk_sum(float v) {
  __shared__ float part[kBlock / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x < kBlock / 32) ? part[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;
}

// One thread per block waits for `count` flags; the block learns the outcome.
__device__ __forceinline__ bool block_wait_flags(const int* flags, int first, int count, int want,
                                                 long long budget, int* status) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int i = 0; i < count && ok; ++i)
      if (!wait_flag_ge_sys(flags + first + i, want, budget)) ok = 0;
    if (!ok && status != nullptr) atomicCAS(status, 0, kStatusTimeoutPeerFlag);
    ok_s = ok;
  }
  __syncthreads();
  return ok_s != 0;
}

}  // namespace

__global__ void signal_peers_kernel(const DmuonSignalArgs a) {
  const int r = threadIdx.x;
  if (r < a.world) {
    __threadfence_system();
    st_release_sys(a.peer_flags[r] + a.slot, a.value);
  }
}

__global__ void wait_flags_kernel(const DmuonWaitArgs a) {
  block_wait_flags(a.local_flags, a.first, a.count, a.want, a.budget_cycles, a.status);
}

// kW: compile-time upper bound of the number of sources (1, 2, 4 or 8).  The per-thread buffer of loads in
// flight is kW x 8 floats, so the one-source form (a gradient already reduced in the switch) and the
// two-rank form keep four times the occupancy of the eight-rank form.
template <typename TG, typename TM, typename TX, int kW>
__global__ void __launch_bounds__(kBlock) peer_prologue_kernel(const DmuonPeerPrologueArgs a) {
  if (a.ready_flags != nullptr) {
    if (!block_wait_flags(a.ready_flags, 0, a.world, a.ready_want, a.budget_cycles, a.status)) return;
  }
  const int t = blockIdx.y;
  const long long off = a.offset[t];
  TM* m = reinterpret_cast<TM*>(a.mom[t]);
  TX* x = reinterpret_cast<TX*>(a.x[t]);
  const long long n = a.numel[t];
  const float gs = (a.gscale ? *a.gscale : 1.f) * a.scale;
  const float xs = a.xscale ? a.xscale[a.slot[t]] : 1.f;
  const float mu = a.mu;
  const int W = a.world;
  const TG* g[kW];
#pragma unroll
  for (int r = 0; r < kW; ++r)
    g[r] = (r < W) ? reinterpret_cast<const TG*>(a.peer_base[r]) + off : nullptr;
  bool vec = al16(x) && (m == nullptr || al16(m));
#pragma unroll
  for (int r = 0; r < kW; ++r)
    if (r < W) vec = vec && al16(g[r]);
  const long long nvec = vec ? (n / kVec) : 0;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  float acc = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < nvec; i += stride) {
    float sum[kVec];
#pragma unroll
    for (int k = 0; k < kVec; ++k) sum[k] = 0.f;
    // all peer loads are issued before the first use: W independent 16-byte
    // requests in flight per thread
    float gv[kW][kVec];
#pragma unroll
    for (int r = 0; r < kW; ++r)
      if (r < W) ld8<TG>(g[r] + i * kVec, gv[r]);
#pragma unroll
    for (int r = 0; r < kW; ++r)
      if (r < W) {
#pragma unroll
        for (int k = 0; k < kVec; ++k) sum[k] += gv[r][k];
      }
    float uv[kVec];
    if (m != nullptr) {
      float mv[kVec];
      ld8<TM>(m + i * kVec, mv);
#pragma unroll
      for (int k = 0; k < kVec; ++k) {
        const float gg = sum[k] * gs;
        mv[k] = Cv<TM>::to(Cv<TM>::from(fmaf(mu, mv[k], gg)));
        uv[k] = a.nesterov ? fmaf(mu, mv[k], gg) : mv[k];
      }
      st8<TM>(m + i * kVec, mv);
    } else {
#pragma unroll
      for (int k = 0; k < kVec; ++k) uv[k] = sum[k] * gs;
    }
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
      acc = fmaf(uv[k], uv[k], acc);
      uv[k] *= xs;
    }
    st8<TX>(x + i * kVec, uv);
  }
  for (long long i = nvec * kVec + static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < n;
       i += stride) {
    float s = 0.f;
    for (int r = 0; r < W; ++r) s += Cv<TG>::to(g[r][i]);
    const float gg = s * gs;
    float u = gg;
    if (m != nullptr) {
      const TM mn = Cv<TM>::from(fmaf(mu, Cv<TM>::to(m[i]), gg));
      m[i] = mn;
      u = a.nesterov ? fmaf(mu, Cv<TM>::to(mn), gg) : Cv<TM>::to(mn);
    }
    x[i] = Cv<TX>::from(u * xs);
    acc = fmaf(u, u, acc);
  }
  const float total = blk_sum(acc);
  if (threadIdx.x == 0 && a.sumsq != nullptr && !(total == 0.f)) atomicAdd(a.sumsq + a.slot[t], total);
}

__global__ void __launch_bounds__(kBlock) peer_pull_kernel(const DmuonPullArgs a) {
  const int t = blockIdx.y;
  if (a.local_flags != nullptr) {
    if (!block_wait_flags(a.local_flags, a.flag_slot[t], 1, a.want, a.budget_cycles, a.status)) return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(a.src[t]);
  uint4* dst = reinterpret_cast<uint4*>(a.dst[t]);
  const long long n16 = a.nbytes[t] >> 4;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x;
  // four independent 16-byte peer loads in flight per thread
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 v0 = src[i], v1 = src[i + stride], v2 = src[i + 2 * stride], v3 = src[i + 3 * stride];
    dst[i] = v0; dst[i + stride] = v1; dst[i + 2 * stride] = v2; dst[i + 3 * stride] = v3;
  }
  for (; i < n16; i += stride) dst[i] = src[i];
}

// mode 0: local <- in-switch sum over all ranks; mode 1: all ranks <- local.
template <int kDtype>
__global__ void __launch_bounds__(kBlock) multicast_copy_kernel(const DmuonMulticastArgs a) {
  const int t = blockIdx.y;
  const long long n16 = a.nbytes[t] >> 4;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x;
  if (a.mode == 0) {
    const uint4* src = reinterpret_cast<const uint4*>(a.src[t]);
    uint4* dst = reinterpret_cast<uint4*>(a.dst[t]);
    auto ldr = [](const uint4* p) {
      if constexpr (kDtype == DMUON_BF16) return multimem_ld_reduce_bf16x8(p);
      else if constexpr (kDtype == DMUON_FP16) return multimem_ld_reduce_f16x8(p);
      else return multimem_ld_reduce_f32x4(p);
    };
    // four independent reduce-loads in flight per thread
    for (; i + 3 * stride < n16; i += 4 * stride) {
      const uint4 v0 = ldr(src + i), v1 = ldr(src + i + stride), v2 = ldr(src + i + 2 * stride),
                  v3 = ldr(src + i + 3 * stride);
      dst[i] = v0; dst[i + stride] = v1; dst[i + 2 * stride] = v2; dst[i + 3 * stride] = v3;
    }
    for (; i < n16; i += stride) dst[i] = ldr(src + i);
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(a.src[t]);
    uint4* dst = reinterpret_cast<uint4*>(a.dst[t]);
    for (; i < n16; i += stride) multimem_st_16B(dst + i, src[i]);
  }
}

static int sm_count() {
  static int cached[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static int grid_x(long long max_items, int ntensors, int override_blocks) {
  if (override_blocks > 0) return override_blocks;
  const long long sms = sm_count();
  long long need = (max_items + kBlock - 1) / kBlock;
  long long cap = (sms * 4 + ntensors - 1) / ntensors;
  if (cap < sms * 2) cap = sms * 2;
  long long b = need < cap ? need : cap;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace dmuon

using namespace dmuon;

#define DMUON_PEER_DISPATCH(code, T, ...)                             \
  switch (code) {                                                     \
    case DMUON_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case DMUON_FP16: { using T = __half; __VA_ARGS__; break; }        \
    default: { using T = float; __VA_ARGS__; break; }                 \
  }

extern "C" int dmuon_signal_peers(const DmuonSignalArgs* a, void* stream_v) {
  if (a->world <= 0 || a->world > DMUON_MAX_PEERS) return -1;
  signal_peers_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_wait_flags(const DmuonWaitArgs* a, void* stream_v) {
  if (a->count <= 0) return 0;
  wait_flags_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_peer_prologue(const DmuonPeerPrologueArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS || a->world <= 0 || a->world > DMUON_MAX_PEERS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  long long mx = 0;
  for (int i = 0; i < a->n; ++i) mx = a->numel[i] > mx ? a->numel[i] : mx;
  dim3 grid(grid_x((mx + kVec - 1) / kVec, a->n, a->max_blocks_per_tensor), a->n);
#define DMUON_PEER_PROLOGUE_LAUNCH(KW)                                                                     \
  DMUON_PEER_DISPATCH(a->grad_dtype, TG,                                                                  \
    DMUON_PEER_DISPATCH(a->mom_dtype, TM,                                                                 \
      DMUON_PEER_DISPATCH(a->x_dtype, TX, peer_prologue_kernel<TG, TM, TX, KW><<<grid, kBlock, 0, st>>>(*a))))
  if (a->world <= 1) {
    DMUON_PEER_PROLOGUE_LAUNCH(1);
  } else if (a->world <= 2) {
    DMUON_PEER_PROLOGUE_LAUNCH(2);
  } else if (a->world <= 4) {
    DMUON_PEER_PROLOGUE_LAUNCH(4);
  } else {
    DMUON_PEER_PROLOGUE_LAUNCH(8);
  }
#undef DMUON_PEER_PROLOGUE_LAUNCH
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_peer_pull(const DmuonPullArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS) return -1;
  long long mx = 0;
  for (int i = 0; i < a->n; ++i) {
    if ((a->nbytes[i] & 15) || (reinterpret_cast<uintptr_t>(a->src[i]) & 15) ||
        (reinterpret_cast<uintptr_t>(a->dst[i]) & 15))
      return -1;
    mx = a->nbytes[i] > mx ? a->nbytes[i] : mx;
  }
  dim3 grid(grid_x(mx >> 4, a->n, a->blocks_per_tensor), a->n);
  peer_pull_kernel<<<grid, kBlock, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_multicast_copy(const DmuonMulticastArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS || (a->mode != 0 && a->mode != 1)) return -1;
  long long mx = 0;
  for (int i = 0; i < a->n; ++i) {
    if ((a->nbytes[i] & 15) || (reinterpret_cast<uintptr_t>(a->src[i]) & 15) ||
        (reinterpret_cast<uintptr_t>(a->dst[i]) & 15))
      return -1;
    mx = a->nbytes[i] > mx ? a->nbytes[i] : mx;
  }
  dim3 grid(grid_x(mx >> 4, a->n, a->blocks_per_tensor), a->n);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  switch (a->dtype) {
    case DMUON_BF16: multicast_copy_kernel<DMUON_BF16><<<grid, kBlock, 0, st>>>(*a); break;
    case DMUON_FP16: multicast_copy_kernel<DMUON_FP16><<<grid, kBlock, 0, st>>>(*a); break;
    default: multicast_copy_kernel<DMUON_FP32><<<grid, kBlock, 0, st>>>(*a); break;
  }
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

namespace dmuon {
__global__ void scalar_allreduce_kernel(const DmuonScalarAllreduceArgs a) {
  const int t = threadIdx.x;
  const int par = a.epoch & 1;
  float* mine = a.peer_vals[a.rank] + par * DMUON_SCALAR_MAX;
  if (t < a.n) mine[t] = a.local[t];
  __threadfence_system();
  __syncwarp();
  if (t < a.world) st_release_sys(a.peer_flags[t] + par * DMUON_MAX_PEERS + a.rank, a.epoch);
  bool ok = true;
  if (t < a.world) ok = wait_flag_ge_sys(a.peer_flags[a.rank] + par * DMUON_MAX_PEERS + t, a.epoch, a.budget_cycles);
  const unsigned all_ok = __ballot_sync(0xffffffffu, ok);
  if (all_ok != 0xffffffffu) {
    if (t == 0) atomicCAS(a.status, 0, 4);
    return;                                   // sums stay untouched; the host raises on the status word
  }
  __threadfence_system();
  if (t < a.n) {
    float s = 0.f;
    for (int r = 0; r < a.world; ++r) {
      const volatile float* v = a.peer_vals[r] + par * DMUON_SCALAR_MAX;
      s += v[t];                              // fixed rank order: the same bits on every rank
    }
    a.out[t] = s;
    if (a.coef != nullptr) a.coef[t] = fminf(1.f, a.max_norm / (sqrtf(s) + 1e-6f));
  }
}
}  // namespace dmuon

extern "C" int dmuon_scalar_allreduce(const DmuonScalarAllreduceArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_SCALAR_MAX || a->world <= 0 || a->world > DMUON_MAX_PEERS || a->rank < 0 || a->rank >= a->world)
    return -22;
  scalar_allreduce_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(*a);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// One asynchronous copy on the copy engines (no SM is involved, so transfers
// that overlap forward / backward GEMMs take nothing from them).  Either
// pointer may be a peer mapping of another GPU's symmetric buffer.
extern "C" int dmuon_copy_async(void* dst, const void* src, long long nbytes, void* stream_v) {
  if (nbytes <= 0) return 0;
  return static_cast<int>(
      cudaMemcpyAsync(dst, src, static_cast<size_t>(nbytes), cudaMemcpyDefault, reinterpret_cast<cudaStream_t>(stream_v)));
}
