// Tensor-parallel gather + prologue and pull + apply over peer memory
// (see tp_peer_sm100.cuh).  Elementwise, HBM / NVLink bound: 8 elements per
// thread and step with 128-bit accesses whenever the shard width, the pitch and
// the base addresses allow it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "tp_peer_sm100.cuh"
#include "vec8.cuh"

namespace dmuon {
void count_launch();

namespace {

__device__ __forceinline__ float tp_block_sum(float v) {
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

template <typename TG, typename TM, typename TX>
__global__ void __launch_bounds__(kBlock) tp_gather_prologue_kernel(const DmuonTpGatherArgs a) {
  const int t = blockIdx.y;
  const TG* g = reinterpret_cast<const TG*>(a.src[t]);
  TM* m = reinterpret_cast<TM*>(a.mom[t]);
  TX* x = reinterpret_cast<TX*>(a.x[t]);
  const long long rows = a.rows[t], cols = a.cols[t], pitch = a.pitch[t];
  const float gs = a.gscale ? *a.gscale : 1.f;
  const float xs = a.xscale ? a.xscale[a.slot[t]] : 1.f;
  const float mu = a.mu;
  float acc = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  const bool vec = (cols % kVec) == 0 && (pitch % kVec) == 0 && aligned16(g) && aligned16(x) &&
                   (m == nullptr || aligned16(m));
  if (vec) {
    const long long cv = cols / kVec;
    const long long nv = rows * cv;
    for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < nv; i += stride) {
      const long long r = i / cv, c = (i - r * cv) * kVec;
      const long long d = r * pitch + c;
      float gv[kVec], uv[kVec];
      load8<TG>(g + r * cols + c, gv);
      if (m != nullptr) {
        float mv[kVec];
        load8<TM>(m + d, mv);
#pragma unroll
        for (int k = 0; k < kVec; ++k) {
          const float gg = gv[k] * gs;
          mv[k] = Conv<TM>::to(Conv<TM>::from(fmaf(mu, mv[k], gg)));
          uv[k] = a.nesterov ? fmaf(mu, mv[k], gg) : mv[k];
        }
        store8<TM>(m + d, mv);
      } else {
#pragma unroll
        for (int k = 0; k < kVec; ++k) uv[k] = gv[k] * gs;
      }
#pragma unroll
      for (int k = 0; k < kVec; ++k) {
        acc = fmaf(uv[k], uv[k], acc);
        uv[k] *= xs;
      }
      store8<TX>(x + d, uv);
    }
  } else {
    const long long n = rows * cols;
    for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < n; i += stride) {
      const long long r = i / cols, c = i - r * cols;
      const long long d = r * pitch + c;
      const float gg = Conv<TG>::to(g[i]) * gs;
      float u = gg;
      if (m != nullptr) {
        const TM mn = Conv<TM>::from(fmaf(mu, Conv<TM>::to(m[d]), gg));
        m[d] = mn;
        u = a.nesterov ? fmaf(mu, Conv<TM>::to(mn), gg) : Conv<TM>::to(mn);
      }
      x[d] = Conv<TX>::from(u * xs);
      acc = fmaf(u, u, acc);
    }
  }
  const float total = tp_block_sum(acc);
  if (threadIdx.x == 0 && a.sumsq != nullptr && !(total == 0.f)) atomicAdd(a.sumsq + a.slot[t], total);
}

template <typename TD>
__global__ void __launch_bounds__(kBlock) tp_apply_delta_kernel(const DmuonTpApplyArgs a) {
  const int t = blockIdx.y;
  const float* s = a.src[t];
  TD* w = reinterpret_cast<TD*>(a.dst[t]);
  const long long rows = a.rows[t], cols = a.cols[t], pitch = a.pitch[t];
  const float decay = a.decay[t];
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  const bool vec = (cols % kVec) == 0 && (pitch % kVec) == 0 && aligned16(s) && aligned16(w);
  if (vec) {
    const long long cv = cols / kVec;
    const long long nv = rows * cv;
    for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < nv; i += stride) {
      const long long r = i / cv, c = (i - r * cv) * kVec;
      float dv[kVec], wv[kVec];
      load8<float>(s + r * pitch + c, dv);
      load8<TD>(w + r * cols + c, wv);
#pragma unroll
      for (int k = 0; k < kVec; ++k) wv[k] = fmaf(wv[k], decay, dv[k]);
      store8<TD>(w + r * cols + c, wv);
    }
  } else {
    const long long n = rows * cols;
    for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < n; i += stride) {
      const long long r = i / cols, c = i - r * cols;
      w[i] = Conv<TD>::from(fmaf(Conv<TD>::to(w[i]), decay, s[r * pitch + c]));
    }
  }
}

int tp_grid_x(long long max_items, int ntensors) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms = n;
  }
  long long need = (max_items + kBlock - 1) / kBlock;
  long long cap = (static_cast<long long>(sms) * 4 + ntensors - 1) / ntensors;
  if (cap < 2LL * sms) cap = 2LL * sms;
  long long b = need < cap ? need : cap;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace
}  // namespace dmuon

using namespace dmuon;

#define DMUON_TP_DISPATCH(code, T, ...)                               \
  switch (code) {                                                     \
    case DMUON_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case DMUON_FP16: { using T = __half; __VA_ARGS__; break; }        \
    default: { using T = float; __VA_ARGS__; break; }                 \
  }

extern "C" int dmuon_tp_gather_prologue(const DmuonTpGatherArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS) return -1;
  long long mx = 0;
  for (int i = 0; i < a->n; ++i) {
    if (a->rows[i] <= 0 || a->cols[i] <= 0 || a->pitch[i] < a->cols[i] || a->src[i] == nullptr || a->x[i] == nullptr)
      return -1;
    const long long items = static_cast<long long>(a->rows[i]) * a->cols[i];
    mx = items > mx ? items : mx;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid(tp_grid_x((mx + kVec - 1) / kVec, a->n), a->n);
  DMUON_TP_DISPATCH(a->src_dtype, TG,
    DMUON_TP_DISPATCH(a->mom_dtype, TM,
      DMUON_TP_DISPATCH(a->x_dtype, TX, tp_gather_prologue_kernel<TG, TM, TX><<<grid, kBlock, 0, st>>>(*a))));
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_tp_apply_delta(const DmuonTpApplyArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS) return -1;
  long long mx = 0;
  for (int i = 0; i < a->n; ++i) {
    if (a->rows[i] <= 0 || a->cols[i] <= 0 || a->pitch[i] < a->cols[i] || a->src[i] == nullptr || a->dst[i] == nullptr)
      return -1;
    const long long items = static_cast<long long>(a->rows[i]) * a->cols[i];
    mx = items > mx ? items : mx;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid(tp_grid_x((mx + kVec - 1) / kVec, a->n), a->n);
  DMUON_TP_DISPATCH(a->dst_dtype, TD, tp_apply_delta_kernel<TD><<<grid, kBlock, 0, st>>>(*a));
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
