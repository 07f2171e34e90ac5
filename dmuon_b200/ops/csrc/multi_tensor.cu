// Multi-tensor elementwise kernels for sm_100a: Muon prologue (momentum,
// Nesterov, cast, Frobenius norm), AdamW, clip sum-of-squares / scale, casts.
//
// All of them are HBM-bound, so each thread moves 8 elements per step with
// 128-bit accesses and every tensor is touched exactly once.  They replace
// chains of ATen foreach kernels in the reference (dmuon/optim/muon.py:1687-1694
// momentum, :1901-1916 AdamW, dmuon/optim/newton_schulz.py:371-379 normalise,
// dmuon/csrc/fast_clip_kernel.cu:34-106 clip).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "multi_tensor.cuh"
#include "vec8.cuh"

namespace dmuon {
void count_launch();

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float warp_part[kBlock / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) warp_part[w] = v;
  __syncthreads();
  float t = (threadIdx.x < kBlock / 32) ? warp_part[threadIdx.x] : 0.f;
  if (w == 0) {
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;  // valid on thread 0
}

// dispatch a runtime dtype code to a template parameter
#define DMUON_DISPATCH(code, T, ...)                      \
  switch (code) {                                         \
    case DMUON_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case DMUON_FP16: { using T = __half; __VA_ARGS__; break; }        \
    default: { using T = float; __VA_ARGS__; break; }                 \
  }

// ---------------------------------------------------------------- Muon prologue
template <typename TG, typename TM, typename TX>
__global__ void __launch_bounds__(kBlock) prologue_kernel(const DmuonPrologueArgs a) {
  const int t = blockIdx.y;
  const TG* g = reinterpret_cast<const TG*>(a.grad[t]);
  TM* m = reinterpret_cast<TM*>(a.mom[t]);
  TX* x = reinterpret_cast<TX*>(a.x[t]);
  const long long n = a.numel[t];
  const float gs = a.gscale ? *a.gscale : 1.f;
  const float xs = a.xscale ? a.xscale[a.slot[t]] : 1.f;
  const float mu = a.mu;
  float acc = 0.f;
  const bool vec = aligned16(g) && aligned16(m) && aligned16(x);
  const long long nvec = vec ? (n / kVec) : 0;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < nvec; i += stride) {
    float gv[kVec], mv[kVec], uv[kVec];
    load8<TG>(g + i * kVec, gv);
    load8<TM>(m + i * kVec, mv);
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
      const float gg = gv[k] * gs;
      // round the stored momentum first so that u uses what the next step will read
      mv[k] = Conv<TM>::to(Conv<TM>::from(fmaf(mu, mv[k], gg)));
      uv[k] = a.nesterov ? fmaf(mu, mv[k], gg) : mv[k];
      acc = fmaf(uv[k], uv[k], acc);
      uv[k] *= xs;
    }
    store8<TM>(m + i * kVec, mv);
    store8<TX>(x + i * kVec, uv);
  }
  for (long long i = nvec * kVec + static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < n;
       i += stride) {
    const float gg = Conv<TG>::to(g[i]) * gs;
    const TM mn = Conv<TM>::from(fmaf(mu, Conv<TM>::to(m[i]), gg));
    m[i] = mn;
    const float u = a.nesterov ? fmaf(mu, Conv<TM>::to(mn), gg) : Conv<TM>::to(mn);
    x[i] = Conv<TX>::from(u * xs);
    acc = fmaf(u, u, acc);
  }
  const float total = block_sum(acc);
  if (threadIdx.x == 0 && total != 0.f) atomicAdd(a.sumsq + a.slot[t], total);
}

__global__ void norm_scales_kernel(const DmuonNormArgs a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < a.n) {
    const float s = 1.f / (sqrtf(a.sumsq[i]) + a.eps);
    a.scale[i] = s;
    a.scale2[i] = s * s;
  }
}

// ---------------------------------------------------------------- AdamW
template <typename TP, typename TG, typename TS>
__global__ void __launch_bounds__(kBlock) adamw_kernel(const DmuonAdamWArgs a) {
  const int t = blockIdx.y;
  TP* p = reinterpret_cast<TP*>(a.param[t]);
  const TG* g = reinterpret_cast<const TG*>(a.grad[t]);
  TS* m = reinterpret_cast<TS*>(a.exp_avg[t]);
  TS* v = reinterpret_cast<TS*>(a.exp_avg_sq[t]);
  __nv_bfloat16* pub = reinterpret_cast<__nv_bfloat16*>(a.publish[t]);
  const long long n = a.numel[t];
  const float gs = a.gscale ? *a.gscale : 1.f;
  const float decay = 1.f - a.lr * a.weight_decay;
  const float step_size = a.step_size[t];
  const float isb2 = a.inv_sqrt_bc2[t];
  const float b1 = a.beta1, b2 = a.beta2, eps = a.eps;
  const bool vec = aligned16(p) && aligned16(g) && aligned16(m) && aligned16(v) && (!pub || aligned16(pub));
  const long long nvec = vec ? (n / kVec) : 0;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < nvec; i += stride) {
    float pv[kVec], gv[kVec], mv[kVec], vv[kVec];
    load8<TP>(p + i * kVec, pv);
    load8<TG>(g + i * kVec, gv);
    load8<TS>(m + i * kVec, mv);
    load8<TS>(v + i * kVec, vv);
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
      const float gg = gv[k] * gs;
      mv[k] = fmaf(b1, mv[k], (1.f - b1) * gg);
      vv[k] = fmaf(b2, vv[k], (1.f - b2) * gg * gg);
      const float denom = sqrtf(vv[k]) * isb2 + eps;
      pv[k] = pv[k] * decay - step_size * (mv[k] / denom);
    }
    store8<TP>(p + i * kVec, pv);
    store8<TS>(m + i * kVec, mv);
    store8<TS>(v + i * kVec, vv);
    if (pub) store8<__nv_bfloat16>(pub + i * kVec, pv);
  }
  for (long long i = nvec * kVec + static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < n;
       i += stride) {
    const float gg = Conv<TG>::to(g[i]) * gs;
    const float mm = fmaf(b1, Conv<TS>::to(m[i]), (1.f - b1) * gg);
    const float vv = fmaf(b2, Conv<TS>::to(v[i]), (1.f - b2) * gg * gg);
    const float denom = sqrtf(vv) * isb2 + eps;
    const float pn = Conv<TP>::to(p[i]) * decay - step_size * (mm / denom);
    p[i] = Conv<TP>::from(pn);
    m[i] = Conv<TS>::from(mm);
    v[i] = Conv<TS>::from(vv);
    if (pub) pub[i] = __float2bfloat16_rn(pn);
  }
}

// ---------------------------------------------------------------- clip
template <typename T>
__device__ __forceinline__ float sumsq_tensor(const T* x, long long n) {
  float acc = 0.f;
  const bool vec = aligned16(x);
  const long long nvec = vec ? (n / kVec) : 0;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < nvec; i += stride) {
    float v[kVec];
    load8<T>(x + i * kVec, v);
#pragma unroll
    for (int k = 0; k < kVec; ++k) acc = fmaf(v[k], v[k], acc);
  }
  for (long long i = nvec * kVec + static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < n;
       i += stride) {
    const float v = Conv<T>::to(x[i]);
    acc = fmaf(v, v, acc);
  }
  return acc;
}

__global__ void __launch_bounds__(kBlock) clip_sumsq_kernel(const DmuonClipArgs a) {
  const int t = blockIdx.y;
  float acc;
  DMUON_DISPATCH(a.dtype[t], T, acc = sumsq_tensor<T>(reinterpret_cast<const T*>(a.tensor[t]), a.numel[t]));
  const float total = block_sum(acc);
  // a NaN/Inf partial sum must reach the segment total, so no "!= 0" shortcut on it
  if (threadIdx.x == 0 && !(total == 0.f)) atomicAdd(a.seg_sumsq + a.segment[t], total);
}

template <typename T>
__device__ __forceinline__ void scale_tensor(T* x, long long n, float c) {
  const bool vec = aligned16(x);
  const long long nvec = vec ? (n / kVec) : 0;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < nvec; i += stride) {
    float v[kVec];
    load8<T>(x + i * kVec, v);
#pragma unroll
    for (int k = 0; k < kVec; ++k) v[k] *= c;
    store8<T>(x + i * kVec, v);
  }
  for (long long i = nvec * kVec + static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < n;
       i += stride)
    x[i] = Conv<T>::from(Conv<T>::to(x[i]) * c);
}

__global__ void __launch_bounds__(kBlock) clip_scale_kernel(const DmuonClipArgs a) {
  const int t = blockIdx.y;
  const float c = a.seg_coef[a.segment[t]];
  DMUON_DISPATCH(a.dtype[t], T, scale_tensor<T>(reinterpret_cast<T*>(a.tensor[t]), a.numel[t], c));
}

// ---------------------------------------------------------------- cast
template <typename TS, typename TD>
__global__ void __launch_bounds__(kBlock) cast_kernel(const DmuonCastArgs a) {
  const int t = blockIdx.y;
  const TS* s = reinterpret_cast<const TS*>(a.src[t]);
  TD* d = reinterpret_cast<TD*>(a.dst[t]);
  const long long n = a.numel[t];
  const float c = a.scale ? a.scale[a.slot[t]] : 1.f;
  const bool vec = aligned16(s) && aligned16(d);
  const long long nvec = vec ? (n / kVec) : 0;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  for (long long i = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < nvec; i += stride) {
    float v[kVec];
    load8<TS>(s + i * kVec, v);
#pragma unroll
    for (int k = 0; k < kVec; ++k) v[k] *= c;
    store8<TD>(d + i * kVec, v);
  }
  for (long long i = nvec * kVec + static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; i < n;
       i += stride)
    d[i] = Conv<TD>::from(Conv<TS>::to(s[i]) * c);
}

static int blocks_per_tensor(int ntensors, const long long* numel) {
  long long mx = 0;
  for (int i = 0; i < ntensors; ++i) mx = numel[i] > mx ? numel[i] : mx;
  long long need = (mx + static_cast<long long>(kBlock) * kVec - 1) / (static_cast<long long>(kBlock) * kVec);
  // About 8 resident blocks per SM overall when the tensors are alike, but never
  // fewer than 4 per SM for one row: a launch that mixes one huge tensor with
  // many small ones (embedding + norms) must still fill the GPU for the huge
  // one; surplus blocks of small rows exit at once.
  long long cap = (148LL * 8 + ntensors - 1) / ntensors;
  if (cap < 148LL * 4) cap = 148LL * 4;
  long long b = need < cap ? need : cap;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace dmuon

using namespace dmuon;

extern "C" int dmuon_muon_prologue(const DmuonPrologueArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid(blocks_per_tensor(a->n, a->numel), a->n);
  DMUON_DISPATCH(a->grad_dtype, TG,
    DMUON_DISPATCH(a->mom_dtype, TM,
      DMUON_DISPATCH(a->x_dtype, TX, prologue_kernel<TG, TM, TX><<<grid, kBlock, 0, st>>>(*a))));
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_norm_scales(const DmuonNormArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  norm_scales_kernel<<<(a->n + 127) / 128, 128, 0, st>>>(*a);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_adamw(const DmuonAdamWArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid(blocks_per_tensor(a->n, a->numel), a->n);
  DMUON_DISPATCH(a->param_dtype, TP,
    DMUON_DISPATCH(a->grad_dtype, TG,
      DMUON_DISPATCH(a->state_dtype, TS, adamw_kernel<TP, TG, TS><<<grid, kBlock, 0, st>>>(*a))));
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_clip_sumsq(const DmuonClipArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid(blocks_per_tensor(a->n, a->numel), a->n);
  clip_sumsq_kernel<<<grid, kBlock, 0, st>>>(*a);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_clip_scale(const DmuonClipArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid(blocks_per_tensor(a->n, a->numel), a->n);
  clip_scale_kernel<<<grid, kBlock, 0, st>>>(*a);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_cast(const DmuonCastArgs* a, void* stream_v) {
  if (a->n <= 0) return 0;
  if (a->n > DMUON_MAX_TENSORS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  dim3 grid(blocks_per_tensor(a->n, a->numel), a->n);
  DMUON_DISPATCH(a->src_dtype, TS,
    DMUON_DISPATCH(a->dst_dtype, TD, cast_kernel<TS, TD><<<grid, kBlock, 0, st>>>(*a)));
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
