// Fused activation-side kernels for sm_100a: SwiGLU forward / backward, rotary
// embedding in place on the projection outputs, softmax cross-entropy that
// leaves the logit gradient in the logit buffer.
//
// All are HBM-bound: 128-bit accesses, fp32 arithmetic, each tensor read once
// and written once.  The cross-entropy runs one 1024-thread block per row, so
// at most two rows per SM are in flight (296 rows x 256 KB for a 128k bf16
// vocabulary = 76 MB, inside the 126 MB L2) and the gradient pass re-reads the
// row from L2, not from HBM.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "model_ops.cuh"
#include "multi_tensor.cuh"
#include "vec8.cuh"

namespace dmuon {
void count_launch();

namespace {

constexpr int kSmCount = 148;

#define DMUON_MODEL_DISPATCH(code, T, ...)                            \
  switch (code) {                                                     \
    case DMUON_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case DMUON_FP16: { using T = __half; __VA_ARGS__; break; }        \
    case DMUON_FP32: { using T = float; __VA_ARGS__; break; }         \
    default: return -22;                                              \
  }

inline int grid_for(long long work_items) {
  long long blocks = (work_items + kBlock - 1) / kBlock;
  const long long cap = static_cast<long long>(kSmCount) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

__device__ __forceinline__ float sigmoidf_fast(float x) { return 1.f / (1.f + __expf(-x)); }

// Gate activations of the gated MLPs: value and derivative in one go.
//   ACT 0: silu(x) = x sigmoid(x)          ACT 1: gelu, tanh approximation
template <int ACT>
__device__ __forceinline__ void act_and_grad(float x, float& y, float& dy) {
  if constexpr (ACT == 0) {
    const float s = sigmoidf_fast(x);
    y = x * s;
    dy = s + y * (1.f - s);
  } else {
    const float k = 0.7978845608028654f, c = 0.044715f;
    const float inner = k * (x + c * x * x * x);
    const float t = 1.f - 2.f / (1.f + __expf(2.f * inner));   // tanh(inner)
    y = 0.5f * x * (1.f + t);
    dy = 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * c * x * x);
  }
}

// ---------------------------------------------------------------- SwiGLU
template <typename T, int ACT>
__global__ void __launch_bounds__(kBlock) swiglu_fwd_kernel(const T* __restrict__ g, const T* __restrict__ u,
                                                            T* __restrict__ o, long long n) {
  const bool vec = aligned16(g) && aligned16(u) && aligned16(o);
  const long long nvec = vec ? n / kVec : 0;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  const long long tid = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x;
  for (long long i = tid; i < nvec; i += stride) {
    float gv[kVec], uv[kVec], ov[kVec];
    load8<T>(g + i * kVec, gv);
    load8<T>(u + i * kVec, uv);
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
      float y, dy;
      act_and_grad<ACT>(gv[k], y, dy);
      ov[k] = y * uv[k];
    }
    store8<T>(o + i * kVec, ov);
  }
  for (long long i = nvec * kVec + tid; i < n; i += stride) {
    float y, dy;
    act_and_grad<ACT>(Conv<T>::to(g[i]), y, dy);
    o[i] = Conv<T>::from(y * Conv<T>::to(u[i]));
  }
}

// dg / du may alias g / u: each thread reads its elements before writing them.
template <typename T, int ACT>
__global__ void __launch_bounds__(kBlock) swiglu_bwd_kernel(const T* g, const T* u, const T* __restrict__ d,
                                                            T* dg, T* du, long long n) {
  const bool vec = aligned16(g) && aligned16(u) && aligned16(d) && aligned16(dg) && aligned16(du);
  const long long nvec = vec ? n / kVec : 0;
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  const long long tid = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x;
  for (long long i = tid; i < nvec; i += stride) {
    float gv[kVec], uv[kVec], dv[kVec], a[kVec], b[kVec];
    load8<T>(g + i * kVec, gv);
    load8<T>(u + i * kVec, uv);
    load8<T>(d + i * kVec, dv);
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
      float y, dy;
      act_and_grad<ACT>(gv[k], y, dy);
      a[k] = dv[k] * uv[k] * dy;
      b[k] = dv[k] * y;
    }
    store8<T>(dg + i * kVec, a);
    store8<T>(du + i * kVec, b);
  }
  for (long long i = nvec * kVec + tid; i < n; i += stride) {
    const float uu = Conv<T>::to(u[i]), dd = Conv<T>::to(d[i]);
    float y, dy;
    act_and_grad<ACT>(Conv<T>::to(g[i]), y, dy);
    dg[i] = Conv<T>::from(dd * uu * dy);
    du[i] = Conv<T>::from(dd * y);
  }
}

// ---------------------------------------------------------------- rotary embedding
// One work item = 8 pairs (i, i + D/2) of one head of one row.
template <typename T>
__global__ void __launch_bounds__(kBlock) rope_kernel(T* q, T* k, const float* __restrict__ cos_t,
                                                      const float* __restrict__ sin_t, long long rows, int seq,
                                                      int q_heads, int k_heads, int head_dim, long long q_rs,
                                                      long long k_rs, float sign) {
  const int half = head_dim / 2;
  const int chunks = half / kVec;
  const long long q_items = rows * q_heads * chunks;
  const long long total = q_items + (k ? rows * k_heads * chunks : 0);
  const long long stride = static_cast<long long>(gridDim.x) * kBlock;
  for (long long it = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x; it < total; it += stride) {
    T* base;
    long long r;
    int c;
    if (it < q_items) {
      c = static_cast<int>(it % chunks);
      const long long rh = it / chunks;
      r = rh / q_heads;
      base = q + r * q_rs + (rh % q_heads) * head_dim;
    } else {
      const long long j = it - q_items;
      c = static_cast<int>(j % chunks);
      const long long rh = j / chunks;
      r = rh / k_heads;
      base = k + r * k_rs + (rh % k_heads) * head_dim;
    }
    const int pos = static_cast<int>(r % seq);
    float x1[kVec], x2[kVec], cs[kVec], sn[kVec], o1[kVec], o2[kVec];
    load8<T>(base + c * kVec, x1);
    load8<T>(base + half + c * kVec, x2);
    load8<float>(cos_t + static_cast<long long>(pos) * half + c * kVec, cs);
    load8<float>(sin_t + static_cast<long long>(pos) * half + c * kVec, sn);
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      const float s = sn[e] * sign;
      o1[e] = x1[e] * cs[e] - x2[e] * s;
      o2[e] = x2[e] * cs[e] + x1[e] * s;
    }
    store8<T>(base + c * kVec, o1);
    store8<T>(base + half + c * kVec, o2);
  }
}

// ---------------------------------------------------------------- softmax cross-entropy
constexpr int kXentBlock = 1024;

struct MaxSum {
  float m, s;
};

__device__ __forceinline__ MaxSum combine(MaxSum a, MaxSum b) {
  const float m = fmaxf(a.m, b.m);
  if (m == -CUDART_INF_F) return {m, 0.f};
  return {m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}

__device__ __forceinline__ MaxSum block_combine(MaxSum v) {
  __shared__ float sm[kXentBlock / 32], ss[kXentBlock / 32];
  __shared__ float out_m, out_s;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = combine(v, other);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sm[w] = v.m; ss[w] = v.s; }
  __syncthreads();
  if (w == 0) {
    MaxSum t{sm[l], ss[l]};   // kXentBlock / 32 == 32 warps
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxSum other{__shfl_xor_sync(0xffffffffu, t.m, o), __shfl_xor_sync(0xffffffffu, t.s, o)};
      t = combine(t, other);
    }
    if (l == 0) { out_m = t.m; out_s = t.s; }
  }
  __syncthreads();
  return {out_m, out_s};
}

template <typename T>
__global__ void __launch_bounds__(kXentBlock) softmax_xent_kernel(T* logits, const long long* __restrict__ labels,
                                                                  float* __restrict__ row_loss, int vocab, long long ld,
                                                                  float grad_scale) {
  const long long r = blockIdx.x;
  T* x = logits + r * ld;
  const long long label = labels[r];
  const bool vec = aligned16(x);
  const int nvec = vec ? vocab / kVec : 0;
  if (label < 0 || label >= vocab) {            // ignored position: no loss, zero gradient
    float z[kVec] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = threadIdx.x; i < nvec; i += kXentBlock) store8<T>(x + static_cast<long long>(i) * kVec, z);
    for (int i = nvec * kVec + threadIdx.x; i < vocab; i += kXentBlock) x[i] = Conv<T>::from(0.f);
    if (threadIdx.x == 0) row_loss[r] = 0.f;
    return;
  }
  MaxSum acc{-CUDART_INF_F, 0.f};
  for (int i = threadIdx.x; i < nvec; i += kXentBlock) {
    float v[kVec];
    load8<T>(x + static_cast<long long>(i) * kVec, v);
    float m = v[0];
#pragma unroll
    for (int e = 1; e < kVec; ++e) m = fmaxf(m, v[e]);
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < kVec; ++e) s += __expf(v[e] - m);
    acc = combine(acc, MaxSum{m, s});
  }
  for (int i = nvec * kVec + threadIdx.x; i < vocab; i += kXentBlock)
    acc = combine(acc, MaxSum{Conv<T>::to(x[i]), 1.f});
  const float x_label = Conv<T>::to(x[label]);   // read before the barriers below, i.e. before any write
  const MaxSum tot = block_combine(acc);
  if (threadIdx.x == 0) row_loss[r] = __logf(tot.s) + tot.m - x_label;
  const float inv = grad_scale / tot.s;
  for (int i = threadIdx.x; i < nvec; i += kXentBlock) {
    float v[kVec];
    load8<T>(x + static_cast<long long>(i) * kVec, v);
    const long long first = static_cast<long long>(i) * kVec;
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      v[e] = __expf(v[e] - tot.m) * inv;
      if (first + e == label) v[e] -= grad_scale;
    }
    store8<T>(x + first, v);
  }
  for (int i = nvec * kVec + threadIdx.x; i < vocab; i += kXentBlock) {
    float g = __expf(Conv<T>::to(x[i]) - tot.m) * inv;
    if (i == label) g -= grad_scale;
    x[i] = Conv<T>::from(g);
  }
}

}  // namespace
}  // namespace dmuon

using namespace dmuon;

extern "C" int dmuon_swiglu_fwd(const void* gate, const void* up, void* out, long long n, int act, int dtype,
                                void* stream_v) {
  if (n <= 0) return 0;
  if (act != 0 && act != 1) return -22;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  const int grid = grid_for((n + kVec - 1) / kVec);
  DMUON_MODEL_DISPATCH(dtype, T,
    if (act == 0)
      swiglu_fwd_kernel<T, 0><<<grid, kBlock, 0, st>>>(static_cast<const T*>(gate), static_cast<const T*>(up),
                                                       static_cast<T*>(out), n);
    else
      swiglu_fwd_kernel<T, 1><<<grid, kBlock, 0, st>>>(static_cast<const T*>(gate), static_cast<const T*>(up),
                                                       static_cast<T*>(out), n));
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_swiglu_bwd(const void* gate, const void* up, const void* d_out, void* d_gate, void* d_up,
                                long long n, int act, int dtype, void* stream_v) {
  if (n <= 0) return 0;
  if (act != 0 && act != 1) return -22;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  const int grid = grid_for((n + kVec - 1) / kVec);
  DMUON_MODEL_DISPATCH(dtype, T,
    if (act == 0)
      swiglu_bwd_kernel<T, 0><<<grid, kBlock, 0, st>>>(static_cast<const T*>(gate), static_cast<const T*>(up),
                                                       static_cast<const T*>(d_out), static_cast<T*>(d_gate),
                                                       static_cast<T*>(d_up), n);
    else
      swiglu_bwd_kernel<T, 1><<<grid, kBlock, 0, st>>>(static_cast<const T*>(gate), static_cast<const T*>(up),
                                                       static_cast<const T*>(d_out), static_cast<T*>(d_gate),
                                                       static_cast<T*>(d_up), n));
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_rope_inplace(void* q, void* k, const float* cos_t, const float* sin_t, long long rows, int seq,
                                  int q_heads, int k_heads, int head_dim, long long q_row_stride,
                                  long long k_row_stride, int inverse, int dtype, void* stream_v) {
  if (rows <= 0) return 0;
  if (head_dim <= 0 || head_dim % (2 * kVec) != 0 || seq <= 0) return -22;
  // every vector access must stay 16-byte aligned
  const long long esz = dtype == DMUON_FP32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (k && (reinterpret_cast<uintptr_t>(k) & 15)) ||
      (q_row_stride * esz) % 16 || (k && (k_row_stride * esz) % 16) ||
      (reinterpret_cast<uintptr_t>(cos_t) & 15) || (reinterpret_cast<uintptr_t>(sin_t) & 15))
    return -22;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  const long long items = rows * (q_heads + (k ? k_heads : 0)) * (head_dim / 2 / kVec);
  const int grid = grid_for(items);
  const float sign = inverse ? -1.f : 1.f;
  DMUON_MODEL_DISPATCH(dtype, T,
    rope_kernel<T><<<grid, kBlock, 0, st>>>(static_cast<T*>(q), static_cast<T*>(k), cos_t, sin_t, rows, seq, q_heads,
                                            k_heads, head_dim, q_row_stride, k_row_stride, sign));
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmuon_softmax_xent_inplace(void* logits, const long long* labels, float* row_loss, long long rows,
                                          int vocab, long long ld, float grad_scale, int dtype, void* stream_v) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || ld < vocab || rows > 2147483647LL) return -22;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  DMUON_MODEL_DISPATCH(dtype, T,
    softmax_xent_kernel<T><<<static_cast<unsigned>(rows), kXentBlock, 0, st>>>(static_cast<T*>(logits), labels,
                                                                              row_loss, vocab, ld, grad_scale));
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
