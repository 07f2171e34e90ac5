// 128-bit vector access helpers shared by the elementwise kernels: every thread
// moves 8 elements per step (one 16-byte access for 16-bit types, two for fp32)
// and does its arithmetic in fp32.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace dmuon {

constexpr int kBlock = 256;
constexpr int kVec = 8;

template <typename T>
struct Conv;
template <>
struct Conv<__nv_bfloat16> {
  static __device__ __forceinline__ float to(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from(float x) { return __float2bfloat16_rn(x); }
};
template <>
struct Conv<__half> {
  static __device__ __forceinline__ float to(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from(float x) { return __float2half_rn(x); }
};
template <>
struct Conv<float> {
  static __device__ __forceinline__ float to(float x) { return x; }
  static __device__ __forceinline__ float from(float x) { return x; }
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[kVec]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < kVec; ++i) v[i] = Conv<T>::to(e[i]);
  } else {
    float4 a = reinterpret_cast<const float4*>(p)[0];
    float4 b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[kVec]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < kVec; ++i) e[i] = Conv<T>::from(v[i]);
    *reinterpret_cast<uint4*>(p) = raw;
  } else {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

__device__ __forceinline__ bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

}  // namespace dmuon
