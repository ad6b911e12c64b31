// Shared device helpers for the sm_100a kernels of renee_b200.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define RB_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side (renee_b200/ops/cuda.py)
enum RbDtype : int { RB_F32 = 0, RB_BF16 = 1, RB_F16 = 2 };

// Slots of the device-resident hyper-parameter block (renee_b200/optim/hparams.py)
enum RbHp : int {
  HP_LR_XFC = 0, HP_LR_ENC = 1, HP_SEED = 2,
  HP_SCALE = 8, HP_INV_SCALE = 9, HP_FOUND_INF = 10, HP_TRACKER = 11, HP_ADAM_STEP = 12
};

#define RB_LAUNCH_CHECK() do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return (int)e_; } while (0)

namespace rb {

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// 8 consecutive elements of T, moved with the widest aligned access available
template <typename T> struct Vec8 {
  T v[8];
};

template <typename T>
__device__ __forceinline__ void load8(const T* __restrict__ p, float (&out)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = to_f(e[i]);
  } else {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  }
}

template <typename T>
__device__ __forceinline__ void store8(T* __restrict__ p, const float (&in)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = from_f<T>(in[i]);
    *reinterpret_cast<uint4*>(p) = raw;
  } else {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(in[4], in[5], in[6], in[7]);
  }
}

// Rounds through T (what a store followed by a load would give)
template <typename T> __device__ __forceinline__ float round_through(float x) { return to_f(from_f<T>(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Counter-based dropout RNG; must stay bit-identical to renee_b200/ops/rng.py::mix32
__device__ __forceinline__ uint32_t mix32(uint32_t seed, uint32_t stream, uint32_t idx) {
  uint32_t x = idx * 0x9E3779B1u + seed;
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  x += stream * 0x27D4EB2Fu;
  x ^= x >> 15; x *= 0x2C1B3C6Du; x ^= x >> 12; x *= 0x297A2D39u; x ^= x >> 15;
  return x;
}
__device__ __forceinline__ bool keep(uint32_t seed, uint32_t stream, uint32_t idx, float p) {
  return (float)(mix32(seed, stream, idx) >> 8) * (1.0f / 16777216.0f) >= p;
}

}  // namespace rb
