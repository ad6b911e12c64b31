// Shared device helpers for the sm_100a kernels of renee_b200.
#pragma once
#include <type_traits>
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

// 8 elements kept in their storage format (4 registers for 16-bit types) and expanded on demand:
// lets a kernel hold several vectors across a reduction without paying 8 registers per vector.
template <typename T> struct Raw8 { uint4 v; };
template <> struct Raw8<float> { float4 a, b; };

template <typename T> __device__ __forceinline__ Raw8<T> load_raw8(const T* __restrict__ p) {
  Raw8<T> r;
  r.v = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <> __device__ __forceinline__ Raw8<float> load_raw8<float>(const float* __restrict__ p) {
  Raw8<float> r;
  r.a = *reinterpret_cast<const float4*>(p);
  r.b = *reinterpret_cast<const float4*>(p + 4);
  return r;
}
template <typename T> __device__ __forceinline__ void unpack8(const Raw8<T>& r, float (&out)[8]) {
  const T* e = reinterpret_cast<const T*>(&r.v);
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = to_f(e[i]);
}
template <> __device__ __forceinline__ void unpack8<float>(const Raw8<float>& r, float (&out)[8]) {
  out[0] = r.a.x; out[1] = r.a.y; out[2] = r.a.z; out[3] = r.a.w;
  out[4] = r.b.x; out[5] = r.b.y; out[6] = r.b.z; out[7] = r.b.w;
}

// Rounds through T (what a store followed by a load would give)
template <typename T> __device__ __forceinline__ float round_through(float x) { return to_f(from_f<T>(x)); }

// fp32 -> fp16 with stochastic rounding: add uniform noise below the 13 mantissa bits fp16 drops, then
// truncate.  Unbiased for values in fp16's normal range, which keeps updates smaller than half an ulp
// of W from being lost systematically late in the learning-rate schedule.
__device__ __forceinline__ __half sr_half(float x, uint32_t rnd) {
  uint32_t b = __float_as_uint(x);
  b = (b + (rnd & 0x1FFFu)) & ~0x1FFFu;
  return __float2half_rz(__uint_as_float(b));
}
// The same for either 16-bit type, returned as the fp32 value of the rounded number (bf16 drops 16 bits).
template <typename T> __device__ __forceinline__ float sr_round(float x, uint32_t rnd) {
  if (std::is_same<T, __half>::value) return __half2float(sr_half(x, rnd));
  const uint32_t b = (__float_as_uint(x) + (rnd & 0xFFFFu)) & ~0xFFFFu;
  return __uint_as_float(b);
}

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

// One 16-byte reduction instead of four 4-byte ones (p must be 16-byte aligned)
__device__ __forceinline__ void red_add_f32x4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Standard normal CDF Phi(z) = 0.5 erfc(-z / sqrt 2), and e = exp(-z^2 / 2) as a by-product (the GELU
// gradient needs it for the density).  erfc(|x|) = t (a1 + t (a2 + t (a3 + t (a4 + t a5)))) exp(-x^2) with
// t = 1 / (1 + p |x|) (Abramowitz & Stegun 7.1.26, |error| <= 1.5e-7): the negative tail comes out of the
// product directly, without the cancellation of 1 + erf, and the whole thing is 2 special-function
// instructions and about 12 FMA-pipe ones -- which matters because the GELU kernels are bound by
// instruction issue rather than by HBM.
__device__ __forceinline__ float normal_cdf(float z, float& e) {
  const float ax = fabsf(z) * 0.70710678118654752f;
  float t;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, ax, 1.f)));
  float p = 1.061405429f;
  p = fmaf(p, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  e = __expf(-ax * ax);
  const float half = 0.5f * p * t * e;
  return z < 0.f ? half : 1.f - half;
}

// Exact (erf) GELU and its derivative: gelu(z) = z Phi(z), gelu'(z) = Phi(z) + z phi(z)
__device__ __forceinline__ float gelu_f(float z) {
  float e;
  return z * normal_cdf(z, e);
}
__device__ __forceinline__ float gelu_grad_f(float z) {
  float e;
  const float cdf = normal_cdf(z, e);
  return fmaf(z * 0.39894228040143268f, e, cdf);
}

// Number of SMs of the current device (queried once per process; all GPUs of a job are alike)
inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1)
      n = 1;
  }
  return n;
}

// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization attribute may
// start (set up barriers, allocate TMEM, fetch descriptors) while its predecessor in the stream is still running,
// once every CTA of the predecessor has executed launch_dependents (or exited); it must execute grid_dep_wait
// before its first access to global memory, which blocks until the predecessor has completed and its writes are
// visible.  Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Host side: one switch for the whole library and a launch helper that sets the attribute.  A kernel launched
// through launch_pdl MUST execute grid_dep_wait() before its first access to global memory.
inline int& pdl_flag() {
  static int on = 1;
  return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_flag() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
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
