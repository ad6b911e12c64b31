// Encoder optimizer kernels over flat buffers:
//   grad_check     raises the found-inf flag if any gradient element is non-finite
//   adamw          fused AdamW (decoupled decay) with gradient unscaling, bias correction, the skip on
//                  found-inf, and the write of the low-precision compute copy of the parameters
//   scaler_update  loss-scale state machine (growth / back-off), Adam step counter, flag reset
// They replace apex FusedAdam + torch GradScaler's foreach kernels as the reference uses them
// (main.py:180-181, dl_base.py:372-374).  All step-varying scalars are read from the device-resident
// hyper-parameter block, so the launches can be replayed from a CUDA graph with no host round trip.
#include "common.cuh"

namespace rb {

template <typename T>
__global__ void __launch_bounds__(256) grad_check_kernel(const T* __restrict__ g, size_t n_vec, float* __restrict__ hp) {
  bool bad = false;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
    float a[8];
    load8(g + i * 8, a);
#pragma unroll
    for (int j = 0; j < 8; ++j) bad |= !isfinite(a[j]);
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) hp[HP_FOUND_INF] = 1.0f;
}

template <typename TG, typename TP>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p32, float* __restrict__ m, float* __restrict__ v,
                                                    const TG* __restrict__ g, TP* __restrict__ p16, size_t n_vec,
                                                    size_t n_decay, const float* __restrict__ hp, float beta1, float beta2,
                                                    float eps, float wd, float grad_mult) {
  if (hp[HP_FOUND_INF] != 0.f) return;
  const float lr = hp[HP_LR_ENC];
  const float step = hp[HP_ADAM_STEP] + 1.0f;
  const float inv_scale = hp[HP_INV_SCALE] * grad_mult;
  const float bc1 = 1.f - powf(beta1, step);
  const float bc2 = 1.f - powf(beta2, step);
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
    const size_t e = i * 8;
    float gg[8], pp[8], mm[8], vv[8];
    load8(g + e, gg);
    load8(p32 + e, pp);
    load8(m + e, mm);
    load8(v + e, vv);
    const float decay = (e < n_decay) ? 1.f - lr * wd : 1.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gr = gg[j] * inv_scale;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gr;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gr * gr;
      const float denom = sqrtf(vv[j] * inv_bc2) + eps;
      pp[j] = pp[j] * decay - lr * (mm[j] * inv_bc1) / denom;
    }
    store8(p32 + e, pp);
    store8(m + e, mm);
    store8(v + e, vv);
    if (p16 != nullptr) store8(p16 + e, pp);
  }
}

__global__ void scaler_update_kernel(float* hp, int enabled, float growth, float backoff, float interval) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (hp[HP_FOUND_INF] != 0.f) {
    if (enabled) hp[HP_SCALE] *= backoff;
    hp[HP_TRACKER] = 0.f;
  } else {
    hp[HP_ADAM_STEP] += 1.f;
    hp[HP_TRACKER] += 1.f;
    if (enabled && hp[HP_TRACKER] >= interval) {
      hp[HP_SCALE] *= growth;
      hp[HP_TRACKER] = 0.f;
    }
  }
  hp[HP_INV_SCALE] = 1.f / hp[HP_SCALE];
  hp[HP_FOUND_INF] = 0.f;
}

}  // namespace rb

using namespace rb;

static int flat_blocks(size_t n_vec) {
  size_t b = (n_vec + 255) / 256;
  return (int)(b > rb::sm_count() * 8 ? rb::sm_count() * 8 : (b == 0 ? 1 : b));
}

RB_API int rb_grad_check(int dtype, const void* g, long long n, float* hp, cudaStream_t st) {
  if (n % 8) return -3;
  const size_t n_vec = (size_t)n / 8;
  switch (dtype) {
    case RB_F32: grad_check_kernel<float><<<flat_blocks(n_vec), 256, 0, st>>>((const float*)g, n_vec, hp); break;
    case RB_BF16: grad_check_kernel<__nv_bfloat16><<<flat_blocks(n_vec), 256, 0, st>>>((const __nv_bfloat16*)g, n_vec, hp); break;
    case RB_F16: grad_check_kernel<__half><<<flat_blocks(n_vec), 256, 0, st>>>((const __half*)g, n_vec, hp); break;
    default: return -1;
  }
  RB_LAUNCH_CHECK();
  return 0;
}

// p16 may be null (fp32 encoder: the master buffer is the compute copy)
RB_API int rb_adamw(int dtype, float* p32, float* m, float* v, const void* g, void* p16, long long n, long long n_decay,
                    const float* hp, float beta1, float beta2, float eps, float wd, float grad_mult, cudaStream_t st) {
  if (n % 8 || n_decay % 8) return -3;
  const size_t n_vec = (size_t)n / 8;
  const int blocks = flat_blocks(n_vec);
  switch (dtype) {
    case RB_F32:
      adamw_kernel<float, float><<<blocks, 256, 0, st>>>(p32, m, v, (const float*)g, (float*)p16, n_vec, (size_t)n_decay,
                                                           hp, beta1, beta2, eps, wd, grad_mult);
      break;
    case RB_BF16:
      adamw_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, st>>>(p32, m, v, (const __nv_bfloat16*)g,
                                                                         (__nv_bfloat16*)p16, n_vec, (size_t)n_decay, hp,
                                                                         beta1, beta2, eps, wd, grad_mult);
      break;
    case RB_F16:
      adamw_kernel<__half, __half><<<blocks, 256, 0, st>>>(p32, m, v, (const __half*)g, (__half*)p16, n_vec,
                                                           (size_t)n_decay, hp, beta1, beta2, eps, wd, grad_mult);
      break;
    default: return -1;
  }
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_scaler_update(float* hp, int enabled, float growth, float backoff, int interval, cudaStream_t st) {
  scaler_update_kernel<<<1, 32, 0, st>>>(hp, enabled, growth, backoff, (float)interval);
  RB_LAUNCH_CHECK();
  return 0;
}
