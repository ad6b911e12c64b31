// Self-attention forward/backward for short sequences (S <= 128, head dim 32 or 64): one CTA per
// (batch, head) keeps Q, K, V (and dO) of that head in shared memory, so each token's projections are
// read from HBM once per pass.  Fused in: the q/k/v bias add, the 1/sqrt(hd) scale, the key-padding
// mask, softmax, attention dropout (counter-based, recomputed in the backward) and the head
// split/merge addressing of the packed [T, 3H] projection buffer.
// Stands in for the attention inside the HF DistilBERT block that the reference trains through
// (dl_base.py:128; attention-dropout 0.1, 12 heads x 64).
#include "common.cuh"

namespace rb {

template <typename T, int HD>
__global__ void __launch_bounds__(128) attention_fwd_kernel(
    const T* __restrict__ qkv, const T* __restrict__ bqkv, const int* __restrict__ mask, T* __restrict__ ctx,
    T* __restrict__ probs, int S, int H, int nh, float p, const int* __restrict__ seed_ptr, uint32_t stream) {
  extern __shared__ float smf[];
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int KP = HD + 1;
  float* sQ = smf;                 // [S][HD]
  float* sK = sQ + S * HD;         // [S][HD+1]
  float* sV = sK + S * KP;         // [S][HD]
  float* sW = sV + S * HD;         // [4][S]
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const float scale = rsqrtf((float)HD);
  for (int i = tid; i < S * HD; i += blockDim.x) {
    const int s = i / HD, d = i % HD;
    const size_t base = (size_t)(b * S + s) * 3 * H + h * HD + d;
    sQ[s * HD + d] = (to_f(qkv[base]) + to_f(bqkv[h * HD + d])) * scale;
    sK[s * KP + d] = to_f(qkv[base + H]) + to_f(bqkv[H + h * HD + d]);
    sV[s * HD + d] = to_f(qkv[base + 2 * H]) + to_f(bqkv[2 * H + h * HD + d]);
  }
  __syncthreads();
  float* w = sW + warp * S;
  for (int i = warp; i < S; i += 4) {
    float sc[4];
    float mx = -1e30f;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      sc[jj] = -1e30f;
      if (j < S && mask[b * S + j] != 0) {
        float a = 0.f;
#pragma unroll 16
        for (int d = 0; d < HD; ++d) a += sQ[i * HD + d] * sK[j * KP + d];
        sc[jj] = a;
      }
      mx = fmaxf(mx, sc[jj]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      // a fully masked row (no valid key) degenerates to uniform weights, like softmax over equal scores
      sc[jj] = (j < S) ? __expf(sc[jj] - mx) : 0.f;
      sum += sc[jj];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    const size_t prow = ((size_t)(b * nh + h) * S + i) * S;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      if (j < S) {
        float pr = round_through<T>(sc[jj] * inv);
        probs[prow + j] = from_f<T>(pr);
        if (p > 0.f) pr = keep(seed, stream, (uint32_t)(prow + j), p) ? pr * inv_keep : 0.f;
        w[j] = pr;
      }
    }
    __syncwarp();
#pragma unroll
    for (int dd = 0; dd < HD / 32; ++dd) {
      const int d = lane + 32 * dd;
      float a = 0.f;
      for (int j = 0; j < S; ++j) a += w[j] * sV[j * HD + d];
      ctx[(size_t)(b * S + i) * H + h * HD + d] = from_f<T>(a);
    }
    __syncwarp();
  }
}

template <typename T, int HD>
__global__ void __launch_bounds__(128) attention_bwd_kernel(
    const T* __restrict__ dctx, const T* __restrict__ qkv, const T* __restrict__ bqkv, const T* __restrict__ probs,
    T* __restrict__ dqkv, int S, int H, int nh, float p, const int* __restrict__ seed_ptr, uint32_t stream) {
  extern __shared__ float smf[];
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int RP = HD + 2;       // padded row of the 16-bit operand tiles (odd number of 32-bit words)
  const int SP = S + 1;
  float* sDS = smf;                // [S][S+1]
  float* sWt = sDS + S * SP;       // [S][S+1]  dropped-out weights
  T* sQ = reinterpret_cast<T*>(sWt + S * SP);   // [S][RP] each
  T* sK = sQ + S * RP;
  T* sV = sK + S * RP;
  T* sDO = sV + S * RP;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const float scale = rsqrtf((float)HD);
  for (int i = tid; i < S * HD; i += blockDim.x) {
    const int s = i / HD, d = i % HD;
    const size_t base = (size_t)(b * S + s) * 3 * H + h * HD + d;
    sQ[s * RP + d] = from_f<T>(to_f(qkv[base]) + to_f(bqkv[h * HD + d]));
    sK[s * RP + d] = from_f<T>(to_f(qkv[base + H]) + to_f(bqkv[H + h * HD + d]));
    sV[s * RP + d] = from_f<T>(to_f(qkv[base + 2 * H]) + to_f(bqkv[2 * H + h * HD + d]));
    sDO[s * RP + d] = dctx[(size_t)(b * S + s) * H + h * HD + d];
  }
  __syncthreads();
  // phase 1: rows of dS and of the dropped-out weights
  for (int i = warp; i < S; i += 4) {
    const size_t prow = ((size_t)(b * nh + h) * S + i) * S;
    float pr[4], dp[4];
    float dot = 0.f;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      pr[jj] = 0.f; dp[jj] = 0.f;
      if (j < S) {
        pr[jj] = to_f(probs[prow + j]);
        float a = 0.f;
#pragma unroll 16
        for (int d = 0; d < HD; ++d) a += to_f(sDO[i * RP + d]) * to_f(sV[j * RP + d]);
        float m = 1.f;
        if (p > 0.f) m = keep(seed, stream, (uint32_t)(prow + j), p) ? inv_keep : 0.f;
        dp[jj] = a * m;
        sWt[i * SP + j] = pr[jj] * m;
        dot += dp[jj] * pr[jj];
      }
    }
    dot = warp_sum(dot);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      if (j < S) sDS[i * SP + j] = pr[jj] * (dp[jj] - dot) * scale;
    }
  }
  __syncthreads();
  // phase 2: dQ (row i), dK and dV (row j)
  for (int r = warp; r < S; r += 4) {
    const size_t out = (size_t)(b * S + r) * 3 * H + h * HD;
#pragma unroll
    for (int dd = 0; dd < HD / 32; ++dd) {
      const int d = lane + 32 * dd;
      float dq = 0.f, dk = 0.f, dv = 0.f;
      for (int t = 0; t < S; ++t) {
        dq += sDS[r * SP + t] * to_f(sK[t * RP + d]);
        dk += sDS[t * SP + r] * to_f(sQ[t * RP + d]);
        dv += sWt[t * SP + r] * to_f(sDO[t * RP + d]);
      }
      dqkv[out + d] = from_f<T>(dq);
      dqkv[out + H + d] = from_f<T>(dk);
      dqkv[out + 2 * H + d] = from_f<T>(dv);
    }
  }
}

}  // namespace rb

using namespace rb;

template <typename T>
static int launch_fwd(const void* qkv, const void* bqkv, const int* mask, void* ctx, void* probs, int b, int S, int H,
                      int nh, float p, const int* seed, unsigned stream_id, cudaStream_t st) {
  const int hd = H / nh;
  const size_t smem = ((size_t)S * hd * 2 + (size_t)S * (hd + 1) + 4 * (size_t)S) * sizeof(float);
  dim3 grid(nh, b);
  if (hd == 64) {
    auto k = attention_fwd_kernel<T, 64>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
    k<<<grid, 128, smem, st>>>((const T*)qkv, (const T*)bqkv, mask, (T*)ctx, (T*)probs, S, H, nh, p, seed, stream_id);
  } else if (hd == 32) {
    auto k = attention_fwd_kernel<T, 32>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
    k<<<grid, 128, smem, st>>>((const T*)qkv, (const T*)bqkv, mask, (T*)ctx, (T*)probs, S, H, nh, p, seed, stream_id);
  } else {
    return -4;
  }
  return 0;
}

template <typename T>
static int launch_bwd(const void* dctx, const void* qkv, const void* bqkv, const void* probs, void* dqkv, int b, int S,
                      int H, int nh, float p, const int* seed, unsigned stream_id, cudaStream_t st) {
  const int hd = H / nh;
  const size_t smem = 2 * (size_t)S * (S + 1) * sizeof(float) + 4 * (size_t)S * (hd + 2) * sizeof(T);
  if (smem > 227 * 1024) return -6;
  dim3 grid(nh, b);
  if (hd == 64) {
    auto k = attention_bwd_kernel<T, 64>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
    k<<<grid, 128, smem, st>>>((const T*)dctx, (const T*)qkv, (const T*)bqkv, (const T*)probs, (T*)dqkv, S, H, nh, p,
                               seed, stream_id);
  } else if (hd == 32) {
    auto k = attention_bwd_kernel<T, 32>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
    k<<<grid, 128, smem, st>>>((const T*)dctx, (const T*)qkv, (const T*)bqkv, (const T*)probs, (T*)dqkv, S, H, nh, p,
                               seed, stream_id);
  } else {
    return -4;
  }
  return 0;
}

// Returns -6 when the tiles do not fit in shared memory (caller falls back to composing library ops).
RB_API int rb_attention_fwd(int dtype, const void* qkv, const void* bqkv, const int* mask, void* ctx, void* probs, int b,
                            int S, int H, int nh, float p, const int* seed, unsigned stream_id, cudaStream_t st) {
  if (S > 128 || S < 1 || H % nh) return -4;
  int rc;
  switch (dtype) {
    case RB_F32: rc = launch_fwd<float>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st); break;
    case RB_BF16: rc = launch_fwd<__nv_bfloat16>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st); break;
    case RB_F16: rc = launch_fwd<__half>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st); break;
    default: return -1;
  }
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_attention_bwd(int dtype, const void* dctx, const void* qkv, const void* bqkv, const void* probs,
                            void* dqkv, int b, int S, int H, int nh, float p, const int* seed, unsigned stream_id,
                            cudaStream_t st) {
  if (S > 128 || S < 1 || H % nh) return -4;
  int rc;
  switch (dtype) {
    case RB_F32: rc = launch_bwd<float>(dctx, qkv, bqkv, probs, dqkv, b, S, H, nh, p, seed, stream_id, st); break;
    case RB_BF16: rc = launch_bwd<__nv_bfloat16>(dctx, qkv, bqkv, probs, dqkv, b, S, H, nh, p, seed, stream_id, st); break;
    case RB_F16: rc = launch_bwd<__half>(dctx, qkv, bqkv, probs, dqkv, b, S, H, nh, p, seed, stream_id, st); break;
    default: return -1;
  }
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}
