// Tensor-core self-attention forward/backward for 16-bit activations, S <= 128, head dim 32 or 64.
// Same fusion and interface as attention.cu (bias add, scale, key-padding mask, softmax, counter-based
// attention dropout, head split/merge addressing); the five small matrix products per (batch, head)
//   S = Q K^T,  O = P V,  dP = dO V^T,  dQ = dS K,  dK = dS^T Q,  dV = P~^T dO
// run on the tensor cores through warp-level 16x16x16 MMA fragments over shared-memory tiles.  One CTA
// of 4 warps owns one (batch, head); the sequence is padded to a multiple of 16 inside shared memory.
// (tcgen05 needs M >= 64 per instruction; at S = 32 a head is a quarter of that, so the warp-level
// MMA is the shape that fits this op.  The classifier GEMMs, where the FLOPs are, use tcgen05.)
#include <mma.h>
#include "common.cuh"

namespace rb {
using namespace nvcuda;

template <typename T> struct WT;
template <> struct WT<__nv_bfloat16> { using type = __nv_bfloat16; };
template <> struct WT<__half> { using type = __half; };

// One warp converts its 16x16 fp32 staging tile to T and writes it to global rows (row stride ld).
template <typename T>
__device__ __forceinline__ void flush_tile(const float* stage, T* dst, int ld, int rows_valid, int lane) {
  // lane handles row (lane / 2), 8 consecutive columns
  const int r = lane >> 1, c = (lane & 1) * 8;
  if (r < rows_valid) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = stage[r * 20 + c + j];
    store8(dst + (size_t)r * ld + c, v);
  }
}

template <typename T, int HD>
__global__ void __launch_bounds__(256) attention_fwd_tc_kernel(
    const T* __restrict__ qkv, const T* __restrict__ bqkv, const int* __restrict__ mask, T* __restrict__ ctx,
    T* __restrict__ probs, int S, int Sp, int H, int nh, float p, const int* __restrict__ seed_ptr, uint32_t stream) {
  using W = typename WT<T>::type;
  extern __shared__ __align__(128) uint8_t sm_raw[];
  constexpr int RP = HD + 8;
  const int PP = Sp + 8, FP = Sp + 4;
  T* sQ = reinterpret_cast<T*>(sm_raw);
  T* sK = sQ + Sp * RP;
  T* sV = sK + Sp * RP;
  T* sP = sV + Sp * RP;
  float* sS = reinterpret_cast<float*>(sP + Sp * PP);
  float* sStage = sS + Sp * FP;        // [warps][16][20]
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const float scale = rsqrtf((float)HD);
  for (int i = tid; i < Sp * (HD / 8); i += blockDim.x) {
    const int s = i / (HD / 8), d = (i % (HD / 8)) * 8;
    float q[8], k[8], v[8];
    if (s < S) {
      const size_t base = (size_t)(b * S + s) * 3 * H + h * HD + d;
      float bq[8], bk[8], bv[8];
      load8(qkv + base, q); load8(qkv + base + H, k); load8(qkv + base + 2 * H, v);
      load8(bqkv + h * HD + d, bq); load8(bqkv + H + h * HD + d, bk); load8(bqkv + 2 * H + h * HD + d, bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) { q[j] += bq[j]; k[j] += bk[j]; v[j] += bv[j]; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { q[j] = 0.f; k[j] = 0.f; v[j] = 0.f; }
    }
    store8(sQ + s * RP + d, q); store8(sK + s * RP + d, k); store8(sV + s * RP + d, v);
  }
  __syncthreads();
  const int nt = Sp / 16;
  for (int t = warp; t < nt * nt; t += nw) {
    const int ti = t / nt, tj = t % nt;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
    wmma::fill_fragment(acc, 0.f);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, W, wmma::row_major> a;
      wmma::fragment<wmma::matrix_b, 16, 16, 16, W, wmma::col_major> bm;
      wmma::load_matrix_sync(a, reinterpret_cast<const W*>(sQ + ti * 16 * RP + k * 16), RP);
      wmma::load_matrix_sync(bm, reinterpret_cast<const W*>(sK + tj * 16 * RP + k * 16), RP);
      wmma::mma_sync(acc, a, bm, acc);
    }
    wmma::store_matrix_sync(sS + ti * 16 * FP + tj * 16, acc, FP, wmma::mem_row_major);
  }
  __syncthreads();
  for (int i = warp; i < Sp; i += nw) {
    float sc[4];
    float mx = -1e30f;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      sc[jj] = -1e30f;
      if (i < S && j < S && mask[b * S + j] != 0) sc[jj] = sS[i * FP + j] * scale;
      mx = fmaxf(mx, sc[jj]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      sc[jj] = (j < S) ? __expf(sc[jj] - mx) : 0.f;
      sum += sc[jj];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    const size_t prow = ((size_t)(b * nh + h) * S + i) * S;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      if (j < Sp) {
        float pr = 0.f;
        if (i < S && j < S) {
          pr = round_through<T>(sc[jj] * inv);
          probs[prow + j] = from_f<T>(pr);
          if (p > 0.f) pr = keep(seed, stream, (uint32_t)(prow + j), p) ? pr * inv_keep : 0.f;
        }
        sP[i * PP + j] = from_f<T>(pr);
      }
    }
  }
  __syncthreads();
  float* stage = sStage + warp * 16 * 20;
  for (int t = warp; t < nt * (HD / 16); t += nw) {
    const int ti = t / (HD / 16), td = t % (HD / 16);
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
    wmma::fill_fragment(acc, 0.f);
    for (int k = 0; k < nt; ++k) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, W, wmma::row_major> a;
      wmma::fragment<wmma::matrix_b, 16, 16, 16, W, wmma::row_major> bm;
      wmma::load_matrix_sync(a, reinterpret_cast<const W*>(sP + ti * 16 * PP + k * 16), PP);
      wmma::load_matrix_sync(bm, reinterpret_cast<const W*>(sV + k * 16 * RP + td * 16), RP);
      wmma::mma_sync(acc, a, bm, acc);
    }
    wmma::store_matrix_sync(stage, acc, 20, wmma::mem_row_major);
    __syncwarp();
    flush_tile<T>(stage, ctx + (size_t)(b * S + ti * 16) * H + h * HD + td * 16, H, min(16, S - ti * 16), lane);
    __syncwarp();
  }
}

template <typename T, int HD>
__global__ void __launch_bounds__(256) attention_bwd_tc_kernel(
    const T* __restrict__ dctx, const T* __restrict__ qkv, const T* __restrict__ bqkv, const T* __restrict__ probs,
    T* __restrict__ dqkv, int S, int Sp, int H, int nh, float p, const int* __restrict__ seed_ptr, uint32_t stream,
    float* __restrict__ bias_acc) {
  using W = typename WT<T>::type;
  extern __shared__ __align__(128) uint8_t sm_raw[];
  constexpr int RP = HD + 8;
  const int PP = Sp + 8, FP = Sp + 4;
  T* sQ = reinterpret_cast<T*>(sm_raw);
  T* sK = sQ + Sp * RP;
  T* sV = sK + Sp * RP;
  T* sDO = sV + Sp * RP;
  T* sDS = sDO + Sp * RP;
  T* sW = sDS + Sp * PP;
  float* sF = reinterpret_cast<float*>(sW + Sp * PP);
  float* sStage = sF + Sp * FP;
  float* sBias = sStage + 8 * 16 * 20;   // [3][HD] column sums of dQ, dK, dV = this head's q/k/v bias gradients
  if (bias_acc != nullptr)
    for (int i = threadIdx.x; i < 3 * HD; i += blockDim.x) sBias[i] = 0.f;
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const float scale = rsqrtf((float)HD);
  for (int i = tid; i < Sp * (HD / 8); i += blockDim.x) {
    const int s = i / (HD / 8), d = (i % (HD / 8)) * 8;
    float q[8], k[8], v[8], g[8];
    if (s < S) {
      const size_t base = (size_t)(b * S + s) * 3 * H + h * HD + d;
      float bq[8], bk[8], bv[8];
      load8(qkv + base, q); load8(qkv + base + H, k); load8(qkv + base + 2 * H, v);
      load8(bqkv + h * HD + d, bq); load8(bqkv + H + h * HD + d, bk); load8(bqkv + 2 * H + h * HD + d, bv);
      load8(dctx + (size_t)(b * S + s) * H + h * HD + d, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) { q[j] += bq[j]; k[j] += bk[j]; v[j] += bv[j]; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { q[j] = 0.f; k[j] = 0.f; v[j] = 0.f; g[j] = 0.f; }
    }
    store8(sQ + s * RP + d, q); store8(sK + s * RP + d, k); store8(sV + s * RP + d, v); store8(sDO + s * RP + d, g);
  }
  __syncthreads();
  const int nt = Sp / 16;
  // dP = dO V^T
  for (int t = warp; t < nt * nt; t += nw) {
    const int ti = t / nt, tj = t % nt;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
    wmma::fill_fragment(acc, 0.f);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, W, wmma::row_major> a;
      wmma::fragment<wmma::matrix_b, 16, 16, 16, W, wmma::col_major> bm;
      wmma::load_matrix_sync(a, reinterpret_cast<const W*>(sDO + ti * 16 * RP + k * 16), RP);
      wmma::load_matrix_sync(bm, reinterpret_cast<const W*>(sV + tj * 16 * RP + k * 16), RP);
      wmma::mma_sync(acc, a, bm, acc);
    }
    wmma::store_matrix_sync(sF + ti * 16 * FP + tj * 16, acc, FP, wmma::mem_row_major);
  }
  __syncthreads();
  // rows of dS and of the dropped-out weights
  for (int i = warp; i < Sp; i += nw) {
    const size_t prow = ((size_t)(b * nh + h) * S + i) * S;
    float pr[4], dp[4], m[4];
    float dot = 0.f;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      pr[jj] = 0.f; dp[jj] = 0.f; m[jj] = 0.f;
      if (i < S && j < S) {
        pr[jj] = to_f(probs[prow + j]);
        m[jj] = 1.f;
        if (p > 0.f) m[jj] = keep(seed, stream, (uint32_t)(prow + j), p) ? inv_keep : 0.f;
        dp[jj] = sF[i * FP + j] * m[jj];
        dot += dp[jj] * pr[jj];
      }
    }
    dot = warp_sum(dot);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = lane + 32 * jj;
      if (j < Sp) {
        sDS[i * PP + j] = from_f<T>(pr[jj] * (dp[jj] - dot) * scale);
        sW[i * PP + j] = from_f<T>(pr[jj] * m[jj]);
      }
    }
  }
  __syncthreads();
  float* stage = sStage + warp * 16 * 20;
  const int ntd = HD / 16;
  // 3 * nt * ntd output tiles: which = 0 dQ = dS K, 1 dK = dS^T Q, 2 dV = P~^T dO
  for (int t = warp; t < 3 * nt * ntd; t += nw) {
    const int which = t / (nt * ntd);
    const int tr = (t % (nt * ntd)) / ntd, td = t % ntd;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
    wmma::fill_fragment(acc, 0.f);
    for (int k = 0; k < nt; ++k) {
      wmma::fragment<wmma::matrix_b, 16, 16, 16, W, wmma::row_major> bm;
      if (which == 0) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, W, wmma::row_major> a;
        wmma::load_matrix_sync(a, reinterpret_cast<const W*>(sDS + tr * 16 * PP + k * 16), PP);
        wmma::load_matrix_sync(bm, reinterpret_cast<const W*>(sK + k * 16 * RP + td * 16), RP);
        wmma::mma_sync(acc, a, bm, acc);
      } else {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, W, wmma::col_major> a;   // transposed view: (m, k) = src[k][m]
        const T* src = (which == 1) ? sDS : sW;
        const T* rhs = (which == 1) ? sQ : sDO;
        wmma::load_matrix_sync(a, reinterpret_cast<const W*>(src + k * 16 * PP + tr * 16), PP);
        wmma::load_matrix_sync(bm, reinterpret_cast<const W*>(rhs + k * 16 * RP + td * 16), RP);
        wmma::mma_sync(acc, a, bm, acc);
      }
    }
    wmma::store_matrix_sync(stage, acc, 20, wmma::mem_row_major);
    __syncwarp();
    const int rows_valid = min(16, S - tr * 16);
    flush_tile<T>(stage, dqkv + (size_t)(b * S + tr * 16) * 3 * H + which * H + h * HD + td * 16, 3 * H, rows_valid, lane);
    if (bias_acc != nullptr && lane < 16) {
      float cs = 0.f;
      for (int r = 0; r < rows_valid; ++r) cs += round_through<T>(stage[r * 20 + lane]);
      atomicAdd(&sBias[which * HD + td * 16 + lane], cs);
    }
    __syncwarp();
  }
  if (bias_acc != nullptr) {
    // the bias gradient of the packed projection is the column sum of dqkv: add this (batch, head)'s part to
    // one of the replicas of the step-wide accumulator (converted later by the deferred finalize kernel)
    __syncthreads();
    float* my_acc = bias_acc + (size_t)((blockIdx.y * gridDim.x + blockIdx.x) % 8) * 3 * H;
    for (int i = threadIdx.x; i < 3 * HD; i += blockDim.x)
      atomicAdd(my_acc + (i / HD) * H + h * HD + (i % HD), sBias[i]);
  }
}

}  // namespace rb

using namespace rb;

static size_t fwd_smem(int Sp, int hd, size_t esz) {
  return (size_t)3 * Sp * (hd + 8) * esz + (size_t)Sp * (Sp + 8) * esz + (size_t)Sp * (Sp + 4) * 4 + 8 * 16 * 20 * 4;
}
static size_t bwd_smem(int Sp, int hd, size_t esz) {
  return (size_t)4 * Sp * (hd + 8) * esz + (size_t)2 * Sp * (Sp + 8) * esz + (size_t)Sp * (Sp + 4) * 4 + 8 * 16 * 20 * 4 +
         3 * (size_t)hd * 4;
}

template <typename T, int HD>
static int launch_fwd_tc(const void* qkv, const void* bqkv, const int* mask, void* ctx, void* probs, int b, int S, int H,
                         int nh, float p, const int* seed, unsigned stream_id, cudaStream_t st) {
  const int Sp = (S + 15) / 16 * 16;
  const size_t smem = fwd_smem(Sp, HD, sizeof(T));
  auto k = attention_fwd_tc_kernel<T, HD>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
  // 8 warps per (batch, head) for long sequences (64+ tiles of work per product), 4 for short ones
  k<<<dim3(nh, b), Sp >= 64 ? 256 : 128, smem, st>>>((const T*)qkv, (const T*)bqkv, mask, (T*)ctx, (T*)probs, S, Sp, H, nh, p, seed, stream_id);
  return 0;
}

template <typename T, int HD>
static int launch_bwd_tc(const void* dctx, const void* qkv, const void* bqkv, const void* probs, void* dqkv, int b, int S,
                         int H, int nh, float p, const int* seed, unsigned stream_id, float* bias_acc, cudaStream_t st) {
  const int Sp = (S + 15) / 16 * 16;
  const size_t smem = bwd_smem(Sp, HD, sizeof(T));
  if (smem > 227 * 1024) return -6;
  auto k = attention_bwd_tc_kernel<T, HD>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
  k<<<dim3(nh, b), Sp >= 64 ? 256 : 128, smem, st>>>((const T*)dctx, (const T*)qkv, (const T*)bqkv, (const T*)probs, (T*)dqkv, S, Sp, H, nh,
                                    p, seed, stream_id, bias_acc);
  return 0;
}

// dtype: 1 = bf16, 2 = fp16 (fp32 activations use the CUDA-core kernels of attention.cu).
// bias_acc (backward, nullable): 8 replicas x [3H] fp32; when given, the column sums of dqkv (the q/k/v bias
// gradients) are accumulated there so that no separate pass over dqkv is needed.
RB_API int rb_attention_fwd_tc(int dtype, const void* qkv, const void* bqkv, const int* mask, void* ctx, void* probs,
                               int b, int S, int H, int nh, float p, const int* seed, unsigned stream_id,
                               cudaStream_t st) {
  if (S > 128 || S < 1 || H % nh || H % 8) return -4;
  const int hd = H / nh;
  int rc = -4;
  if (dtype == RB_BF16 && hd == 64) rc = launch_fwd_tc<__nv_bfloat16, 64>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st);
  else if (dtype == RB_BF16 && hd == 32) rc = launch_fwd_tc<__nv_bfloat16, 32>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st);
  else if (dtype == RB_F16 && hd == 64) rc = launch_fwd_tc<__half, 64>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st);
  else if (dtype == RB_F16 && hd == 32) rc = launch_fwd_tc<__half, 32>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_attention_bwd_tc(int dtype, const void* dctx, const void* qkv, const void* bqkv, const void* probs,
                               void* dqkv, int b, int S, int H, int nh, float p, const int* seed, unsigned stream_id,
                               float* bias_acc, cudaStream_t st) {
  if (S > 128 || S < 1 || H % nh || H % 8) return -4;
  const int hd = H / nh;
  int rc = -4;
  if (dtype == RB_BF16 && hd == 64) rc = launch_bwd_tc<__nv_bfloat16, 64>(dctx, qkv, bqkv, probs, dqkv, b, S, H, nh, p, seed, stream_id, bias_acc, st);
  else if (dtype == RB_BF16 && hd == 32) rc = launch_bwd_tc<__nv_bfloat16, 32>(dctx, qkv, bqkv, probs, dqkv, b, S, H, nh, p, seed, stream_id, bias_acc, st);
  else if (dtype == RB_F16 && hd == 64) rc = launch_bwd_tc<__half, 64>(dctx, qkv, bqkv, probs, dqkv, b, S, H, nh, p, seed, stream_id, bias_acc, st);
  else if (dtype == RB_F16 && hd == 32) rc = launch_bwd_tc<__half, 32>(dctx, qkv, bqkv, probs, dqkv, b, S, H, nh, p, seed, stream_id, bias_acc, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}
