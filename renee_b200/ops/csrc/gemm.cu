// Encoder GEMMs for sm_100a: one persistent tcgen05 / TMEM kernel family with the element-wise neighbours of
// every linear layer fused into the epilogue.  They stand in for the cuBLAS calls behind the reference's HF
// nn.Linear layers and its FP32Linear (main.py:126-129, dl_base.py:104-111) and for the ATen kernels around
// them (bias add, GELU, dropout, residual add, GELU backward, bias-gradient column sums).
//
//   layout NT  C[M,N] = A[M,K] · B[N,K]^T   forward   (activations x weight^T)       A, B K-major
//   layout NN  C[M,N] = A[M,K] · B[K,N]     dgrad     (output gradient x weight)     A K-major, B MN-major
//   layout TN  C[M,N] = A[K,M]^T · B[K,N]   wgrad     (output gradient^T x input)    A, B MN-major, split-K
//
//   epilogues  STORE                C = acc
//              BIAS_GELU            F = acc + bias ;  C = gelu(F)                    (FFN-1 forward; F kept for backward)
//              BIAS_DROPOUT_RESID   C = R + dropout(acc + bias)                      (out-proj / FFN-2 forward: the LayerNorm input)
//              ADD                  C = acc + R                                      (dgrad joined with the residual gradient)
//              GELU_BWD             C = acc * gelu'(F) ;  column sums of C -> bias gradient accumulators
//              SPLITK               fp32 partials reduced in L2, the last CTA of a tile converts and stores
//
// Structure: one CTA per SM walks the work items (tile x K-split); 320 threads = warp 0 TMA producer, warp 1
// TMEM owner + MMA issuer, warps 2..9 epilogue (two warps per TMEM lane quarter, half of the tile's columns
// each).  128 x BN x 64 tiles (BN = 64 / 128 / 256) in a 4-stage shared-memory ring that keeps streaming
// across item boundaries; TMEM holds two accumulators so the epilogue of item i runs under the main loop of
// item i + 1.  Every wait is bounded (tc.cuh): a protocol error ends with a status word, never with a hang.
// No TMA multicast is used: every CTA loads its own operand tiles.
#include <type_traits>
#include "tc.cuh"

namespace rb {
namespace eg {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;            // 16 KB
constexpr int B_BYTES_MAX = 256 * BK * 2;       // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES_MAX;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 320;
constexpr int ACC_BUFS = 2;
constexpr int ACC_STRIDE = 256;                 // TMEM columns between the two accumulators
constexpr int TMEM_COLS = ACC_BUFS * ACC_STRIDE;

enum Layout : int { L_NT = 0, L_NN = 1, L_TN = 2 };
enum Epi : int { E_STORE = 0, E_BIAS_GELU = 1, E_BIAS_DROPOUT_RESID = 2, E_ADD = 3, E_GELU_BWD = 4, E_SPLITK = 5 };

struct Params {
  int M, N;                      // output rows / columns
  int BN;                        // N tile: 64, 128 or 256
  int n_m_tiles, n_n_tiles;
  int splits, kb_total, kb_per_split;
  void* C; int ldc;
  const void* bias;              // [N]                             BIAS_GELU, BIAS_DROPOUT_RESID
  const void* R; int ldr;        // residual (BIAS_DROPOUT_RESID, ADD) or stored pre-activation F (GELU_BWD)
  void* F; int ldf;              // pre-activation output           BIAS_GELU
  float p; const int* seed; uint32_t stream;        // dropout      BIAS_DROPOUT_RESID
  float* colacc; int col_tot; int col_off;          // GELU_BWD: replicas of [col_tot] floats, this vector at col_off
  float* sk_scratch; unsigned* sk_counters;         // SPLITK: [tiles][BM*BN] fp32 (zero between launches), [tiles]
  int* status;
};

constexpr int kColReplicas = 8;   // must equal the replica count of the deferred column reductions (encoder_ops.cu)

template <typename T> __device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = from_f<T>(v[i]);
  return raw;
}
template <typename T> __device__ __forceinline__ void unpack8_ldg(const T* p, float* out) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = to_f(e[i]);
}

// Sum over the 32 lanes of v[c] for every c in 0..31: lane L returns the total of column L (31 shuffles).
__device__ __forceinline__ float warp_colsum32(float (&v)[32], int lane) {
#pragma unroll
  for (int n = 16; n >= 1; n >>= 1) {
    const bool upper = (lane & n) != 0;
#pragma unroll
    for (int i = 0; i < n; ++i) {
      const float send = upper ? v[i] : v[i + n];
      const float keep_ = upper ? v[i + n] : v[i];
      v[i] = keep_ + __shfl_xor_sync(0xffffffffu, send, n);
    }
  }
  return v[0];
}

// One 32-column fragment of one output row: v[j] is the accumulator of (row, col0 + j).
template <typename T, int EPI>
__device__ __forceinline__ void epilogue_fragment(const Params& p, float (&v)[32], int row, bool row_ok, int col0,
                                                  int lane, uint32_t seed, float inv_keep, int tile, int r, int c_in_tile) {
  T* C = reinterpret_cast<T*>(p.C);
  if (EPI == E_STORE || (EPI == E_SPLITK && p.splits == 1)) {
    if (row_ok) {
#pragma unroll
      for (int j8 = 0; j8 < 4; ++j8) {
        const int c = col0 + 8 * j8;
        if (c < p.N) *reinterpret_cast<uint4*>(C + (size_t)row * p.ldc + c) = pack8<T>(v + 8 * j8);
      }
    }
  } else if (EPI == E_SPLITK) {
    if (row_ok) {
      float* s = p.sk_scratch + (size_t)tile * (BM * p.BN) + (size_t)r * p.BN + c_in_tile;
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4)
        if (col0 + 4 * j4 < p.N) red_add_f32x4(s + 4 * j4, v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
    }
  } else if (EPI == E_BIAS_GELU) {
    if (row_ok) {
      T* F = reinterpret_cast<T*>(p.F);
#pragma unroll
      for (int j8 = 0; j8 < 4; ++j8) {
        const int c = col0 + 8 * j8;
        if (c < p.N) {
          float b[8], f[8], a[8];
          unpack8_ldg<T>(reinterpret_cast<const T*>(p.bias) + c, b);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            f[j] = round_through<T>(v[8 * j8 + j] + b[j]);      // backward differentiates at the stored value
            a[j] = gelu_f(f[j]);
          }
          *reinterpret_cast<uint4*>(F + (size_t)row * p.ldf + c) = pack8<T>(f);
          *reinterpret_cast<uint4*>(C + (size_t)row * p.ldc + c) = pack8<T>(a);
        }
      }
    }
  } else if (EPI == E_BIAS_DROPOUT_RESID) {
    if (row_ok) {
#pragma unroll
      for (int j8 = 0; j8 < 4; ++j8) {
        const int c = col0 + 8 * j8;
        if (c < p.N) {
          float b[8], res[8], o[8];
          unpack8_ldg<T>(reinterpret_cast<const T*>(p.bias) + c, b);
          unpack8_ldg<T>(reinterpret_cast<const T*>(p.R) + (size_t)row * p.ldr + c, res);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float t = v[8 * j8 + j] + b[j];
            if (p.p > 0.f) t = keep(seed, p.stream, (uint32_t)(row * p.N + c + j), p.p) ? t * inv_keep : 0.f;
            o[j] = res[j] + t;
          }
          *reinterpret_cast<uint4*>(C + (size_t)row * p.ldc + c) = pack8<T>(o);
        }
      }
    }
  } else if (EPI == E_ADD) {
    if (row_ok) {
#pragma unroll
      for (int j8 = 0; j8 < 4; ++j8) {
        const int c = col0 + 8 * j8;
        if (c < p.N) {
          float res[8], o[8];
          unpack8_ldg<T>(reinterpret_cast<const T*>(p.R) + (size_t)row * p.ldr + c, res);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[8 * j8 + j] + res[j];
          *reinterpret_cast<uint4*>(C + (size_t)row * p.ldc + c) = pack8<T>(o);
        }
      }
    }
  } else {  // E_GELU_BWD
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
      const int c = col0 + 8 * j8;
      if (row_ok && c < p.N) {
        float f[8];
        unpack8_ldg<T>(reinterpret_cast<const T*>(p.R) + (size_t)row * p.ldr + c, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[8 * j8 + j] = round_through<T>(v[8 * j8 + j] * gelu_grad_f(f[j]));
        *reinterpret_cast<uint4*>(C + (size_t)row * p.ldc + c) = pack8<T>(v + 8 * j8);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[8 * j8 + j] = 0.f;
      }
    }
    if (p.colacc != nullptr) {
      const float s = warp_colsum32(v, lane);        // lane L: sum of column col0 + L over this warp's 32 rows
      if (col0 + lane < p.N)
        atomicAdd(p.colacc + (size_t)(blockIdx.x % kColReplicas) * p.col_tot + p.col_off + col0 + lane, s);
    }
  }
}

template <typename T, int LAYOUT, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
enc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  constexpr bool A_MN = (LAYOUT == L_TN);
  constexpr bool B_MN = (LAYOUT != L_NT);
  constexpr int FMT = (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) ? 1 : 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;          // [ACC_BUFS]
  uint64_t* tmem_empty_bar = tmem_full_bar + ACC_BUFS;   // [ACC_BUFS]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tmem_empty_bar + ACC_BUFS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* s_last = s_abort + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_items = p.n_m_tiles * p.n_n_tiles * p.splits;
  const uint32_t b_bytes = (uint32_t)p.BN * BK * 2;

  if (threadIdx.x == 0) {
    tc::prefetch_tmap(&tmA);
    tc::prefetch_tmap(&tmB);
    for (int s = 0; s < STAGES; ++s) { tc::mbar_init(full_bar + s, 1); tc::mbar_init(empty_bar + s, 1); }
    for (int a = 0; a < ACC_BUFS; ++a) { tc::mbar_init(tmem_full_bar + a, 1); tc::mbar_init(tmem_empty_bar + a, 8); }
    *s_abort = 0;
    *s_last = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_ptr_smem, TMEM_COLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  bool aborted = false;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer: one continuous stream of (item, k block) stages
    int it = 0;
    for (int item = blockIdx.x; item < n_items && !aborted; item += gridDim.x) {
      const int tile = item / p.splits, split = item - tile * p.splits;
      const int m0 = (tile / p.n_n_tiles) * BM, n0 = (tile % p.n_n_tiles) * p.BN;
      const int kb0 = split * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!tc::mbar_wait(empty_bar + s, ph ^ 1, aborted, p.status, tc::SITE_EMPTY, kb)) break;
        uint8_t* sA = smem + s * STAGE_BYTES;
        uint8_t* sB = sA + A_BYTES;
        tc::mbar_expect_tx(full_bar + s, A_BYTES + b_bytes);
        if (A_MN) {
          tc::tma_load_2d(sA, &tmA, full_bar + s, m0, kb * BK);
          tc::tma_load_2d(sA + 8192, &tmA, full_bar + s, m0 + 64, kb * BK);
        } else {
          tc::tma_load_2d(sA, &tmA, full_bar + s, kb * BK, m0);
        }
        if (B_MN) {
          for (int i = 0; i < p.BN / 64; ++i) tc::tma_load_2d(sB + i * 8192, &tmB, full_bar + s, n0 + 64 * i, kb * BK);
        } else {
          tc::tma_load_2d(sB, &tmB, full_bar + s, kb * BK, n0);
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer: accumulator (t_local & 1), reused every second item once the epilogue drained it
    const uint32_t idesc = tc::make_idesc(FMT, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, p.BN);
    int it = 0, t_local = 0;
    for (int item = blockIdx.x; item < n_items && !aborted; item += gridDim.x, ++t_local) {
      const int tile = item / p.splits, split = item - tile * p.splits;
      const int kb0 = split * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
      const int buf = t_local & 1;
      const uint32_t use = (uint32_t)(t_local >> 1);
      if (!tc::mbar_wait(tmem_empty_bar + buf, (use & 1) ^ 1, aborted, p.status, tc::SITE_TMEM_EMPTY, item)) break;
      tc::tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)buf * ACC_STRIDE;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!tc::mbar_wait(full_bar + s, ph, aborted, p.status, tc::SITE_FULL, kb)) break;
        tc::tc_fence_after();
        const uint32_t sA = tc::smem_u32(smem + s * STAGE_BYTES);
        const uint32_t sB = sA + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t ad = A_MN ? tc::make_smem_desc(sA + k * 2048, 8192, 1024) : tc::make_smem_desc(sA + k * 32, 16, 1024);
          const uint64_t bd = B_MN ? tc::make_smem_desc(sB + k * 2048, 8192, 1024) : tc::make_smem_desc(sB + k * 32, 16, 1024);
          tc::umma_f16(d_tmem, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        tc::umma_commit(empty_bar + s);
      }
      if (aborted) break;
      tc::umma_commit(tmem_full_bar + buf);
    }
  } else if (warp >= 2) {
    // ---------------- epilogue: 8 warps; warp w reads TMEM lanes 32 (w & 3) .. +31, columns of half (w - 2) / 4
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int half_cols = p.BN >> 1;
    uint32_t seed = 0u;
    float inv_keep = 1.f;
    if (EPI == E_BIAS_DROPOUT_RESID && p.p > 0.f) { seed = (uint32_t)(*p.seed); inv_keep = 1.f / (1.f - p.p); }
    int t_local = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++t_local) {
      const int tile = item / p.splits;
      const int m0 = (tile / p.n_n_tiles) * BM, n0 = (tile % p.n_n_tiles) * p.BN;
      const int row = m0 + r;
      const bool row_ok = row < p.M;
      const int buf = t_local & 1;
      const uint32_t use = (uint32_t)(t_local >> 1);
      if (!tc::mbar_wait(tmem_full_bar + buf, use & 1, aborted, p.status, tc::SITE_TMEM_FULL, item)) *s_abort = 1;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (*s_abort) break;                                   // the same answer in all eight warps
      tc::tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * ACC_STRIDE + (uint32_t)(half * half_cols);
      for (int c0 = 0; c0 < half_cols; c0 += 32) {
        float v[32];
        tc::tmem_ld32(tbase + c0, v);
        const int c_in_tile = half * half_cols + c0;
        epilogue_fragment<T, EPI>(p, v, row, row_ok, n0 + c_in_tile, lane, seed, inv_keep, tile, r, c_in_tile);
      }
      // every tcgen05.ld of this item has completed (tmem_ld32 waits): hand the accumulator back to the MMA warp
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(tmem_empty_bar + buf);
      if (EPI == E_SPLITK && p.splits > 1) {
        // split-K fix-up: the CTA that adds the last partial of a tile converts the sum and re-zeroes the scratch
        __threadfence();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (threadIdx.x == 64) *s_last = (atomicAdd(p.sk_counters + tile, 1u) == (unsigned)(p.splits - 1)) ? 1 : 0;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (*s_last) {
          __threadfence();
          if (row_ok) {
            T* C = reinterpret_cast<T*>(p.C);
            float* srow = p.sk_scratch + (size_t)tile * (BM * p.BN) + (size_t)r * p.BN + half * half_cols;
            for (int c = 0; c < half_cols; c += 8) {
              const int col = n0 + half * half_cols + c;
              if (col < p.N) {
                const float4 x0 = __ldcg(reinterpret_cast<const float4*>(srow + c));
                const float4 x1 = __ldcg(reinterpret_cast<const float4*>(srow + c + 4));
                __stcg(reinterpret_cast<float4*>(srow + c), make_float4(0.f, 0.f, 0.f, 0.f));
                __stcg(reinterpret_cast<float4*>(srow + c + 4), make_float4(0.f, 0.f, 0.f, 0.f));
                const float o[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                *reinterpret_cast<uint4*>(C + (size_t)row * p.ldc + col) = pack8<T>(o);
              }
            }
          }
          if (threadIdx.x == 64) p.sk_counters[tile] = 0u;
        }
      }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------ LayerNorm of a stored input
// y = LN(pre) with the row statistics kept for the backward pass; `pre` was written by the BIAS_DROPOUT_RESID
// epilogue.  One warp per row, 16-byte accesses.
template <typename T, int NV>
__global__ void __launch_bounds__(128) ln_fwd_kernel(const T* __restrict__ pre, const T* __restrict__ gamma,
                                                     const T* __restrict__ beta, T* __restrict__ y,
                                                     float* __restrict__ mean, float* __restrict__ rstd, int rows, int H,
                                                     float eps) {
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  float v[NV][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (lane + 32 * i) * 8;
    if (col < H) {
      load8(pre + (size_t)row * H + col, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[i][j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
    }
  }
  const float mu = warp_sum(sum) / H;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (lane + 32 * i) * 8;
    if (col < H) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mu; sq += d * d; }
    }
  }
  const float rs = rsqrtf(warp_sum(sq) / H + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (lane + 32 * i) * 8;
    if (col < H) {
      float g[8], b[8], o[8];
      load8(gamma + col, g);
      load8(beta + col, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mu) * rs * g[j] + b[j];
      store8(y + (size_t)row * H + col, o);
    }
  }
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
}

}  // namespace eg
}  // namespace rb

using namespace rb;
using namespace rb::eg;

template <typename T, int LAYOUT, int EPI>
static int launch_enc_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int ctas, cudaStream_t st) {
  static bool attr_set = false;
  auto k = enc_gemm_kernel<T, LAYOUT, EPI>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -5;
    attr_set = true;
  }
  k<<<ctas, THREADS, SMEM_BYTES, st>>>(ta, tb, p);
  return 0;
}

template <typename T>
static int dispatch_enc_gemm(int layout, int epi, const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int ctas,
                             cudaStream_t st) {
  if (layout == L_NT) {
    if (epi == E_STORE) return launch_enc_gemm<T, L_NT, E_STORE>(ta, tb, p, ctas, st);
    if (epi == E_BIAS_GELU) return launch_enc_gemm<T, L_NT, E_BIAS_GELU>(ta, tb, p, ctas, st);
    if (epi == E_BIAS_DROPOUT_RESID) return launch_enc_gemm<T, L_NT, E_BIAS_DROPOUT_RESID>(ta, tb, p, ctas, st);
  } else if (layout == L_NN) {
    if (epi == E_STORE) return launch_enc_gemm<T, L_NN, E_STORE>(ta, tb, p, ctas, st);
    if (epi == E_ADD) return launch_enc_gemm<T, L_NN, E_ADD>(ta, tb, p, ctas, st);
    if (epi == E_GELU_BWD) return launch_enc_gemm<T, L_NN, E_GELU_BWD>(ta, tb, p, ctas, st);
  } else if (layout == L_TN) {
    if (epi == E_SPLITK) return launch_enc_gemm<T, L_TN, E_SPLITK>(ta, tb, p, ctas, st);
  }
  return -4;
}

// N tile: the candidate with the fewest rounds x tile cost over the SMs (small problems want more, smaller tiles)
static int pick_bn(int M, int N, int forced) {
  if (forced == 64 || forced == 128 || forced == 256) return forced;
  const int sms = sm_count();
  const int mt = (M + BM - 1) / BM;
  int best = 256;
  long best_cost = -1;
  for (int bn = 256; bn >= 64; bn >>= 1) {
    if (bn > 64 && bn / 2 >= N) continue;                  // a narrower tile already covers every column
    const long tiles = (long)mt * ((N + bn - 1) / bn);
    const long cost = ((tiles + sms - 1) / sms) * (bn + 48);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

// C = op(A) op(B) with a fused epilogue; see the head of this file.  Leading dimensions in elements.
//   layout 0 (NT): A[M, lda>=K], B[N, ldb>=K];  1 (NN): A[M, lda>=K], B[K, ldb>=N];  2 (TN): A[K, lda>=M], B[K, ldb>=N]
//   dtype: RB_BF16 or RB_F16 (operands, C, bias, R and F all have it; accumulation is fp32)
//   splits (TN only): K-splits; > 1 needs sk_scratch of n_tiles * 128 * BN floats (zero on entry, left zero) and
//   sk_counters of n_tiles words (zero on entry, left zero).  bn_forced: 0 = choose.
// Returns 0, or -3 for an unsupported shape (the caller then uses the library GEMM).
RB_API int rb_enc_gemm(int dtype, int layout, int epi, const void* A, const void* B, void* C, int M, int N, int K, int lda,
                       int ldb, int ldc, const void* bias, const void* R, int ldr, void* F, int ldf, float p_drop,
                       const int* seed, unsigned stream_id, float* colacc, int col_tot, int col_off, float* sk_scratch,
                       unsigned* sk_counters, int splits, int bn_forced, int* status, cudaStream_t st) {
  if (dtype != RB_BF16 && dtype != RB_F16) return -1;
  if (M < 1 || N < 1 || K < 1 || N % 8 || lda % 8 || ldb % 8 || ldc % 8 || ldr % 8 || ldf % 8) return -3;
  if (layout == L_TN && M % 8) return -3;
  const bool bf16 = dtype == RB_BF16;
  const int BN = pick_bn(M, N, bn_forced);
  CUtensorMap ta, tb;
  int rc;
  if (layout == L_TN) rc = tc::make_tmap_2d(&ta, A, K, M, lda, 64, 64, bf16);
  else rc = tc::make_tmap_2d(&ta, A, M, K, lda, 64, BM, bf16);
  if (rc) return rc;
  if (layout == L_NT) rc = tc::make_tmap_2d(&tb, B, N, K, ldb, 64, BN, bf16);
  else rc = tc::make_tmap_2d(&tb, B, K, N, ldb, 64, 64, bf16);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.BN = BN;
  p.n_m_tiles = (M + BM - 1) / BM; p.n_n_tiles = (N + BN - 1) / BN;
  p.kb_total = (K + BK - 1) / BK;
  if (layout != L_TN || splits < 1) splits = 1;
  if (splits > p.kb_total) splits = p.kb_total;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
  if (p.splits > 1 && (sk_scratch == nullptr || sk_counters == nullptr)) return -3;
  p.C = C; p.ldc = ldc; p.bias = bias; p.R = R; p.ldr = ldr; p.F = F; p.ldf = ldf;
  p.p = p_drop; p.seed = seed; p.stream = stream_id;
  p.colacc = colacc; p.col_tot = col_tot; p.col_off = col_off;
  p.sk_scratch = sk_scratch; p.sk_counters = sk_counters; p.status = status;
  if ((epi == E_BIAS_GELU || epi == E_BIAS_DROPOUT_RESID) && bias == nullptr) return -3;
  if ((epi == E_BIAS_DROPOUT_RESID || epi == E_ADD || epi == E_GELU_BWD) && R == nullptr) return -3;
  if (epi == E_BIAS_GELU && F == nullptr) return -3;
  if (epi == E_BIAS_DROPOUT_RESID && p_drop > 0.f && seed == nullptr) return -3;
  const int n_items = p.n_m_tiles * p.n_n_tiles * p.splits;
  const int ctas = n_items < sm_count() ? n_items : sm_count();
  rc = bf16 ? dispatch_enc_gemm<__nv_bfloat16>(layout, epi, ta, tb, p, ctas, st)
            : dispatch_enc_gemm<__half>(layout, epi, ta, tb, p, ctas, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

// What rb_enc_gemm will use for (M, N, K): N tile, K-splits for layout TN, number of tiles (scratch sizing).
RB_API int rb_enc_gemm_plan(int layout, int M, int N, int K, int bn_forced, int* bn_out, int* splits_out, int* tiles_out) {
  const int BN = pick_bn(M, N, bn_forced);
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int splits = 1;
  if (layout == L_TN) {
    const int kb = (K + BK - 1) / BK;
    splits = sm_count() / tiles;
    if (splits < 1) splits = 1;
    if (splits > 16) splits = 16;
    if (splits > kb) splits = kb;
  }
  *bn_out = BN; *splits_out = splits; *tiles_out = tiles;
  return 0;
}

#define EG_DISPATCH_NV(H, ...)                                                     \
  {                                                                                \
    const int nv_ = ((H) + 255) / 256;                                             \
    if (nv_ <= 1) { constexpr int NV = 1; __VA_ARGS__; }                           \
    else if (nv_ <= 2) { constexpr int NV = 2; __VA_ARGS__; }                      \
    else if (nv_ <= 3) { constexpr int NV = 3; __VA_ARGS__; }                      \
    else if (nv_ <= 4) { constexpr int NV = 4; __VA_ARGS__; }                      \
    else if (nv_ <= 8) { constexpr int NV = 8; __VA_ARGS__; }                      \
    else return -2;                                                                \
  }

RB_API int rb_ln_fwd(int dtype, const void* pre, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                     int rows, int H, float eps, cudaStream_t st) {
  if (H % 8 || rows < 1) return -3;
  const int blocks = (rows + 3) / 4;
  switch (dtype) {
    case RB_F32: { using T = float; EG_DISPATCH_NV(H, (ln_fwd_kernel<T, NV><<<blocks, 128, 0, st>>>((const T*)pre, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, H, eps))); break; }
    case RB_BF16: { using T = __nv_bfloat16; EG_DISPATCH_NV(H, (ln_fwd_kernel<T, NV><<<blocks, 128, 0, st>>>((const T*)pre, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, H, eps))); break; }
    case RB_F16: { using T = __half; EG_DISPATCH_NV(H, (ln_fwd_kernel<T, NV><<<blocks, 128, 0, st>>>((const T*)pre, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, H, eps))); break; }
    default: return -1;
  }
  RB_LAUNCH_CHECK();
  return 0;
}
