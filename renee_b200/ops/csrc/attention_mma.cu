// Register-resident self-attention forward/backward for 16-bit activations, head dim 64, S <= 512
// (one CTA per (batch, head) up to 128 tokens; blocked kernels, further down, for 129..512).
// Same fusion and interface as attention_tc.cu (bias add, scale, key-padding mask, softmax, counter-based
// attention dropout, head split/merge addressing, q/k/v bias gradients), organised so that the score
// matrix never touches shared memory:
//   * one CTA per (batch, head); the padded sequence SP is 32, 64 or 128 and the CTA has SP/16 warps;
//   * a warp owns 16 query rows.  S = Q K^T (forward) or dP = dO V^T (backward) for those rows is
//     accumulated in registers by m16n8k16 MMAs fed with ldmatrix, the softmax / softmax-gradient runs on
//     the accumulator fragments (a row lives in one quad: two shuffles per reduction), and the fragments
//     are re-packed in place as the A operand of the next product (O = P~ V, dQ = dS K);
//   * only dK = dS^T Q and dV = P~^T dO need other warps' rows: dS and P~ go through shared memory once
//     and each warp then owns 16 key rows.
// Shared memory per CTA: 3 (forward) or 4 (backward) [SP][72] operand tiles, plus two [SP][SP+8] tiles in
// the backward: 14 KB / 24 KB at SP = 32, so many CTAs share an SM at short sequences; 55 KB / 143 KB at
// SP = 128.  At S = 32 a head is a quarter of the 128-row tcgen05 tile, so the warp-level MMA is the
// shape that fits this op; the classifier GEMMs, where the FLOPs are, use tcgen05.
// Reference behaviour: the attention of the HF DistilBERT layers that main.py:225-262 wraps.
#include <type_traits>
#include "common.cuh"

namespace rb {
namespace amma {

constexpr int HD = 64;
constexpr int RP = HD + 8;   // operand row pitch (elements): 144 B keeps the 8 rows of an ldmatrix on distinct banks

template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
};
template <> struct Pack<__half> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
};

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  return v;
}

// acc[j] (j = 8-wide tile of columns) += A(16 rows r0.. of `a`, all HD columns) * B^T, B = SP rows of `bsm`:
// the shape of Q K^T and of dO V^T.  Both operands are [row][RP] tiles.
template <typename T, int SP>
__device__ __forceinline__ void rows_times_transposed(float (&acc)[SP / 8][4], const T* a, const T* bsm, int r0, int lane) {
  uint32_t af[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk)
    ldsm4(af[kk], a + (r0 + (lane & 7) + ((lane >> 3) & 1) * 8) * RP + kk * 16 + (lane >> 4) * 8);
#pragma unroll
  for (int j = 0; j < SP / 8; ++j) {
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk += 2) {
      uint32_t bf[4];   // {b0, b1} of k-step kk, {b0, b1} of k-step kk + 1
      ldsm4(bf, bsm + (8 * j + (lane & 7)) * RP + kk * 16 + (lane >> 3) * 8);
      mma16816<T>(acc[j], af[kk], bf[0], bf[1]);
      mma16816<T>(acc[j], af[kk + 1], bf[2], bf[3]);
    }
  }
}

// out[jd] (jd = 8-wide tile of the HD columns) += A * B for a 16 x SP A held as packed fragments
// (afr[kq] = the 16 x 16 block of columns 16 kq..) and B = the SP rows of the [row][RP] tile `bsm`.
template <typename T, int SP>
__device__ __forceinline__ void frag_times_rows(float (&out)[HD / 8][4], const uint32_t (&afr)[SP / 16][4], const T* bsm, int lane) {
#pragma unroll
  for (int kq = 0; kq < SP / 16; ++kq) {
#pragma unroll
    for (int jd = 0; jd < HD / 8; jd += 2) {
      uint32_t bf[4];   // {b0, b1} of column tile jd, {b0, b1} of column tile jd + 1
      ldsm4_t(bf, bsm + (16 * kq + (lane & 7) + ((lane >> 3) & 1) * 8) * RP + 8 * jd + (lane >> 4) * 8);
      mma16816<T>(out[jd], afr[kq], bf[0], bf[1]);
      mma16816<T>(out[jd + 1], afr[kq], bf[2], bf[3]);
    }
  }
}

// out[jd] += A^T * B where A is the [SP][PP] tile `asm_` (rows = reduction index) restricted to its 16 columns
// c0.., and B = the SP rows of the [row][RP] tile `bsm`: the shape of dS^T Q and of P~^T dO.
template <typename T, int SP>
__device__ __forceinline__ void transposed_times_rows(float (&out)[HD / 8][4], const T* asm_, int PP, int c0, const T* bsm, int lane) {
#pragma unroll
  for (int kq = 0; kq < SP / 16; ++kq) {
    uint32_t af[4];
    const int mi = lane >> 3;
    ldsm4_t(af, asm_ + (16 * kq + (lane & 7) + (mi >> 1) * 8) * PP + c0 + (mi & 1) * 8);
#pragma unroll
    for (int jd = 0; jd < HD / 8; jd += 2) {
      uint32_t bf[4];
      ldsm4_t(bf, bsm + (16 * kq + (lane & 7) + ((lane >> 3) & 1) * 8) * RP + 8 * jd + (lane >> 4) * 8);
      mma16816<T>(out[jd], af, bf[0], bf[1]);
      mma16816<T>(out[jd + 1], af, bf[2], bf[3]);
    }
  }
}

// Writes the warp's 16 x HD accumulator tile (rows row0.. of the sequence) to global rows of stride ld and,
// when col_sums != nullptr, adds the column sums of the rounded values to col_sums[0..HD) in shared memory.
template <typename T>
__device__ __forceinline__ void write_rows(const float (&out)[HD / 8][4], T* dst, int ld, int row0, int S, int lane,
                                           float* col_sums) {
  const int g = lane >> 2, t = lane & 3;
  const bool v0 = row0 + g < S, v1 = row0 + g + 8 < S;
#pragma unroll
  for (int jd = 0; jd < HD / 8; ++jd) {
    const uint32_t lo = Pack<T>::pack(out[jd][0], out[jd][1]);
    const uint32_t hi = Pack<T>::pack(out[jd][2], out[jd][3]);
    if (v0) *reinterpret_cast<uint32_t*>(dst + (size_t)g * ld + 8 * jd + 2 * t) = lo;
    if (v1) *reinterpret_cast<uint32_t*>(dst + (size_t)(g + 8) * ld + 8 * jd + 2 * t) = hi;
    if (col_sums != nullptr) {
      const float2 a = Pack<T>::unpack(lo), b = Pack<T>::unpack(hi);
      float s0 = (v0 ? a.x : 0.f) + (v1 ? b.x : 0.f);
      float s1 = (v0 ? a.y : 0.f) + (v1 ? b.y : 0.f);
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      }
      if (g == 0) {
        atomicAdd(col_sums + 8 * jd + 2 * t, s0);
        atomicAdd(col_sums + 8 * jd + 2 * t + 1, s1);
      }
    }
  }
}

// Stages (q + bq, k + bk, v + bv [, dO]) of one (batch, head) as [SP][RP] tiles; rows >= S are zero.
// The CTA has SP * 2 threads and the tiles SP * 8 segments of 8 columns, so a thread owns the same 8 columns of
// four rows: all of its global loads are issued before the first one is used.
template <typename T, int SP, bool WITH_DO>
__device__ __forceinline__ void stage_operands(const T* __restrict__ qkv, const T* __restrict__ bqkv, const T* __restrict__ dctx,
                                               T* sQ, T* sK, T* sV, T* sDO, int b, int h, int S, int H) {
  constexpr int ROWS_PER_PASS = SP * 2 / 8;
  const int d = (threadIdx.x & 7) * 8, s0 = threadIdx.x >> 3;
  Raw8<T> rq[4], rk[4], rv[4], rg[4];
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int s = s0 + it * ROWS_PER_PASS;
    if (s < S) {
      const size_t base = (size_t)(b * S + s) * 3 * H + h * HD + d;
      rq[it] = load_raw8(qkv + base); rk[it] = load_raw8(qkv + base + H); rv[it] = load_raw8(qkv + base + 2 * H);
      if constexpr (WITH_DO) rg[it] = load_raw8(dctx + (size_t)(b * S + s) * H + h * HD + d);
    }
  }
  float bq[8], bk[8], bv[8];
  load8(bqkv + h * HD + d, bq); load8(bqkv + H + h * HD + d, bk); load8(bqkv + 2 * H + h * HD + d, bv);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int s = s0 + it * ROWS_PER_PASS;
    float q[8], k[8], v[8];
    if (s < S) {
      unpack8(rq[it], q); unpack8(rk[it], k); unpack8(rv[it], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) { q[j] += bq[j]; k[j] += bk[j]; v[j] += bv[j]; }
      if constexpr (WITH_DO) *reinterpret_cast<uint4*>(sDO + s * RP + d) = rg[it].v;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { q[j] = 0.f; k[j] = 0.f; v[j] = 0.f; }
      if constexpr (WITH_DO) *reinterpret_cast<uint4*>(sDO + s * RP + d) = make_uint4(0u, 0u, 0u, 0u);
    }
    store8(sQ + s * RP + d, q); store8(sK + s * RP + d, k); store8(sV + s * RP + d, v);
  }
}

template <typename T, int SP>
__global__ void __launch_bounds__(SP * 2, SP == 128 ? 2 : 1) attention_fwd_mma_kernel(
    const T* __restrict__ qkv, const T* __restrict__ bqkv, const int* __restrict__ mask, T* __restrict__ ctx,
    T* __restrict__ probs, int S, int H, int nh, float p, const int* __restrict__ seed_ptr, uint32_t stream) {
  rb::grid_dep_wait();        // launched with launch_pdl: nothing above touches global memory
  rb::grid_dep_launch();      // the kernel that follows may start its set-up; it waits for this grid before reading
  extern __shared__ __align__(128) uint8_t sm_raw[];
  T* sQ = reinterpret_cast<T*>(sm_raw);
  T* sK = sQ + SP * RP;
  T* sV = sK + SP * RP;
  uint8_t* sCode = reinterpret_cast<uint8_t*>(sV + SP * RP);   // per key: 0 = beyond S, 1 = attend, 2 = masked
  const int h = blockIdx.x, b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const float scale = rsqrtf((float)HD);
  for (int j = threadIdx.x; j < SP; j += blockDim.x) sCode[j] = j < S ? (mask[b * S + j] != 0 ? 1 : 2) : 0;
  stage_operands<T, SP, false>(qkv, bqkv, nullptr, sQ, sK, sV, nullptr, b, h, S, H);
  __syncthreads();
  const int r0 = warp * 16;
  float acc[SP / 8][4];
#pragma unroll
  for (int j = 0; j < SP / 8; ++j) { acc[j][0] = 0.f; acc[j][1] = 0.f; acc[j][2] = 0.f; acc[j][3] = 0.f; }
  rows_times_transposed<T, SP>(acc, sQ, sK, r0, lane);
  // softmax of rows r0 + g (elements 0, 1 of each tile) and r0 + g + 8 (elements 2, 3)
  float mx0 = -1e30f, mx1 = -1e30f;
#pragma unroll
  for (int j = 0; j < SP / 8; ++j) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const bool on = sCode[8 * j + 2 * t + e] == 1;
      acc[j][e] = on ? acc[j][e] * scale : -1e30f;
      acc[j][2 + e] = on ? acc[j][2 + e] * scale : -1e30f;
      mx0 = fmaxf(mx0, acc[j][e]);
      mx1 = fmaxf(mx1, acc[j][2 + e]);
    }
  }
  mx0 = quad_max(mx0); mx1 = quad_max(mx1);
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int j = 0; j < SP / 8; ++j) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const bool in_range = sCode[8 * j + 2 * t + e] != 0;
      acc[j][e] = in_range ? __expf(acc[j][e] - mx0) : 0.f;
      acc[j][2 + e] = in_range ? __expf(acc[j][2 + e] - mx1) : 0.f;
      sum0 += acc[j][e];
      sum1 += acc[j][2 + e];
    }
  }
  sum0 = quad_sum(sum0); sum1 = quad_sum(sum1);
  const int i0 = r0 + g, i1 = r0 + g + 8;
  const float inv0 = i0 < S ? 1.f / sum0 : 0.f, inv1 = i1 < S ? 1.f / sum1 : 0.f;
  const size_t prow0 = ((size_t)(b * nh + h) * S + i0) * S, prow1 = ((size_t)(b * nh + h) * S + i1) * S;
  const bool pair_store = (S & 1) == 0;   // then every (row, even column) element is 4-byte aligned
  uint32_t pf[SP / 16][4];                // P~ as the A operand of O = P~ V
#pragma unroll
  for (int j = 0; j < SP / 8; ++j) {
    const int c = 8 * j + 2 * t;
    // the stored probabilities are the rounded ones, as in the unfused op
    const uint32_t u0 = Pack<T>::pack(acc[j][0] * inv0, acc[j][1] * inv0);
    const uint32_t u1 = Pack<T>::pack(acc[j][2] * inv1, acc[j][3] * inv1);
    if (i0 < S) {
      if (pair_store) { if (c < S) *reinterpret_cast<uint32_t*>(probs + prow0 + c) = u0; }
      else {
        const T* e = reinterpret_cast<const T*>(&u0);
        if (c < S) probs[prow0 + c] = e[0];
        if (c + 1 < S) probs[prow0 + c + 1] = e[1];
      }
    }
    if (i1 < S) {
      if (pair_store) { if (c < S) *reinterpret_cast<uint32_t*>(probs + prow1 + c) = u1; }
      else {
        const T* e = reinterpret_cast<const T*>(&u1);
        if (c < S) probs[prow1 + c] = e[0];
        if (c + 1 < S) probs[prow1 + c + 1] = e[1];
      }
    }
    float2 q0 = Pack<T>::unpack(u0), q1 = Pack<T>::unpack(u1);
    if (p > 0.f) {
      q0.x = keep(seed, stream, (uint32_t)(prow0 + c), p) ? q0.x * inv_keep : 0.f;
      q0.y = keep(seed, stream, (uint32_t)(prow0 + c + 1), p) ? q0.y * inv_keep : 0.f;
      q1.x = keep(seed, stream, (uint32_t)(prow1 + c), p) ? q1.x * inv_keep : 0.f;
      q1.y = keep(seed, stream, (uint32_t)(prow1 + c + 1), p) ? q1.y * inv_keep : 0.f;
    }
    // tiles 2 kq and 2 kq + 1 are the left and right halves of the 16-wide A block kq
    pf[j >> 1][(j & 1) * 2 + 0] = Pack<T>::pack(q0.x, q0.y);
    pf[j >> 1][(j & 1) * 2 + 1] = Pack<T>::pack(q1.x, q1.y);
  }
  float out[HD / 8][4];
#pragma unroll
  for (int jd = 0; jd < HD / 8; ++jd) { out[jd][0] = 0.f; out[jd][1] = 0.f; out[jd][2] = 0.f; out[jd][3] = 0.f; }
  frag_times_rows<T, SP>(out, pf, sV, lane);
  write_rows<T>(out, ctx + (size_t)(b * S + r0) * H + h * HD, H, r0, S, lane, nullptr);
}

template <typename T, int SP>
__global__ void __launch_bounds__(SP * 2) attention_bwd_mma_kernel(
    const T* __restrict__ dctx, const T* __restrict__ qkv, const T* __restrict__ bqkv, const T* __restrict__ probs,
    T* __restrict__ dqkv, int S, int H, int nh, float p, const int* __restrict__ seed_ptr, uint32_t stream,
    float* __restrict__ bias_acc) {
  rb::grid_dep_wait();
  rb::grid_dep_launch();
  extern __shared__ __align__(128) uint8_t sm_raw[];
  constexpr int PP = SP + 8;   // 4-byte fragment stores of a quad group land on distinct banks
  T* sQ = reinterpret_cast<T*>(sm_raw);
  T* sK = sQ + SP * RP;
  T* sV = sK + SP * RP;
  T* sDO = sV + SP * RP;
  T* sDS = sDO + SP * RP;      // [query][key] dS
  T* sW = sDS + SP * PP;       // [query][key] dropped-out probabilities P~
  float* sBias = reinterpret_cast<float*>(sW + SP * PP);   // [3][HD] column sums of dQ, dK, dV
  const int h = blockIdx.x, b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const float scale = rsqrtf((float)HD);
  if (bias_acc != nullptr)
    for (int i = threadIdx.x; i < 3 * HD; i += blockDim.x) sBias[i] = 0.f;
  stage_operands<T, SP, true>(qkv, bqkv, dctx, sQ, sK, sV, sDO, b, h, S, H);
  __syncthreads();
  const int r0 = warp * 16;
  {
    // dP for this warp's 16 query rows, then dS and P~ in registers
    float acc[SP / 8][4];
#pragma unroll
    for (int j = 0; j < SP / 8; ++j) { acc[j][0] = 0.f; acc[j][1] = 0.f; acc[j][2] = 0.f; acc[j][3] = 0.f; }
    rows_times_transposed<T, SP>(acc, sDO, sV, r0, lane);
    const int i0 = r0 + g, i1 = r0 + g + 8;
    const size_t prow0 = ((size_t)(b * nh + h) * S + i0) * S, prow1 = ((size_t)(b * nh + h) * S + i1) * S;
    const bool pair_load = (S & 1) == 0;
    uint32_t wf[SP / 8][2];   // P~ pairs of rows i0 / i1, later the probabilities' products
    float dot0 = 0.f, dot1 = 0.f;
#pragma unroll
    for (int j = 0; j < SP / 8; ++j) {
      const int c = 8 * j + 2 * t;
      float2 pr0 = make_float2(0.f, 0.f), pr1 = make_float2(0.f, 0.f);
      if (i0 < S && c < S) {
        if (pair_load) pr0 = Pack<T>::unpack(*reinterpret_cast<const uint32_t*>(probs + prow0 + c));
        else { pr0.x = to_f(probs[prow0 + c]); if (c + 1 < S) pr0.y = to_f(probs[prow0 + c + 1]); }
      }
      if (i1 < S && c < S) {
        if (pair_load) pr1 = Pack<T>::unpack(*reinterpret_cast<const uint32_t*>(probs + prow1 + c));
        else { pr1.x = to_f(probs[prow1 + c]); if (c + 1 < S) pr1.y = to_f(probs[prow1 + c + 1]); }
      }
      float m00 = 1.f, m01 = 1.f, m10 = 1.f, m11 = 1.f;
      if (p > 0.f) {
        m00 = keep(seed, stream, (uint32_t)(prow0 + c), p) ? inv_keep : 0.f;
        m01 = keep(seed, stream, (uint32_t)(prow0 + c + 1), p) ? inv_keep : 0.f;
        m10 = keep(seed, stream, (uint32_t)(prow1 + c), p) ? inv_keep : 0.f;
        m11 = keep(seed, stream, (uint32_t)(prow1 + c + 1), p) ? inv_keep : 0.f;
      }
      // dP~ -> dP through the dropout mask; acc keeps dP, the probabilities move to wf as P (plain) for now
      acc[j][0] *= m00; acc[j][1] *= m01; acc[j][2] *= m10; acc[j][3] *= m11;
      dot0 += acc[j][0] * pr0.x + acc[j][1] * pr0.y;
      dot1 += acc[j][2] * pr1.x + acc[j][3] * pr1.y;
      // dS needs the row's dot product first: park P * dP and P, finish below
      const uint32_t w0 = Pack<T>::pack(pr0.x * m00, pr0.y * m01), w1 = Pack<T>::pack(pr1.x * m10, pr1.y * m11);
      *reinterpret_cast<uint32_t*>(sW + i0 * PP + c) = w0;
      *reinterpret_cast<uint32_t*>(sW + i1 * PP + c) = w1;
      wf[j][0] = Pack<T>::pack(pr0.x, pr0.y);   // exact: the probabilities are already T values
      wf[j][1] = Pack<T>::pack(pr1.x, pr1.y);
    }
    dot0 = quad_sum(dot0); dot1 = quad_sum(dot1);
    uint32_t dsf[SP / 16][4];   // dS as the A operand of dQ = dS K
#pragma unroll
    for (int j = 0; j < SP / 8; ++j) {
      const int c = 8 * j + 2 * t;
      const float2 pr0 = Pack<T>::unpack(wf[j][0]), pr1 = Pack<T>::unpack(wf[j][1]);
      const uint32_t d0 = Pack<T>::pack(pr0.x * (acc[j][0] - dot0) * scale, pr0.y * (acc[j][1] - dot0) * scale);
      const uint32_t d1 = Pack<T>::pack(pr1.x * (acc[j][2] - dot1) * scale, pr1.y * (acc[j][3] - dot1) * scale);
      *reinterpret_cast<uint32_t*>(sDS + i0 * PP + c) = d0;
      *reinterpret_cast<uint32_t*>(sDS + i1 * PP + c) = d1;
      dsf[j >> 1][(j & 1) * 2 + 0] = d0;
      dsf[j >> 1][(j & 1) * 2 + 1] = d1;
    }
    float out[HD / 8][4];
#pragma unroll
    for (int jd = 0; jd < HD / 8; ++jd) { out[jd][0] = 0.f; out[jd][1] = 0.f; out[jd][2] = 0.f; out[jd][3] = 0.f; }
    frag_times_rows<T, SP>(out, dsf, sK, lane);
    write_rows<T>(out, dqkv + (size_t)(b * S + r0) * 3 * H + h * HD, 3 * H, r0, S, lane,
                  bias_acc != nullptr ? sBias : nullptr);
  }
  __syncthreads();
  // this warp's 16 key rows of dK = dS^T Q and dV = P~^T dO
  {
    float out[HD / 8][4];
#pragma unroll
    for (int jd = 0; jd < HD / 8; ++jd) { out[jd][0] = 0.f; out[jd][1] = 0.f; out[jd][2] = 0.f; out[jd][3] = 0.f; }
    transposed_times_rows<T, SP>(out, sDS, PP, r0, sQ, lane);
    write_rows<T>(out, dqkv + (size_t)(b * S + r0) * 3 * H + H + h * HD, 3 * H, r0, S, lane,
                  bias_acc != nullptr ? sBias + HD : nullptr);
#pragma unroll
    for (int jd = 0; jd < HD / 8; ++jd) { out[jd][0] = 0.f; out[jd][1] = 0.f; out[jd][2] = 0.f; out[jd][3] = 0.f; }
    transposed_times_rows<T, SP>(out, sW, PP, r0, sDO, lane);
    write_rows<T>(out, dqkv + (size_t)(b * S + r0) * 3 * H + 2 * H + h * HD, 3 * H, r0, S, lane,
                  bias_acc != nullptr ? sBias + 2 * HD : nullptr);
  }
  if (bias_acc != nullptr) {
    // the bias gradient of the packed projection is the column sum of dqkv: add this (batch, head)'s part to
    // one of the 8 replicas of the step-wide accumulator (converted later by the deferred finalize kernel)
    __syncthreads();
    float* my_acc = bias_acc + (size_t)((blockIdx.y * gridDim.x + blockIdx.x) % 8) * 3 * H;
    for (int i = threadIdx.x; i < 3 * HD; i += blockDim.x)
      atomicAdd(my_acc + (i / HD) * H + h * HD + (i % HD), sBias[i]);
  }
}

template <int SP> constexpr size_t fwd_smem(size_t esz) { return (size_t)3 * SP * RP * esz + SP; }
template <int SP> constexpr size_t bwd_smem(size_t esz) {
  return (size_t)4 * SP * RP * esz + (size_t)2 * SP * (SP + 8) * esz + 3 * HD * sizeof(float);
}

template <typename T, int SP>
static int launch_fwd(const void* qkv, const void* bqkv, const int* mask, void* ctx, void* probs, int b, int S, int H,
                      int nh, float p, const int* seed, unsigned stream_id, cudaStream_t st) {
  auto k = attention_fwd_mma_kernel<T, SP>;
  constexpr size_t smem = fwd_smem<SP>(sizeof(T));
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
  rb::launch_pdl(k, dim3(nh, b), dim3(SP * 2), smem, st, (const T*)qkv, (const T*)bqkv, mask, (T*)ctx, (T*)probs, S, H, nh, p, seed, stream_id);
  return 0;
}

template <typename T, int SP>
static int launch_bwd(const void* dctx, const void* qkv, const void* bqkv, const void* probs, void* dqkv, int b, int S,
                      int H, int nh, float p, const int* seed, unsigned stream_id, float* bias_acc, cudaStream_t st) {
  auto k = attention_bwd_mma_kernel<T, SP>;
  constexpr size_t smem = bwd_smem<SP>(sizeof(T));
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
  rb::launch_pdl(k, dim3(nh, b), dim3(SP * 2), smem, st, (const T*)dctx, (const T*)qkv, (const T*)bqkv, (const T*)probs,
                 (T*)dqkv, S, H, nh, p, seed, stream_id, bias_acc);
  return 0;
}


// ------------------------------------------------------------------------------------ sequences of 129..512 tokens
// Same math and the same fragment routines, blocked: a CTA of 4 warps owns 64 query rows (forward, dQ) or 64 key
// rows (dK, dV) of one (batch, head) and walks the other dimension in blocks of 128 through shared memory.
//   forward   two passes over the key blocks: running row maximum / sum first, then probabilities (stored for the
//             backward, as for short sequences), dropout and O += P~ V.
//   dQ        two passes as well (the softmax gradient needs the whole row's sum of dP * P before any dS):
//             dP = dO V^T per key block, then dS, written to a [b, nh, S, S] workspace, and dQ += dS K.
//   dK, dV    per block of 64 keys, over query blocks: dS and P~ tiles staged in shared memory (P~ rebuilt from
//             the stored probabilities and the counter-based dropout mask), dK += dS^T Q, dV += P~^T dO.
constexpr int QB = 64;     // rows owned by a CTA
constexpr int KBLK = 128;  // rows of the other dimension per step
constexpr int PPK = QB + 8;

// rows first.. of a [*, ld] matrix (pointer already at this (batch, head)'s first column) -> [n_tile][RP] tile
template <typename T>
__device__ __forceinline__ void stage_block(T* dst, const T* __restrict__ src, size_t ld, const T* __restrict__ bias,
                                            int first, int n_tile, int S) {
  for (int i = threadIdx.x; i < n_tile * (HD / 8); i += blockDim.x) {
    const int s = i >> 3, d = (i & 7) * 8;
    float v[8];
    if (first + s < S) {
      load8(src + (size_t)(first + s) * ld + d, v);
      if (bias != nullptr) {
        float bb[8];
        load8(bias + d, bb);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += bb[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    store8(dst + s * RP + d, v);
  }
}

// two consecutive elements idx, idx + 1 of a [.., S] row; ok0 / ok1 say which exist; `pair` = 4-byte access allowed
template <typename T>
__device__ __forceinline__ float2 load_pair(const T* __restrict__ base, size_t idx, bool ok0, bool ok1, bool pair) {
  float2 r = make_float2(0.f, 0.f);
  if (ok0) {
    if (pair) r = Pack<T>::unpack(*reinterpret_cast<const uint32_t*>(base + idx));
    else { r.x = to_f(base[idx]); if (ok1) r.y = to_f(base[idx + 1]); }
  }
  return r;
}
template <typename T>
__device__ __forceinline__ void store_pair(T* __restrict__ base, size_t idx, uint32_t u, bool ok0, bool ok1, bool pair) {
  if (ok0) {
    if (pair) *reinterpret_cast<uint32_t*>(base + idx) = u;
    else {
      const T* e = reinterpret_cast<const T*>(&u);
      base[idx] = e[0];
      if (ok1) base[idx + 1] = e[1];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) attention_fwd_long_kernel(
    const T* __restrict__ qkv, const T* __restrict__ bqkv, const int* __restrict__ mask, T* __restrict__ ctx,
    T* __restrict__ probs, int S, int H, int nh, float p, const int* __restrict__ seed_ptr, uint32_t stream) {
  extern __shared__ __align__(128) uint8_t sm_raw[];
  T* sQ = reinterpret_cast<T*>(sm_raw);
  T* sK = sQ + QB * RP;
  T* sV = sK + KBLK * RP;
  uint8_t* sCode = reinterpret_cast<uint8_t*>(sV + KBLK * RP);   // per key of the block: 0 beyond S, 1 attend, 2 masked
  const int h = blockIdx.x, b = blockIdx.y, q0 = blockIdx.z * QB;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const float scale = rsqrtf((float)HD);
  const T* base = qkv + (size_t)b * S * 3 * H + h * HD;
  stage_block<T>(sQ, base, (size_t)3 * H, bqkv + h * HD, q0, QB, S);
  const int r0 = warp * 16;
  const int i0 = q0 + r0 + g, i1 = i0 + 8;
  const int nkb = (S + KBLK - 1) / KBLK;
  float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f;
  for (int kb = 0; kb < nkb; ++kb) {
    __syncthreads();
    stage_block<T>(sK, base + H, (size_t)3 * H, bqkv + H + h * HD, kb * KBLK, KBLK, S);
    for (int j = threadIdx.x; j < KBLK; j += blockDim.x) {
      const int key = kb * KBLK + j;
      sCode[j] = key < S ? (mask[b * S + key] != 0 ? 1 : 2) : 0;
    }
    __syncthreads();
    float acc[KBLK / 8][4];
#pragma unroll
    for (int j = 0; j < KBLK / 8; ++j) { acc[j][0] = 0.f; acc[j][1] = 0.f; acc[j][2] = 0.f; acc[j][3] = 0.f; }
    rows_times_transposed<T, KBLK>(acc, sQ, sK, r0, lane);
    float bm0 = -1e30f, bm1 = -1e30f;
#pragma unroll
    for (int j = 0; j < KBLK / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int code = sCode[8 * j + 2 * t + e];
        acc[j][e] = code == 1 ? acc[j][e] * scale : -1e30f;
        acc[j][2 + e] = code == 1 ? acc[j][2 + e] * scale : -1e30f;
        if (code != 0) { bm0 = fmaxf(bm0, acc[j][e]); bm1 = fmaxf(bm1, acc[j][2 + e]); }
      }
    }
    const float n0 = fmaxf(m0, quad_max(bm0)), n1 = fmaxf(m1, quad_max(bm1));
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < KBLK / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (sCode[8 * j + 2 * t + e] != 0) { s0 += __expf(acc[j][e] - n0); s1 += __expf(acc[j][2 + e] - n1); }
      }
    }
    l0 = l0 * __expf(m0 - n0) + s0;
    l1 = l1 * __expf(m1 - n1) + s1;
    m0 = n0; m1 = n1;
  }
  l0 = quad_sum(l0); l1 = quad_sum(l1);
  const float inv0 = i0 < S ? 1.f / l0 : 0.f, inv1 = i1 < S ? 1.f / l1 : 0.f;
  const size_t prow0 = ((size_t)(b * nh + h) * S + i0) * S, prow1 = ((size_t)(b * nh + h) * S + i1) * S;
  const bool pair = (S & 1) == 0;
  float out[HD / 8][4];
#pragma unroll
  for (int jd = 0; jd < HD / 8; ++jd) { out[jd][0] = 0.f; out[jd][1] = 0.f; out[jd][2] = 0.f; out[jd][3] = 0.f; }
  for (int kb = 0; kb < nkb; ++kb) {
    __syncthreads();
    stage_block<T>(sK, base + H, (size_t)3 * H, bqkv + H + h * HD, kb * KBLK, KBLK, S);
    stage_block<T>(sV, base + 2 * H, (size_t)3 * H, bqkv + 2 * H + h * HD, kb * KBLK, KBLK, S);
    for (int j = threadIdx.x; j < KBLK; j += blockDim.x) {
      const int key = kb * KBLK + j;
      sCode[j] = key < S ? (mask[b * S + key] != 0 ? 1 : 2) : 0;
    }
    __syncthreads();
    float acc[KBLK / 8][4];
#pragma unroll
    for (int j = 0; j < KBLK / 8; ++j) { acc[j][0] = 0.f; acc[j][1] = 0.f; acc[j][2] = 0.f; acc[j][3] = 0.f; }
    rows_times_transposed<T, KBLK>(acc, sQ, sK, r0, lane);
    uint32_t pf[KBLK / 16][4];
#pragma unroll
    for (int j = 0; j < KBLK / 8; ++j) {
      const int c = 8 * j + 2 * t, key = kb * KBLK + c;
      float e00, e01, e10, e11;
      {
        const int c0 = sCode[c], c1 = sCode[c + 1];
        e00 = c0 != 0 ? __expf((c0 == 1 ? acc[j][0] * scale : -1e30f) - m0) * inv0 : 0.f;
        e01 = c1 != 0 ? __expf((c1 == 1 ? acc[j][1] * scale : -1e30f) - m0) * inv0 : 0.f;
        e10 = c0 != 0 ? __expf((c0 == 1 ? acc[j][2] * scale : -1e30f) - m1) * inv1 : 0.f;
        e11 = c1 != 0 ? __expf((c1 == 1 ? acc[j][3] * scale : -1e30f) - m1) * inv1 : 0.f;
      }
      const uint32_t u0 = Pack<T>::pack(e00, e01), u1 = Pack<T>::pack(e10, e11);
      store_pair<T>(probs, prow0 + key, u0, i0 < S && key < S, key + 1 < S, pair);
      store_pair<T>(probs, prow1 + key, u1, i1 < S && key < S, key + 1 < S, pair);
      float2 q0v = Pack<T>::unpack(u0), q1v = Pack<T>::unpack(u1);
      if (p > 0.f) {
        q0v.x = keep(seed, stream, (uint32_t)(prow0 + key), p) ? q0v.x * inv_keep : 0.f;
        q0v.y = keep(seed, stream, (uint32_t)(prow0 + key + 1), p) ? q0v.y * inv_keep : 0.f;
        q1v.x = keep(seed, stream, (uint32_t)(prow1 + key), p) ? q1v.x * inv_keep : 0.f;
        q1v.y = keep(seed, stream, (uint32_t)(prow1 + key + 1), p) ? q1v.y * inv_keep : 0.f;
      }
      pf[j >> 1][(j & 1) * 2 + 0] = Pack<T>::pack(q0v.x, q0v.y);
      pf[j >> 1][(j & 1) * 2 + 1] = Pack<T>::pack(q1v.x, q1v.y);
    }
    frag_times_rows<T, KBLK>(out, pf, sV, lane);
  }
  write_rows<T>(out, ctx + (size_t)(b * S + q0 + r0) * H + h * HD, H, q0 + r0, S, lane, nullptr);
}

template <typename T>
__global__ void __launch_bounds__(128) attention_bwd_long_dq_kernel(
    const T* __restrict__ dctx, const T* __restrict__ qkv, const T* __restrict__ bqkv, const T* __restrict__ probs,
    T* __restrict__ ds_ws, T* __restrict__ dqkv, int S, int H, int nh, float p, const int* __restrict__ seed_ptr,
    uint32_t stream, float* __restrict__ bias_acc) {
  extern __shared__ __align__(128) uint8_t sm_raw[];
  T* sDO = reinterpret_cast<T*>(sm_raw);
  T* sK = sDO + QB * RP;
  T* sV = sK + KBLK * RP;
  float* sBias = reinterpret_cast<float*>(sV + KBLK * RP);   // [HD] column sums of this CTA's dQ rows
  const int h = blockIdx.x, b = blockIdx.y, q0 = blockIdx.z * QB;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const float scale = rsqrtf((float)HD);
  const T* base = qkv + (size_t)b * S * 3 * H + h * HD;
  if (bias_acc != nullptr)
    for (int i = threadIdx.x; i < HD; i += blockDim.x) sBias[i] = 0.f;
  stage_block<T>(sDO, dctx + (size_t)b * S * H + h * HD, (size_t)H, nullptr, q0, QB, S);
  const int r0 = warp * 16;
  const int i0 = q0 + r0 + g, i1 = i0 + 8;
  const int nkb = (S + KBLK - 1) / KBLK;
  const size_t prow0 = ((size_t)(b * nh + h) * S + i0) * S, prow1 = ((size_t)(b * nh + h) * S + i1) * S;
  const bool pair = (S & 1) == 0;
  float dot0 = 0.f, dot1 = 0.f;
  float out[HD / 8][4];
#pragma unroll
  for (int jd = 0; jd < HD / 8; ++jd) { out[jd][0] = 0.f; out[jd][1] = 0.f; out[jd][2] = 0.f; out[jd][3] = 0.f; }
  for (int pass = 0; pass < 2; ++pass) {
    for (int kb = 0; kb < nkb; ++kb) {
      __syncthreads();
      stage_block<T>(sV, base + 2 * H, (size_t)3 * H, bqkv + 2 * H + h * HD, kb * KBLK, KBLK, S);
      if (pass == 1) stage_block<T>(sK, base + H, (size_t)3 * H, bqkv + H + h * HD, kb * KBLK, KBLK, S);
      __syncthreads();
      float acc[KBLK / 8][4];
#pragma unroll
      for (int j = 0; j < KBLK / 8; ++j) { acc[j][0] = 0.f; acc[j][1] = 0.f; acc[j][2] = 0.f; acc[j][3] = 0.f; }
      rows_times_transposed<T, KBLK>(acc, sDO, sV, r0, lane);
      uint32_t dsf[KBLK / 16][4];
#pragma unroll
      for (int j = 0; j < KBLK / 8; ++j) {
        const int key = kb * KBLK + 8 * j + 2 * t;
        const bool k0 = key < S, k1 = key + 1 < S;
        const float2 pr0 = load_pair<T>(probs, prow0 + key, i0 < S && k0, k1, pair);
        const float2 pr1 = load_pair<T>(probs, prow1 + key, i1 < S && k0, k1, pair);
        float m00 = 1.f, m01 = 1.f, m10 = 1.f, m11 = 1.f;
        if (p > 0.f) {
          m00 = keep(seed, stream, (uint32_t)(prow0 + key), p) ? inv_keep : 0.f;
          m01 = keep(seed, stream, (uint32_t)(prow0 + key + 1), p) ? inv_keep : 0.f;
          m10 = keep(seed, stream, (uint32_t)(prow1 + key), p) ? inv_keep : 0.f;
          m11 = keep(seed, stream, (uint32_t)(prow1 + key + 1), p) ? inv_keep : 0.f;
        }
        const float a00 = acc[j][0] * m00, a01 = acc[j][1] * m01, a10 = acc[j][2] * m10, a11 = acc[j][3] * m11;
        if (pass == 0) {
          dot0 += a00 * pr0.x + a01 * pr0.y;
          dot1 += a10 * pr1.x + a11 * pr1.y;
        } else {
          const uint32_t d0 = Pack<T>::pack(pr0.x * (a00 - dot0) * scale, pr0.y * (a01 - dot0) * scale);
          const uint32_t d1 = Pack<T>::pack(pr1.x * (a10 - dot1) * scale, pr1.y * (a11 - dot1) * scale);
          store_pair<T>(ds_ws, prow0 + key, d0, i0 < S && k0, k1, pair);
          store_pair<T>(ds_ws, prow1 + key, d1, i1 < S && k0, k1, pair);
          dsf[j >> 1][(j & 1) * 2 + 0] = d0;
          dsf[j >> 1][(j & 1) * 2 + 1] = d1;
        }
      }
      if (pass == 1) frag_times_rows<T, KBLK>(out, dsf, sK, lane);
    }
    if (pass == 0) { dot0 = quad_sum(dot0); dot1 = quad_sum(dot1); }
  }
  write_rows<T>(out, dqkv + (size_t)(b * S + q0 + r0) * 3 * H + h * HD, 3 * H, q0 + r0, S, lane,
                bias_acc != nullptr ? sBias : nullptr);
  if (bias_acc != nullptr) {
    __syncthreads();
    const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    float* my_acc = bias_acc + (size_t)(cta % 8) * 3 * H;
    for (int i = threadIdx.x; i < HD; i += blockDim.x) atomicAdd(my_acc + h * HD + i, sBias[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(128) attention_bwd_long_dkv_kernel(
    const T* __restrict__ dctx, const T* __restrict__ qkv, const T* __restrict__ bqkv, const T* __restrict__ probs,
    const T* __restrict__ ds_ws, T* __restrict__ dqkv, int S, int H, int nh, float p, const int* __restrict__ seed_ptr,
    uint32_t stream, float* __restrict__ bias_acc) {
  extern __shared__ __align__(128) uint8_t sm_raw[];
  T* sDS = reinterpret_cast<T*>(sm_raw);      // [query of the block][key of this CTA]
  T* sW = sDS + KBLK * PPK;
  T* sQ = sW + KBLK * PPK;
  T* sDO = sQ + KBLK * RP;
  float* sBias = reinterpret_cast<float*>(sDO + KBLK * RP);   // [2][HD] column sums of this CTA's dK, dV rows
  const int h = blockIdx.x, b = blockIdx.y, key0 = blockIdx.z * QB;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const T* base = qkv + (size_t)b * S * 3 * H + h * HD;
  if (bias_acc != nullptr)
    for (int i = threadIdx.x; i < 2 * HD; i += blockDim.x) sBias[i] = 0.f;
  const bool vec = (S & 7) == 0;     // then every 8-key segment starts 16-byte aligned and lies inside the row
  const int nqb = (S + KBLK - 1) / KBLK;
  float outK[HD / 8][4], outV[HD / 8][4];
#pragma unroll
  for (int jd = 0; jd < HD / 8; ++jd) {
    outK[jd][0] = 0.f; outK[jd][1] = 0.f; outK[jd][2] = 0.f; outK[jd][3] = 0.f;
    outV[jd][0] = 0.f; outV[jd][1] = 0.f; outV[jd][2] = 0.f; outV[jd][3] = 0.f;
  }
  for (int qb = 0; qb < nqb; ++qb) {
    __syncthreads();
    stage_block<T>(sQ, base, (size_t)3 * H, bqkv + h * HD, qb * KBLK, KBLK, S);
    stage_block<T>(sDO, dctx + (size_t)b * S * H + h * HD, (size_t)H, nullptr, qb * KBLK, KBLK, S);
    for (int i = threadIdx.x; i < KBLK * (QB / 8); i += blockDim.x) {
      const int qr = i >> 3, kc = (i & 7) * 8;
      const int q = qb * KBLK + qr, key = key0 + kc;
      float dsv[8], wv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { dsv[j] = 0.f; wv[j] = 0.f; }
      if (q < S && key < S) {
        const size_t idx = ((size_t)(b * nh + h) * S + q) * S + key;
        if (vec) {
          load8(ds_ws + idx, dsv);
          load8(probs + idx, wv);
        } else {
          for (int j = 0; j < 8; ++j)
            if (key + j < S) { dsv[j] = to_f(ds_ws[idx + j]); wv[j] = to_f(probs[idx + j]); }
        }
        if (p > 0.f) {
#pragma unroll
          for (int j = 0; j < 8; ++j) wv[j] = keep(seed, stream, (uint32_t)(idx + j), p) ? wv[j] * inv_keep : 0.f;
        }
      }
      store8(sDS + qr * PPK + kc, dsv);
      store8(sW + qr * PPK + kc, wv);
    }
    __syncthreads();
    transposed_times_rows<T, KBLK>(outK, sDS, PPK, warp * 16, sQ, lane);
    transposed_times_rows<T, KBLK>(outV, sW, PPK, warp * 16, sDO, lane);
  }
  const int k0 = key0 + warp * 16;
  write_rows<T>(outK, dqkv + (size_t)(b * S + k0) * 3 * H + H + h * HD, 3 * H, k0, S, lane,
                bias_acc != nullptr ? sBias : nullptr);
  write_rows<T>(outV, dqkv + (size_t)(b * S + k0) * 3 * H + 2 * H + h * HD, 3 * H, k0, S, lane,
                bias_acc != nullptr ? sBias + HD : nullptr);
  if (bias_acc != nullptr) {
    __syncthreads();
    const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    float* my_acc = bias_acc + (size_t)(cta % 8) * 3 * H;
    for (int i = threadIdx.x; i < 2 * HD; i += blockDim.x)
      atomicAdd(my_acc + (1 + i / HD) * H + h * HD + (i % HD), sBias[i]);
  }
}

constexpr size_t fwd_long_smem(size_t esz) { return (size_t)(QB + 2 * KBLK) * RP * esz + KBLK; }
constexpr size_t dq_long_smem(size_t esz) { return (size_t)(QB + 2 * KBLK) * RP * esz + HD * sizeof(float); }
constexpr size_t dkv_long_smem(size_t esz) {
  return (size_t)2 * KBLK * PPK * esz + (size_t)2 * KBLK * RP * esz + 2 * HD * sizeof(float);
}

template <typename T>
static int launch_fwd_long(const void* qkv, const void* bqkv, const int* mask, void* ctx, void* probs, int b, int S, int H,
                           int nh, float p, const int* seed, unsigned stream_id, cudaStream_t st) {
  auto k = attention_fwd_long_kernel<T>;
  constexpr size_t smem = fwd_long_smem(sizeof(T));
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
  k<<<dim3(nh, b, (S + QB - 1) / QB), 128, smem, st>>>((const T*)qkv, (const T*)bqkv, mask, (T*)ctx, (T*)probs, S, H, nh, p,
                                                        seed, stream_id);
  return 0;
}

template <typename T>
static int launch_bwd_long(const void* dctx, const void* qkv, const void* bqkv, const void* probs, void* ds_ws, void* dqkv,
                           int b, int S, int H, int nh, float p, const int* seed, unsigned stream_id, float* bias_acc,
                           cudaStream_t st) {
  auto kq = attention_bwd_long_dq_kernel<T>;
  auto kkv = attention_bwd_long_dkv_kernel<T>;
  constexpr size_t sq = dq_long_smem(sizeof(T)), skv = dkv_long_smem(sizeof(T));
  if (cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sq) != cudaSuccess) return -5;
  if (cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)skv) != cudaSuccess) return -5;
  const dim3 grid(nh, b, (S + QB - 1) / QB);
  kq<<<grid, 128, sq, st>>>((const T*)dctx, (const T*)qkv, (const T*)bqkv, (const T*)probs, (T*)ds_ws, (T*)dqkv, S, H, nh, p,
                            seed, stream_id, bias_acc);
  kkv<<<grid, 128, skv, st>>>((const T*)dctx, (const T*)qkv, (const T*)bqkv, (const T*)probs, (const T*)ds_ws, (T*)dqkv, S,
                              H, nh, p, seed, stream_id, bias_acc);
  return 0;
}

}  // namespace amma
}  // namespace rb

using namespace rb;

// dtype: 1 = bf16, 2 = fp16.  Requires H / nh == 64, 1 <= S <= 128, H % 8 == 0; returns -4 otherwise (callers
// then use the attention_tc.cu entry points, which also cover head dim 32).
RB_API int rb_attention_fwd_mma(int dtype, const void* qkv, const void* bqkv, const int* mask, void* ctx, void* probs,
                                int b, int S, int H, int nh, float p, const int* seed, unsigned stream_id,
                                cudaStream_t st) {
  if (S > 128 || S < 1 || H % nh || H % 8 || H / nh != amma::HD || (dtype != RB_BF16 && dtype != RB_F16)) return -4;
  int rc;
#define RB_FWD(T, SP) amma::launch_fwd<T, SP>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st)
  if (dtype == RB_BF16) rc = S <= 32 ? RB_FWD(__nv_bfloat16, 32) : S <= 64 ? RB_FWD(__nv_bfloat16, 64) : RB_FWD(__nv_bfloat16, 128);
  else rc = S <= 32 ? RB_FWD(__half, 32) : S <= 64 ? RB_FWD(__half, 64) : RB_FWD(__half, 128);
#undef RB_FWD
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

// bias_acc (nullable): 8 replicas x [3H] fp32; when given, the column sums of dqkv (the q/k/v bias gradients) are
// accumulated there so that no separate pass over dqkv is needed.
RB_API int rb_attention_bwd_mma(int dtype, const void* dctx, const void* qkv, const void* bqkv, const void* probs,
                                void* dqkv, int b, int S, int H, int nh, float p, const int* seed, unsigned stream_id,
                                float* bias_acc, cudaStream_t st) {
  if (S > 128 || S < 1 || H % nh || H % 8 || H / nh != amma::HD || (dtype != RB_BF16 && dtype != RB_F16)) return -4;
  int rc;
#define RB_BWD(T, SP) amma::launch_bwd<T, SP>(dctx, qkv, bqkv, probs, dqkv, b, S, H, nh, p, seed, stream_id, bias_acc, st)
  if (dtype == RB_BF16) rc = S <= 32 ? RB_BWD(__nv_bfloat16, 32) : S <= 64 ? RB_BWD(__nv_bfloat16, 64) : RB_BWD(__nv_bfloat16, 128);
  else rc = S <= 32 ? RB_BWD(__half, 32) : S <= 64 ? RB_BWD(__half, 64) : RB_BWD(__half, 128);
#undef RB_BWD
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

// Sequences of 129..512 tokens (same requirements otherwise).  The backward needs ds_ws, a [b, nh, S, S] scratch of
// the activation dtype (the softmax gradient, written by its first kernel and read by its second); two launches.
static bool long_args_ok(int dtype, int b, int S, int H, int nh) {
  if (S <= 128 || S > 512 || H % nh || H % 8 || H / nh != amma::HD || (dtype != RB_BF16 && dtype != RB_F16)) return false;
  return (long long)b * nh * S * S < (1LL << 32);   // dropout counters are 32-bit element indices
}

RB_API int rb_attention_fwd_long(int dtype, const void* qkv, const void* bqkv, const int* mask, void* ctx, void* probs,
                                 int b, int S, int H, int nh, float p, const int* seed, unsigned stream_id,
                                 cudaStream_t st) {
  if (!long_args_ok(dtype, b, S, H, nh)) return -4;
  const int rc = dtype == RB_BF16
                     ? amma::launch_fwd_long<__nv_bfloat16>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st)
                     : amma::launch_fwd_long<__half>(qkv, bqkv, mask, ctx, probs, b, S, H, nh, p, seed, stream_id, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_attention_bwd_long(int dtype, const void* dctx, const void* qkv, const void* bqkv, const void* probs,
                                 void* ds_ws, void* dqkv, int b, int S, int H, int nh, float p, const int* seed,
                                 unsigned stream_id, float* bias_acc, cudaStream_t st) {
  if (!long_args_ok(dtype, b, S, H, nh) || ds_ws == nullptr) return -4;
  const int rc = dtype == RB_BF16
                     ? amma::launch_bwd_long<__nv_bfloat16>(dctx, qkv, bqkv, probs, ds_ws, dqkv, b, S, H, nh, p, seed,
                                                            stream_id, bias_acc, st)
                     : amma::launch_bwd_long<__half>(dctx, qkv, bqkv, probs, ds_ws, dqkv, b, S, H, nh, p, seed, stream_id,
                                                     bias_acc, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}
